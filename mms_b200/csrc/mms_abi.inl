// mms_abi.inl — host side of the C ABI (included at the end of mms_sim.cu).
namespace mms {

thread_local char g_last_error[256] = "";

static int cuda_fail(cudaError_t e, const char *what)
{
    snprintf(g_last_error, sizeof(g_last_error), "%s: %s", what, cudaGetErrorString(e));
    return MMS_ERR_CUDA;
}

#define MMS_CUDA(call)                                             \
    do {                                                           \
        cudaError_t e_ = (call);                                   \
        if (e_ != cudaSuccess) return mms::cuda_fail(e_, #call);   \
    } while (0)

// numpy's pairwise split of n elements starting at `base`.
static void plan_rec(int64_t base, int64_t n, int32_t *leaf_start, uint8_t *merges, int32_t &count)
{
    if (n <= 128) {
        if (leaf_start) { leaf_start[count] = (int32_t)base; merges[count] = 0; }
        ++count;
        return;
    }
    int64_t half = n / 2;
    half -= half % 8;
    plan_rec(base, half, leaf_start, merges, count);
    plan_rec(base + half, n - half, leaf_start, merges, count);
    if (merges) merges[count - 1] += 1;
}

static int32_t plan_leaves(int64_t n)
{
    if (n <= 0) return 0;
    int32_t count = 0;
    plan_rec(0, n, nullptr, nullptr, count);
    return count;
}

struct Geometry {
    int32_t K, NS, seg_len, seg_per_chunk, warmup, lat_smem_elems, rounds, repair_cap,
        block_warps, narrow_limit, lat_f64;
    size_t smem_stream, smem_repair;
    size_t off_leaf, off_seg_end, off_chunk_start, off_decisions, off_work_count, off_work_items,
        off_repair_from, off_rows, off_seg_src, off_compat, off_seg_leaf, off_group_info,
        off_own_rewritten;
    size_t smem_count;        // shared memory of count_kernel
    size_t total;
};

static size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

// Chunking, shared-memory and scratch geometry of one call.
static int plan_call(int64_t N, const mms_placements *c, const mms_sim_options *opts,
                     uint32_t flags, bool group_good, Geometry *g)
{
    if (!c || N < 0 || c->num_candidates < 0 || c->num_models < 0 || c->max_groups < 0 ||
        c->max_placed < 0 || c->max_slots < 0 || c->max_stages < 1 || c->num_columns < 0)
        return MMS_ERR_ARG;
    if (N > 0x7FFFFFFF) return MMS_ERR_UNSUPPORTED;
    if (c->max_groups > MMS_MAX_GROUPS || c->max_slots > MMS_MAX_SLOTS ||
        c->max_placed > MMS_MAX_PLACED || c->max_stages > MMS_MAX_STAGES ||
        c->num_columns > MMS_MAX_COLUMNS)
        return MMS_ERR_UNSUPPORTED;
    if ((flags & MMS_FLAG_LEGACY_CLOCK) && c->max_stages != 2) return MMS_ERR_ARG;
    if (c->num_scored < 0 || c->num_scored > c->num_candidates) return MMS_ERR_ARG;
    const bool mirrors = c->num_scored != 0 && c->num_scored != c->num_candidates;
    // per-request outputs come from one run per candidate; mirrors need the partner list
    if (mirrors && ((flags & MMS_FLAG_PER_REQUEST) || !c->partner || !c->mirror_swap))
        return MMS_ERR_ARG;

    const int64_t B = c->num_candidates;
    // blocks that fit an SM at once, from the kernel's shared-memory use
    const size_t lat_elems0 = (size_t)c->num_models * c->num_columns * c->max_stages + 8;
    const int lat_on_chip0 = (c->latency_stride == 0 && lat_elems0 * sizeof(float) <= (size_t)kLatSmemBytes)
                                 ? (int)lat_elems0 : 0;
    const SmemLayout L0 = smem_layout(c->num_models, c->max_groups, c->max_placed, c->max_slots,
                                      c->max_stages, group_good, lat_on_chip0);
    int sm_count = 148, dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
        (void)cudaGetLastError();
        sm_count = 148;
    }
    // Warps per block: blocks share the latency table among their warps, so the
    // size that fits the most warps on an SM (233472 bytes, 1024 reserved per
    // block; 232448 at most in one block) wins, the smaller one on a tie.
    int64_t per_sm = 1;
    int block_warps = 1;
    auto fit = [&](const SmemLayout &L, int64_t &best_per_sm, int &best_w) {
        best_per_sm = 1;
        best_w = 1;
        for (int w = 1; w <= kMaxBlockWarps; ++w) {
            const size_t bytes = L.warp0 + (size_t)w * L.warp_bytes;
            if (bytes > 232448) break;
            int64_t warps = (int64_t)(233472 / (bytes + 1024)) * w;
            if (warps > kMaxWarpsPerSm) warps = kMaxWarpsPerSm;
            if (warps >= best_per_sm) { best_per_sm = warps; best_w = w; }
        }
    };
    fit(L0, per_sm, block_warps);
    // The table goes on chip as doubles (no conversion per use) when that costs
    // no resident warp.
    g->lat_f64 = 0;
    if (lat_on_chip0) {
        const SmemLayout L64 = smem_layout(c->num_models, c->max_groups, c->max_placed,
                                           c->max_slots, c->max_stages, group_good, lat_on_chip0,
                                           true);
        int64_t per_sm64;
        int block_warps64;
        fit(L64, per_sm64, block_warps64);
        if (per_sm64 >= per_sm) { g->lat_f64 = 1; block_warps = block_warps64; }
    }
    const int64_t resident_slots = (int64_t)sm_count * per_sm;
    int64_t chunk = opts ? opts->chunk_requests : 0;
    int64_t warm = opts ? opts->warmup_requests : 0;
    // segments: the unit of state snapshots and repairs
    const int64_t seg = 1024;
    const int64_t NS = N / seg > 0 ? N / seg : 1;
    int64_t spc;                                   // segments per chunk
    if (chunk < 0 || N < 8192 || B == 0) {
        spc = NS;
    } else if (chunk > 0) {
        spc = (chunk + seg / 2) / seg;
    } else {
        // Chunks are the units of parallel work: as many as fill nine tenths
        // of ONE wave of the resident warps (SMs x warps per SM at this
        // kernel's shared-memory use; a second wave would pay the run-in
        // twice), but never chunks shorter than 3 segments.  More chunks mean
        // more boundaries to validate and repair.  The chunk length is that
        // ideal rounded to the nearest number of segments, or the next longer
        // one when the chunks would not fit the wave any more.
        const int64_t lanes = resident_slots * kLanes;
        spc = B > 0 ? (20 * NS * B + 9 * lanes) / (18 * lanes) : NS;      // round(NS / K_ideal)
        if (spc < 3) spc = 3;
        if (spc > NS) spc = NS;
        if (B > 0 && ((NS + spc - 1) / spc) * B > lanes) spc += 1;
    }
    if (spc < 1) spc = 1;
    if (spc > NS) spc = NS;
    const int64_t K = (NS + spc - 1) / spc;
    if (K * (B > 0 ? B : 1) >= 0x7FFFFFFFLL) return MMS_ERR_UNSUPPORTED;   // work-list encoding
    // A launch that fills less than half of the GPU goes out in smaller
    // blocks, one per SM: a warp that shares its SM with two others runs
    // faster than one that shares it with eleven while most SMs stand idle.
    // (A nearly full launch keeps the large blocks: the SMs they leave free
    // serve the small kernels of a launch running beside it.)
    const int64_t total_warps = ((B + kLanes - 1) / kLanes) * K;
    if (2 * total_warps <= (int64_t)sm_count * block_warps) {
        block_warps = (int)((total_warps + sm_count - 1) / sm_count);
        if (block_warps < 1) block_warps = 1;
    }
    g->block_warps = block_warps;
    if (warm <= 0) warm = 2048;
    int rounds = opts ? opts->repair_rounds : 0;
    if (rounds <= 0) rounds = kDefaultRepairRounds;
    if (rounds > kMaxRepairRounds) rounds = kMaxRepairRounds;
    int cap = opts ? opts->repair_segments : 0;
    if (cap == 0) cap = kDefaultRepairSegments;
    if (cap < 0) cap = 0;
    g->rounds = rounds; g->repair_cap = cap;
    g->K = (int32_t)K; g->NS = (int32_t)NS; g->seg_len = (int32_t)seg;
    g->seg_per_chunk = (int32_t)spc; g->warmup = (int32_t)warm;

    // the shared table goes on chip (f32), with 8 readable entries of padding
    const size_t lat_elems = (size_t)c->num_models * c->num_columns * c->max_stages + 8;
    g->lat_smem_elems = (c->latency_stride == 0 && lat_elems * sizeof(float) <= (size_t)kLatSmemBytes)
                            ? (int32_t)lat_elems : 0;
    const SmemLayout L = smem_layout(c->num_models, c->max_groups, c->max_placed, c->max_slots,
                                     c->max_stages, group_good, g->lat_smem_elems,
                                     g->lat_smem_elems != 0 && g->lat_f64 != 0);
    g->smem_stream = L.warp0 + (size_t)g->block_warps * L.warp_bytes;
    // ... the repair scratch, then the decoded-request records of the step that decodes ahead
    g->smem_repair = staging_offset(L.total, c->max_slots, c->max_groups) + kStagedBytes;
    if (g->smem_repair > 227 * 1024) return MMS_ERR_UNSUPPORTED;
    // the tally's per-lane histograms (count_kernel)
    g->smem_count = sizeof(uint32_t) * (size_t)(c->max_groups + (c->num_models + 1) / 2) * kLanes;
    if (g->smem_count > 227 * 1024) return MMS_ERR_UNSUPPORTED;
    // one-chunk-per-warp repairs: as many as are resident at once (12 warps of
    // this register use per SM, or what shared memory admits)
    int64_t narrow_per_sm = 233472 / (int64_t)(g->smem_repair + 1024);
    if (narrow_per_sm > 12) narrow_per_sm = 12;
    g->narrow_limit = (int32_t)(narrow_per_sm * sm_count);
    // beside a launch that holds most SMs for itself, what is left over takes few blocks
    if ((flags & MMS_FLAG_CROWDED) && g->narrow_limit > 48) g->narrow_limit = 48;

    size_t off = 0;
    g->off_rows = off;        off += align256(2 * sizeof(uint32_t) * kRowWords * (size_t)((B + kLanes - 1) / kLanes * kLanes) *
                                               (c->num_models + 1) + 256);
    g->off_leaf = off;        off += align256(sizeof(double) * (size_t)plan_leaves(N) * B);
    g->off_decisions = off;   off += align256((c->max_groups > 126 ? 2 : 1) * (size_t)((N + 3) / 4 * 4 + 4) *
                                               (size_t)((B + 31) / 32 * 32));
    g->off_work_count = off;  off += align256(sizeof(uint32_t) * (kMaxRepairRounds + 1));
    g->off_repair_from = off; off += align256(sizeof(int32_t) * (size_t)K * B);
    g->off_work_items = off;  off += align256(sizeof(uint32_t) * (size_t)K * B);
    g->off_seg_src = off;     off += align256(sizeof(int32_t) * (size_t)NS * B);
    g->off_compat = off;      off += align256(sizeof(uint16_t) * (size_t)K * B);
    g->off_seg_leaf = off;    off += align256(sizeof(int32_t) * (size_t)(NS + 1));
    g->off_group_info = off;  off += align256(sizeof(uint32_t) * (size_t)B * c->max_groups + 4);
    g->off_own_rewritten = off; off += align256((size_t)K * B + 4);
    g->off_seg_end = off;     off += K > 1 ? align256(sizeof(double) * (size_t)NS * c->max_slots * B) : 0;
    g->off_chunk_start = off; off += K > 1 ? align256(sizeof(double) * (size_t)K * c->max_slots * B) : 0;
    g->total = off;
    return MMS_OK;
}

// Events around the dominant kernels, see mms_profile_begin().
constexpr int kProfileSlots = 2048;
static cudaEvent_t g_prof_ev[2 * kProfileSlots];
static int32_t g_prof_tag[kProfileSlots];
static int g_prof_created = 0;      // events exist
static int g_prof_on = 0;
static int g_prof_count = 0;

// Brackets what is enqueued between its construction and stop() with two events.
struct ProfileSpan {
    int slot;
    cudaStream_t st;
    ProfileSpan(int32_t tag, cudaStream_t s) : slot(-1), st(s)
    {
        if (g_prof_on && g_prof_count < kProfileSlots) {
            slot = g_prof_count++;
            g_prof_tag[slot] = tag;
            (void)cudaEventRecord(g_prof_ev[2 * slot], st);
        }
    }
    void stop()
    {
        if (slot >= 0) (void)cudaEventRecord(g_prof_ev[2 * slot + 1], st);
        slot = -1;
    }
};

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) is sticky per function and
// device and not cheap; it is issued only when a call needs more than any
// earlier one asked for.
struct SmemGrant { const void *func; int device; size_t bytes; };
constexpr int kMaxGrants = 128;
static SmemGrant g_grants[kMaxGrants];
static int g_num_grants = 0;
static std::mutex g_grant_mutex;

static int allow_smem(const void *func, size_t bytes)
{
    int dev = 0;
    MMS_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(g_grant_mutex);
    SmemGrant *slot = nullptr;
    for (int i = 0; i < g_num_grants; ++i)
        if (g_grants[i].func == func && g_grants[i].device == dev) { slot = &g_grants[i]; break; }
    if (slot && slot->bytes >= bytes) return MMS_OK;
    MMS_CUDA(cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    if (!slot && g_num_grants < kMaxGrants) slot = &g_grants[g_num_grants++];
    if (slot) { slot->func = func; slot->device = dev; slot->bytes = bytes; }
    return MMS_OK;
}

#define MMS_TRY(call)                  \
    do {                               \
        const int rc_ = (call);        \
        if (rc_ != MMS_OK) return rc_; \
    } while (0)

template <bool kFull, bool kGroupGood, bool kLegacy>
static int launch_sim(KernelArgs &ka, const ClearArgs &ca, const Geometry &g, cudaStream_t st)
{
    // everything a call clears, then the tables its kernels read: two launches
    {
        int64_t cells = (int64_t)ka.NS * ka.B;
        if ((int64_t)ka.B * (ka.M + 1) > cells) cells = (int64_t)ka.B * (ka.M + 1);
        int64_t blocks = (cells + 255) / 256;
        if (blocks > 148 * 8) blocks = 148 * 8;
        if (blocks < 1) blocks = 1;
        clear_kernel<<<(unsigned)blocks, 256, 0, st>>>(ka, ca);
        MMS_CUDA(cudaGetLastError());
        build_tables_kernel<<<(unsigned)blocks, 256, 0, st>>>(ka, ca);
        MMS_CUDA(cudaGetLastError());
    }
    auto stream_k = sim_stream_kernel<kFull, kGroupGood, kLegacy>;
    MMS_TRY(allow_smem((const void *)stream_k, g.smem_stream));
    const int64_t per_block = (int64_t)kLanes * g.block_warps;
    const int64_t streams = (int64_t)ka.B * ka.K;
    ProfileSpan stream_span(MMS_PROFILE_STREAM, st);
    stream_k<<<(unsigned)((streams + per_block - 1) / per_block), (unsigned)per_block,
               g.smem_stream, st>>>(ka);
    MMS_CUDA(cudaGetLastError());
    stream_span.stop();
    if (ka.K > 1) {
        auto repair_k = sim_repair_kernel<kFull, kGroupGood, kLegacy, false>;
        auto chain_k = sim_chain_kernel<kFull, kGroupGood, kLegacy, false>;
        auto repair_narrow_k = sim_repair_kernel<kFull, kGroupGood, kLegacy, true>;
        auto chain_narrow_k = sim_chain_kernel<kFull, kGroupGood, kLegacy, true>;
        MMS_TRY(allow_smem((const void *)repair_k, g.smem_repair));
        MMS_TRY(allow_smem((const void *)chain_k, g.smem_repair));
        MMS_TRY(allow_smem((const void *)repair_narrow_k, g.smem_repair));
        MMS_TRY(allow_smem((const void *)chain_narrow_k, g.smem_repair));
        const int64_t bounds = (int64_t)ka.B * (ka.K - 1);
        for (int r = 0; r < g.rounds; ++r) {
            ka.round = r;
            validate_kernel<<<(unsigned)((bounds + 127) / 128), 128, 0, st>>>(ka);
            MMS_CUDA(cudaGetLastError());
            resolve_kernel<<<(unsigned)((ka.Bs + 3) / 4), 4 * kLanes, 0, st>>>(ka);
            MMS_CUDA(cudaGetLastError());
            // sized for the worst case; blocks past the work list return at once
            repair_k<<<(unsigned)((bounds + kLanes - 1) / kLanes), kLanes, g.smem_repair, st>>>(ka);
            MMS_CUDA(cudaGetLastError());
            // the same list one chunk to a warp, when it is short (see sim_repair_kernel)
            const int64_t narrow = bounds < ka.narrow_limit ? bounds : ka.narrow_limit;
            if (narrow > 0) {
                repair_narrow_k<<<(unsigned)narrow, kLanes, g.smem_repair, st>>>(ka);
                MMS_CUDA(cudaGetLastError());
            }
        }
        ProfileSpan chain_span(MMS_PROFILE_CHAIN, st);
        chain_k<<<(unsigned)((ka.Bs + kLanes - 1) / kLanes), kLanes, g.smem_repair, st>>>(ka);
        MMS_CUDA(cudaGetLastError());
        chain_narrow_k<<<(unsigned)ka.Bs, kLanes, g.smem_repair, st>>>(ka);
        MMS_CUDA(cudaGetLastError());
        chain_span.stop();
    }
    return MMS_OK;
}

}  // namespace mms

extern "C" {

int mms_abi_version(void) { return 9; }

const char *mms_last_error(void) { return mms::g_last_error; }

int mms_profile_begin(void)
{
    using namespace mms;
    if (!g_prof_created) {
        for (int i = 0; i < 2 * kProfileSlots; ++i) MMS_CUDA(cudaEventCreate(&g_prof_ev[i]));
        g_prof_created = 1;
    }
    g_prof_count = 0;
    g_prof_on = 1;
    return MMS_OK;
}

int mms_profile_end(int32_t *launches, float *each_ms, int32_t *each_tag, int32_t capacity)
{
    using namespace mms;
    g_prof_on = 0;
    for (int i = 0; i < g_prof_count; ++i) {
        float ms = 0.0f;
        MMS_CUDA(cudaEventSynchronize(g_prof_ev[2 * i + 1]));
        MMS_CUDA(cudaEventElapsedTime(&ms, g_prof_ev[2 * i], g_prof_ev[2 * i + 1]));
        if (each_ms && i < capacity) each_ms[i] = ms;
        if (each_tag && i < capacity) each_tag[i] = g_prof_tag[i];
    }
    if (launches) *launches = g_prof_count;
    g_prof_count = 0;
    return MMS_OK;
}

int32_t mms_sum_plan_leaves(int64_t num_requests)
{
    if (num_requests > 0x7FFFFFFF) return MMS_ERR_UNSUPPORTED;
    return mms::plan_leaves(num_requests);
}

int mms_sum_plan_fill(int64_t num_requests, int32_t *leaf_start, uint8_t *leaf_merges)
{
    if (num_requests < 0 || !leaf_start || !leaf_merges) return MMS_ERR_ARG;
    if (num_requests > 0x7FFFFFFF) return MMS_ERR_UNSUPPORTED;
    int32_t count = 0;
    if (num_requests > 0) mms::plan_rec(0, num_requests, leaf_start, leaf_merges, count);
    leaf_start[count] = (int32_t)num_requests;
    return MMS_OK;
}

int mms_trace_model_histogram(const mms_trace *trace, int32_t num_models, int32_t *hist,
                              void *stream)
{
    if (!trace || !hist || num_models < 0 || trace->num_requests < 0 || trace->num_traces < 0)
        return MMS_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    if (trace->num_traces > 1) {
        const int64_t T = trace->num_traces;
        if (T > 0x7FFFFFFF) return MMS_ERR_UNSUPPORTED;
        const size_t cells = (size_t)T * (num_models + 1) + 1;
        MMS_CUDA(cudaMemsetAsync(hist, 0, sizeof(int32_t) * cells, st));
        if (trace->num_requests == 0) return MMS_OK;
        if (!trace->model_ids || !trace->arrivals) return MMS_ERR_ARG;
        const size_t smem = sizeof(int32_t) * 32 * ((size_t)num_models + 1);
        if (smem > 48 * 1024) return MMS_ERR_UNSUPPORTED;
        const dim3 block(32, 8);
        int64_t slices = (trace->num_requests + 8 * 256 - 1) / (8 * 256);
        if (slices > 64) slices = 64;
        const dim3 grid((unsigned)((T + 31) / 32), (unsigned)slices);
        mms::histogram_traces_kernel<<<grid, block, smem, st>>>(
            trace->arrivals, trace->model_ids, trace->num_requests, (int32_t)T, num_models, hist);
        MMS_CUDA(cudaGetLastError());
        return MMS_OK;
    }
    MMS_CUDA(cudaMemsetAsync(hist, 0, sizeof(int32_t) * ((size_t)num_models + 1), st));
    if (trace->num_requests == 0) return MMS_OK;
    if (!trace->model_ids || !trace->arrivals) return MMS_ERR_ARG;
    if (((size_t)num_models + 1) * sizeof(int32_t) > 48 * 1024) return MMS_ERR_UNSUPPORTED;
    const int threads = 256;
    int64_t want = (trace->num_requests + threads - 1) / threads;
    const int blocks = (int)(want < 592 ? want : 592);   // 4 blocks per SM on 148 SMs
    mms::histogram_kernel<<<blocks, threads, sizeof(int32_t) * ((size_t)num_models + 1), st>>>(
        trace->arrivals, trace->model_ids, trace->num_requests, num_models, hist);
    MMS_CUDA(cudaGetLastError());
    return MMS_OK;
}

size_t mms_sim_workspace_bytes(int64_t num_requests, const mms_placements *cands,
                               const mms_sim_options *opts, uint32_t flags)
{
    mms::Geometry g;
    if (mms::plan_call(num_requests, cands, opts, flags, !(flags & MMS_FLAG_NO_GROUP_GOOD), &g) !=
        MMS_OK)
        return 0;
    return g.total;
}

int mms_sim_mixed(const mms_trace *trace, const mms_placements *cands, const mms_sum_plan *plan,
                  const int32_t *model_hist, const mms_sim_options *opts, const mms_workspace *ws,
                  const mms_results *out, uint32_t flags, void *stream)
{
    using namespace mms;
    if (!trace || !cands || !plan || !ws || !out) return MMS_ERR_ARG;
    if (flags & ~(MMS_FLAG_PER_REQUEST | MMS_FLAG_LEGACY_CLOCK | MMS_FLAG_NO_GROUP_GOOD |
                  MMS_FLAG_CROWDED))
        return MMS_ERR_ARG;
    const int64_t N = trace->num_requests;
    const bool gg = !(flags & MMS_FLAG_NO_GROUP_GOOD);
    if (gg && !out->group_num_good) return MMS_ERR_ARG;
    Geometry g;
    int rc = plan_call(N, cands, opts, flags, gg, &g);
    if (rc) return rc;
    const int32_t B = cands->num_candidates;
    if (B == 0) return MMS_OK;
    if (!out->model_num_requests || !out->model_num_good || !out->group_num_requests ||
        !out->good_total || !out->latency_sum || !out->status || !model_hist)
        return MMS_ERR_ARG;
    if (N > 0 && (!trace->arrivals || !trace->model_ids || !trace->slos)) return MMS_ERR_ARG;
    if (trace->num_traces < 0 || trace->num_traces > 0x7FFFFFFF) return MMS_ERR_ARG;
    if (trace->num_traces > 1 &&
        (cands->num_scored ? cands->num_scored : cands->num_candidates) > trace->num_traces)
        return MMS_ERR_ARG;                 // every scored candidate needs a trace of its own
    if (!cands->model_off || !cands->group_info || !cands->model_rep || !cands->latency)
        return MMS_ERR_ARG;
    const bool full = (flags & MMS_FLAG_PER_REQUEST) != 0;
    if (full && N > 0 && (!out->finish || !out->good)) return MMS_ERR_ARG;
    if (plan->num_leaves != plan_leaves(N)) return MMS_ERR_ARG;
    if (plan->num_leaves > 0 && (!plan->leaf_start || !plan->leaf_merges)) return MMS_ERR_ARG;
    if (g.total > 0 && (!ws->ptr || ws->bytes < g.total)) return MMS_ERR_ARG;

    cudaStream_t st = (cudaStream_t)stream;
    unsigned char *scratch = (unsigned char *)ws->ptr;
    KernelArgs ka;
    memset(&ka, 0, sizeof(ka));
    ka.arrivals = trace->arrivals; ka.model_ids = trace->model_ids; ka.slos = trace->slos;
    ka.N = N; ka.model_hist = model_hist;
    ka.trace_pitch = trace->num_traces > 1 ? (int32_t)trace->num_traces : 1;
    ka.unsorted = trace->num_traces > 1
                      ? model_hist + (size_t)trace->num_traces * (cands->num_models + 1)
                      : model_hist + cands->num_models;
    ka.B = B; ka.Bs = cands->num_scored ? cands->num_scored : B;
    ka.partner = cands->partner; ka.mirror_swap = cands->mirror_swap;
    ka.M = cands->num_models; ka.G = cands->max_groups; ka.P = cands->max_placed;
    ka.T = cands->max_slots; ka.S = cands->max_stages; ka.C = cands->num_columns;
    ka.model_off = cands->model_off; ka.model_rep = cands->model_rep;
    ka.group_info = cands->group_info; ka.latency = cands->latency;
    ka.latency_stride = cands->latency_stride;
    ka.lat_smem_elems = g.lat_smem_elems; ka.block_warps = g.block_warps;
    ka.lat_f64 = g.lat_smem_elems != 0 ? g.lat_f64 : 0;
    ka.K = g.K; ka.NS = g.NS; ka.seg_len = g.seg_len; ka.seg_per_chunk = g.seg_per_chunk;
    ka.warmup = g.warmup;
    ka.num_leaves = plan->num_leaves; ka.leaf_start = plan->leaf_start;
    ka.rep_rows = (uint32_t *)(scratch + g.off_rows);
    ka.leaf_sums = (double *)(scratch + g.off_leaf);
    ka.decisions = scratch + g.off_decisions;
    ka.dec_wide = cands->max_groups > 126;
    ka.dec_pitch = ((int64_t)B + 31) / 32 * 32;
    ka.work_count = (uint32_t *)(scratch + g.off_work_count);
    ka.work_items = (uint32_t *)(scratch + g.off_work_items);
    ka.repair_from = (int32_t *)(scratch + g.off_repair_from);
    ka.seg_src = (int32_t *)(scratch + g.off_seg_src);
    ka.compat = (uint16_t *)(scratch + g.off_compat);
    ka.own_rewritten = (uint8_t *)(scratch + g.off_own_rewritten);
    ka.seg_first_leaf = (int32_t *)(scratch + g.off_seg_leaf);
    ka.repair_cap = g.repair_cap;
    ka.narrow_limit = g.narrow_limit;
    ka.seg_end = (double *)(scratch + g.off_seg_end);
    ka.chunk_start = (double *)(scratch + g.off_chunk_start);
    ka.status = out->status;
    ka.finish = out->finish; ka.good = out->good;
    ka.resimulated = out->resimulated;

    ClearArgs ca;
    ca.group_info_in = cands->group_info;
    ca.group_info = (uint32_t *)(scratch + g.off_group_info);
    ca.model_num_good = out->model_num_good;
    ca.group_num_requests = out->group_num_requests;
    ca.group_num_good = gg ? out->group_num_good : nullptr;
    ca.good_total = out->good_total;
    ka.group_info = ca.group_info;       // the checked copy, contested bits derived on the device
    ProfileSpan call_span(MMS_PROFILE_CALL, st);
    const bool legacy = (flags & MMS_FLAG_LEGACY_CLOCK) != 0;
    const int variant = (full ? 4 : 0) | (gg ? 2 : 0) | (legacy ? 1 : 0);
    switch (variant) {
        case 0: rc = launch_sim<false, false, false>(ka, ca, g, st); break;
        case 1: rc = launch_sim<false, false, true>(ka, ca, g, st); break;
        case 2: rc = launch_sim<false, true, false>(ka, ca, g, st); break;
        case 3: rc = launch_sim<false, true, true>(ka, ca, g, st); break;
        case 4: rc = launch_sim<true, false, false>(ka, ca, g, st); break;
        case 5: rc = launch_sim<true, false, true>(ka, ca, g, st); break;
        case 6: rc = launch_sim<true, true, false>(ka, ca, g, st); break;
        default: rc = launch_sim<true, true, true>(ka, ca, g, st); break;
    }
    if (rc) return rc;

    // tally the recorded decisions of the selected runs (outputs were cleared up front)
    const size_t hist_bytes = g.smem_count;
    auto count_k = ka.dec_wide ? count_kernel<uint16_t> : count_kernel<uint8_t>;
    MMS_TRY(allow_smem((const void *)count_k, hist_bytes));
    int32_t seg_per_block = ka.NS / 96 > 0 ? ka.NS / 96 : 1;   // 16-bit counts: at most 32 segments
    if (seg_per_block > 32) seg_per_block = 32;
    // one more row of blocks (the first) forms the latency sums
    const dim3 count_grid((unsigned)((ka.Bs + kLanes - 1) / kLanes),
                          (unsigned)((ka.NS + seg_per_block - 1) / seg_per_block) + 1);
    count_k<<<count_grid, kLanes, hist_bytes, st>>>(ka, seg_per_block, gg, out->model_num_good,
                                                    out->group_num_requests, out->group_num_good,
                                                    out->good_total, plan->leaf_merges,
                                                    out->latency_sum);
    MMS_CUDA(cudaGetLastError());
    if (ka.M > 0) {
        const int64_t cells = (int64_t)ka.Bs * ka.M;
        model_requests_kernel<<<(unsigned)((cells + 127) / 128), 128, 0, st>>>(ka, out->model_num_requests);
        MMS_CUDA(cudaGetLastError());
    }
    call_span.stop();
    return MMS_OK;
}

}  // extern "C"

extern "C" {

int mms_trace_pack(const double *arrivals, const int32_t *model_ids, const float *slos,
                   const int64_t *offsets, int64_t num_traces, int64_t padded_requests,
                   double *out_arrivals, int32_t *out_model_ids, float *out_slos, void *stream)
{
    if (num_traces < 0 || padded_requests < 0) return MMS_ERR_ARG;
    if (num_traces == 0 || padded_requests == 0) return MMS_OK;
    if (!arrivals || !model_ids || !slos || !offsets || !out_arrivals || !out_model_ids || !out_slos)
        return MMS_ERR_ARG;
    const int64_t bx = (padded_requests + 31) / 32, by = (num_traces + 31) / 32;
    if (bx > 0x7FFFFFFF || by > 65535) return MMS_ERR_UNSUPPORTED;
    mms::pack_traces_kernel<<<dim3((unsigned)bx, (unsigned)by), dim3(32, 8), 0,
                              (cudaStream_t)stream>>>(arrivals, model_ids, slos, offsets,
                                                      num_traces, padded_requests, out_arrivals,
                                                      out_model_ids, out_slos);
    MMS_CUDA(cudaGetLastError());
    return MMS_OK;
}

int mms_argmax_scores(const int64_t *good_total, const double *latency_sum,
                      const int64_t *num_replicas, int64_t num_requests, int32_t num_candidates,
                      const int64_t *index_map, int64_t index_base, int32_t accumulate,
                      double *best, void *stream)
{
    if (num_candidates < 0 || num_requests < 0 || !best) return MMS_ERR_ARG;
    if (num_candidates > 0 && (!good_total || !latency_sum)) return MMS_ERR_ARG;
    mms::argmax_scores_kernel<<<1, mms::kArgmaxThreads, 0, (cudaStream_t)stream>>>(
        good_total, latency_sum, num_replicas, num_requests, num_candidates, index_map,
        index_base, accumulate != 0, best);
    MMS_CUDA(cudaGetLastError());
    return MMS_OK;
}

}  // extern "C"

namespace mms {

// Scratch of mms_sim_mixed_static.  In host code this name is only a handle
// for cudaGetSymbolAddress, never an address a kernel can use.
static __device__ __align__(256) unsigned char g_static_scratch[MMS_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
static void *g_static_scratch_ptr[kMaxDevices];   // device address, per device ordinal
static std::mutex g_static_scratch_mutex;

}  // namespace mms

extern "C" {

int mms_sim_mixed_static(const mms_trace *trace, const mms_placements *cands,
                         const mms_sum_plan *plan, const int32_t *model_hist,
                         const mms_sim_options *opts, const mms_results *out,
                         uint32_t flags, void *stream)
{
    if (!trace || !cands) return MMS_ERR_ARG;
    // the same shape checks as mms_sim_mixed, with the same return codes; only a
    // shape that is fine but needs more scratch than the array holds is new
    mms::Geometry geo;
    const int rc = mms::plan_call(trace->num_requests, cands, opts, flags,
                                  !(flags & MMS_FLAG_NO_GROUP_GOOD), &geo);
    if (rc != MMS_OK) return rc;
    if (geo.total > (size_t)MMS_STATIC_SCRATCH_BYTES) {
        snprintf(mms::g_last_error, sizeof(mms::g_last_error),
                 "mms_sim_mixed_static: needs %zu bytes of scratch, the built-in array holds %u; "
                 "use fewer candidates per call or mms_sim_mixed with a caller workspace",
                 geo.total, (unsigned)MMS_STATIC_SCRATCH_BYTES);
        return MMS_ERR_UNSUPPORTED;
    }
    int dev = -1;
    MMS_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= mms::kMaxDevices) return MMS_ERR_NO_DEVICE;
    {
        // once per device, with that device current (under a lock: two host
        // threads may make the first call together)
        std::lock_guard<std::mutex> lock(mms::g_static_scratch_mutex);
        if (!mms::g_static_scratch_ptr[dev]) {
            void *p = nullptr;
            MMS_CUDA(cudaGetSymbolAddress(&p, mms::g_static_scratch));
            mms::g_static_scratch_ptr[dev] = p;
        }
    }
    mms_workspace ws;
    ws.ptr = mms::g_static_scratch_ptr[dev];
    ws.bytes = (size_t)MMS_STATIC_SCRATCH_BYTES;
    return mms_sim_mixed(trace, cands, plan, model_hist, opts, &ws, out, flags, stream);
}

int mms_trace_next_same_model(const mms_trace *trace, int32_t num_models, int32_t *next_same,
                              void *stream)
{
    if (!trace || num_models < 0 || trace->num_requests < 0) return MMS_ERR_ARG;
    if (trace->num_requests > 0x7FFFFFFF) return MMS_ERR_UNSUPPORTED;
    if (trace->num_requests == 0 || num_models == 0) return MMS_OK;
    if (!trace->model_ids || !next_same) return MMS_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    // requests of unknown models (-1) are never queued; give them a defined value
    MMS_CUDA(cudaMemsetAsync(next_same, 0xFF, sizeof(int32_t) * (size_t)trace->num_requests, st));
    mms::next_same_kernel<<<(num_models + 31) / 32, 32, 0, st>>>(
        trace->model_ids, trace->num_requests, num_models, next_same);
    MMS_CUDA(cudaGetLastError());
    return MMS_OK;
}

}  // extern "C"

namespace mms {

struct BatchGeometry {
    int32_t simd, H, K, chunk_len, warmup, Bp;
    size_t smem_single, smem_simd;
    size_t off_leaf, off_start, off_end, off_counters, off_carry, off_flag, off_tables, off_work,
        total;
    int32_t rounds;
};

constexpr int kBatchRepairRounds = 3;

// Chunking and scratch layout of one mms_sim_batching call.
static int plan_batching(int64_t N, const mms_placements *c, const mms_batching *bt,
                         BatchGeometry *g)
{
    if (!c || !bt || N < 0 || N > 0x7FFFFFFF || c->num_candidates < 0) return MMS_ERR_ARG;
    const int64_t B = c->num_candidates;
    g->H = bt->heap_capacity > 0 ? bt->heap_capacity : c->max_groups + 16;
    // 32 candidates per warp (batch_simd_kernel) once there are enough of them to fill
    // warps; else one candidate per warp
    g->simd = B >= 24 ? 1 : 0;
    g->Bp = (int32_t)((B + kLanes - 1) / kLanes * kLanes);
    g->smem_single = batch_smem(c->num_models, c->max_groups, c->max_placed, c->max_slots,
                                g->H, 1).total;
    g->smem_simd = batch_smem(c->num_models, c->max_groups, c->max_placed, c->max_slots,
                              g->H, kLanes).total;
    if (g->smem_simd > 227 * 1024) g->simd = 0;
    int sm_count = 148, dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
        (void)cudaGetLastError();
        sm_count = 148;
    }
    // Chunks: as many as fill ONE wave of the blocks that can be resident (shared memory
    // decides), none shorter than twice the run-in, and no cut at all when that leaves fewer
    // than two.
    g->warmup = 2048;
    int64_t K = 1;
    if (B > 0 && N >= 4 * 4096) {
        const size_t smem = g->simd ? g->smem_simd : g->smem_single;
        int64_t per_sm = (int64_t)(233472 / (smem + 1024));
        if (per_sm > kBatchBlocksPerSm) per_sm = kBatchBlocksPerSm;
        if (per_sm < 1) per_sm = 1;
        const int64_t blocks_per_chunk = g->simd ? g->Bp / kLanes : B;
        K = per_sm * sm_count / blocks_per_chunk;
        if (K > N / 4096) K = N / 4096;
        if (K < (g->simd ? 2 : 4)) K = 1;
    }
    const int64_t len = (N + K - 1) / (K > 0 ? K : 1);
    g->chunk_len = (int32_t)(len > 0 ? len : 1);
    g->K = (int32_t)(N > 0 ? (N + g->chunk_len - 1) / g->chunk_len : 1);
    const size_t cells = (size_t)g->K * (size_t)(B > 0 ? B : 1);
    const size_t sb = batch_state_bytes(c->num_models, c->max_groups, c->max_slots, g->H);
    size_t off = 0;
    g->off_leaf = off;     off += align256(sizeof(double) * (size_t)plan_leaves(N) * (size_t)B + 8);
    g->off_flag = off;     off += 256;
    g->off_counters = off; off += align256(sizeof(uint32_t) * cells * (2 * c->num_models + 2 * c->max_groups));
    g->off_carry = off;    off += align256(cells * batch_carry_bytes());
    g->off_tables = off;
    if (g->simd)           // t_mrep, t_gcfg, t_status (u32), then t_moff, t_goff, t_gmod (u16)
        off += align256((size_t)g->Bp * (4 * ((size_t)c->max_placed + c->max_groups + 1) +
                                          2 * ((size_t)c->num_models + c->max_groups + 2 +
                                               c->max_placed)) + 64);
    g->rounds = kBatchRepairRounds;
    g->off_work = off;     off += g->K > 1 ? align256(sizeof(uint32_t) * (cells + 64)) : 0;
    g->off_start = off;    off += g->K > 1 ? align256(cells * sb) : 0;
    g->off_end = off;      off += g->K > 1 ? align256(cells * sb) : 0;
    g->total = off;
    return MMS_OK;
}

}  // namespace mms

extern "C" {

size_t mms_sim_batching_workspace_bytes(int64_t num_requests, const mms_placements *cands,
                                        const mms_batching *batching)
{
    mms::BatchGeometry g;
    if (mms::plan_batching(num_requests, cands, batching, &g) != MMS_OK) return 0;
    return g.total;
}

int mms_sim_batching(const mms_trace *trace, const mms_placements *cands,
                     const mms_batching *batching, const int32_t *next_same,
                     const mms_sum_plan *plan, const mms_workspace *ws, const mms_results *out,
                     void *stream)
{
    using namespace mms;
    if (!trace || !cands || !batching || !plan || !ws || !out) return MMS_ERR_ARG;
    const int64_t N = trace->num_requests;
    const int32_t B = cands->num_candidates;
    if (N < 0 || B < 0 || cands->num_models < 0 || cands->max_groups < 0 ||
        cands->max_placed < 0 || cands->max_slots < 0 || cands->max_stages < 1 ||
        cands->num_columns < 0)
        return MMS_ERR_ARG;
    if (N > 0x7FFFFFFF || cands->max_groups > MMS_MAX_GROUPS || cands->max_slots > MMS_MAX_SLOTS ||
        cands->max_placed > MMS_MAX_PLACED || cands->max_stages > MMS_MAX_STAGES ||
        cands->num_columns > MMS_MAX_COLUMNS)
        return MMS_ERR_UNSUPPORTED;
    if (trace->num_traces > 1) return MMS_ERR_UNSUPPORTED;   // one shared trace only
    const int NB = batching->num_batch_sizes;
    if (NB < 1 || NB > 8 || batching->batch_sizes[0] != 1) return MMS_ERR_ARG;
    if (B == 0) return MMS_OK;
    if (!out->model_num_requests || !out->model_num_good || !out->group_num_requests ||
        !out->group_num_good || !out->good_total || !out->latency_sum || !out->status)
        return MMS_ERR_ARG;
    if (N > 0 && (!trace->arrivals || !trace->model_ids || !trace->slos || !next_same ||
                  !out->finish || !out->good))
        return MMS_ERR_ARG;
    if (!cands->model_off || !cands->model_rep || !cands->latency || !batching->group_off ||
        !batching->group_mod || !batching->group_cfg)
        return MMS_ERR_ARG;
    if (plan->num_leaves != plan_leaves(N)) return MMS_ERR_ARG;
    if (plan->num_leaves > 0 && (!plan->leaf_start || !plan->leaf_merges)) return MMS_ERR_ARG;
    BatchGeometry geo;
    if (plan_batching(N, cands, batching, &geo) != MMS_OK) return MMS_ERR_ARG;
    if (!ws->ptr || ws->bytes < geo.total) return MMS_ERR_ARG;

    BatchArgs a;
    memset(&a, 0, sizeof(a));
    a.arrivals = trace->arrivals; a.model_ids = trace->model_ids; a.slos = trace->slos;
    a.next_same = next_same; a.N = N;
    a.B = B; a.M = cands->num_models; a.G = cands->max_groups; a.P = cands->max_placed;
    a.T = cands->max_slots; a.S = cands->max_stages; a.C = cands->num_columns; a.NB = NB;
    a.H = geo.H;
    for (int j = 0; j < NB; ++j) {
        const int32_t bs = batching->batch_sizes[j];
        if (bs < 1 || (bs & (bs - 1)) || (j > 0 && bs <= batching->batch_sizes[j - 1]))
            return MMS_ERR_ARG;
        int col = 0;
        while ((1 << col) < bs) ++col;
        if (col >= NB) return MMS_ERR_ARG;   // the reference would index past the table
        a.batch_sizes[j] = bs;
        a.batch_cols[j] = col;
    }
    a.model_off = cands->model_off; a.model_rep = cands->model_rep;
    a.group_off = batching->group_off; a.group_mod = batching->group_mod;
    a.group_cfg = batching->group_cfg;
    a.latency = cands->latency; a.latency_stride = cands->latency_stride;
    a.finish = out->finish; a.good = out->good;
    a.model_num_requests = out->model_num_requests; a.model_num_good = out->model_num_good;
    a.group_num_requests = out->group_num_requests; a.group_num_good = out->group_num_good;
    a.status = out->status;
    a.lanes = geo.simd ? kLanes : 1;
    if (geo.smem_single > 227 * 1024) return MMS_ERR_UNSUPPORTED;
    unsigned char *scratch = (unsigned char *)ws->ptr;
    a.K = geo.K; a.chunk_len = geo.chunk_len; a.warmup = geo.warmup;
    a.unsorted = (const int32_t *)(scratch + geo.off_flag);
    a.chunk_counters = (uint32_t *)(scratch + geo.off_counters);
    a.carry = scratch + geo.off_carry;
    a.snap_start = scratch + geo.off_start;
    a.snap_end = scratch + geo.off_end;
    a.resimulated = out->resimulated;
    a.Bp = geo.Bp;
    if (geo.simd) {
        const size_t Bp = (size_t)geo.Bp;
        unsigned char *t = scratch + geo.off_tables;
        a.t_mrep = (uint32_t *)t;   t += 4 * Bp * (size_t)a.P;
        a.t_gcfg = (uint32_t *)t;   t += 4 * Bp * (size_t)a.G;
        a.t_status = (uint32_t *)t; t += 4 * Bp;
        a.t_moff = (uint16_t *)t;   t += 2 * Bp * (size_t)(a.M + 1);
        a.t_goff = (uint16_t *)t;   t += 2 * Bp * (size_t)(a.G + 1);
        a.t_gmod = (uint16_t *)t;
    }

    cudaStream_t st = (cudaStream_t)stream;
    MMS_CUDA(cudaMemsetAsync(scratch + geo.off_flag, 0, 256, st));
    MMS_CUDA(cudaMemsetAsync(out->status, 0, sizeof(uint32_t) * (size_t)B, st));
    if (out->resimulated)
        MMS_CUDA(cudaMemsetAsync(out->resimulated, 0, sizeof(int32_t) * (size_t)B, st));
    if (N > 0 && a.K > 1) {
        unsorted_kernel<<<296, 256, 0, st>>>(trace->arrivals, N, (int32_t *)(scratch + geo.off_flag));
        MMS_CUDA(cudaGetLastError());
    }
    MMS_TRY(allow_smem((const void *)batch_chain_kernel, geo.smem_single));
    if (geo.simd) {
        // the lanes add to the chunks' counters in global memory
        MMS_CUDA(cudaMemsetAsync(a.chunk_counters, 0,
                                 sizeof(uint32_t) * (size_t)a.K * B * (2 * a.M + 2 * a.G), st));
        batch_tables_kernel<<<(unsigned)((geo.Bp + 127) / 128), 128, 0, st>>>(a);
        MMS_CUDA(cudaGetLastError());
        MMS_TRY(allow_smem((const void *)batch_simd_kernel, geo.smem_simd));
        ProfileSpan stream_span(MMS_PROFILE_BATCH_STREAM, st);
        batch_simd_kernel<<<(unsigned)((int64_t)a.K * (geo.Bp / kLanes)), kLanes, geo.smem_simd,
                            st>>>(a);
        MMS_CUDA(cudaGetLastError());
        stream_span.stop();
    } else {
        MMS_TRY(allow_smem((const void *)batch_stream_kernel, geo.smem_single));
        ProfileSpan stream_span(MMS_PROFILE_BATCH_STREAM, st);
        batch_stream_kernel<<<(unsigned)((int64_t)B * a.K), kLanes, geo.smem_single, st>>>(a);
        MMS_CUDA(cudaGetLastError());
        stream_span.stop();
    }
    if (a.K > 1) {
        // a few rounds of parallel repairs, one re-simulated chunk per warp, then the chain
        a.work_count = (uint32_t *)(scratch + geo.off_work);
        a.work_items = a.work_count + 64;
        MMS_CUDA(cudaMemsetAsync(a.work_count, 0, sizeof(uint32_t) * 64, st));
        MMS_TRY(allow_smem((const void *)batch_repair_kernel, geo.smem_single));
        const int64_t bounds = (int64_t)B * (a.K - 1);
        ProfileSpan repair_span(MMS_PROFILE_BATCH_REPAIR, st);
        for (int r = 0; r < geo.rounds; ++r) {
            a.round = r;
            batch_validate_kernel<<<(unsigned)((bounds + 127) / 128), 128, 0, st>>>(a);
            MMS_CUDA(cudaGetLastError());
            batch_repair_kernel<<<(unsigned)bounds, kLanes, geo.smem_single, st>>>(a);
            MMS_CUDA(cudaGetLastError());
        }
        repair_span.stop();
        ProfileSpan chain_span(MMS_PROFILE_BATCH_CHAIN, st);
        batch_chain_kernel<<<(unsigned)B, kLanes, geo.smem_single, st>>>(a);
        MMS_CUDA(cudaGetLastError());
        chain_span.stop();
    }
    const int64_t sum_cells = (int64_t)B * (2 * a.M + 2 * a.G);
    batch_sum_kernel<<<(unsigned)((sum_cells + 127) / 128), 128, 0, st>>>(a);
    MMS_CUDA(cudaGetLastError());
    double *leaf_sums = (double *)(scratch + geo.off_leaf);
    if (plan->num_leaves > 0) {
        const int64_t cells = (int64_t)B * plan->num_leaves;
        leaf_sums_from_finish_kernel<<<(unsigned)((cells + 127) / 128), 128, 0, st>>>(
            out->finish, trace->arrivals, N, B, plan->num_leaves, plan->leaf_start, leaf_sums);
        MMS_CUDA(cudaGetLastError());
    }
    KernelArgs fa;                         // what finalize_kernel reads; one run per candidate
    memset(&fa, 0, sizeof(fa));
    fa.B = fa.Bs = B; fa.M = a.M; fa.num_leaves = plan->num_leaves;
    fa.leaf_sums = leaf_sums; fa.status = out->status;
    finalize_kernel<<<(B + 31) / 32, 32, 0, st>>>(
        fa, plan->leaf_merges, out->model_num_good, out->good_total, out->latency_sum);
    MMS_CUDA(cudaGetLastError());
    return MMS_OK;
}

}  // extern "C"
