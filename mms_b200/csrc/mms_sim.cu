// mms_sim.cu — sm_100a kernels and C ABI of the placement-evaluation simulator.
//
// What is simulated: AlpaServe's per-request FIFO pipeline model with SLO
// dropping (alpa_serve/simulator/controller.py:561-628, and :506-558 for the
// one-clock-per-group variant), for a batch of candidate placements against
// one request trace, followed by the fast_stats reductions of
// controller.py:393-403.
//
// Mapping to the GPU: the recurrence over requests is sequential per
// candidate, so one THREAD owns one candidate and walks the trace; the 32
// lanes of a warp are 32 candidates reading the same request (one broadcast
// load per warp).  A candidate's mutable state (stage clocks, counters) and
// its placement tables sit in shared memory, laid out [entry][lane] so that
// lane-private accesses never collide on a bank.  All arithmetic on time is
// fp64 in the reference's order (max, then add; 0.011 s added last), built
// with -fmad=false.
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstring>

#include "mms_sim.h"

namespace {

constexpr double kInf = 1e100;          // alpa_serve/util.py:23
constexpr double kOverhead = 0.011;     // controller.py:575
constexpr int kLanes = 32;              // candidates per block (one warp)
constexpr int kMaxSumDepth = 48;        // pair-sum stack of the numpy order

thread_local char g_last_error[256] = "";

int cuda_fail(cudaError_t e, const char *what)
{
    snprintf(g_last_error, sizeof(g_last_error), "%s: %s", what, cudaGetErrorString(e));
    return MMS_ERR_CUDA;
}

#define MMS_CUDA(call)                                             \
    do {                                                           \
        cudaError_t e_ = (call);                                   \
        if (e_ != cudaSuccess) return cuda_fail(e_, #call);        \
    } while (0)

struct KernelArgs {
    // trace
    const double *arrivals;
    const int32_t *model_ids;
    const float *slos;
    int64_t N;
    // placements
    int32_t B, M, G, P, T, S, C;
    const uint16_t *model_off;
    const uint16_t *model_rep;
    const uint32_t *group_info;
    const float *latency;
    int64_t latency_stride;
    // summation plan
    int32_t num_leaves;
    const int32_t *leaf_start;
    // outputs
    double *leaf_sums;            // [num_leaves][B]
    int32_t *model_num_good;      // [B][M]
    int32_t *group_num_requests;  // [B][G]
    int32_t *group_num_good;      // [B][G] or null
    uint32_t *status;             // [B]
    double *finish;               // [B][N] or null
    uint8_t *good;                // [B][N] or null
};

// Shared-memory carve-up for one block of kLanes candidates.  Every array is
// [entry][lane].
struct SmemLayout {
    size_t clocks, stage_tmp, counters, group_info, model_off, model_rep, total;
    int n_counters;
};

__host__ __device__ inline SmemLayout smem_layout(int M, int G, int P, int T, int S,
                                                  bool group_good)
{
    SmemLayout L;
    size_t off = 0;
    L.clocks = off;      off += sizeof(double) * (size_t)T * kLanes;
    L.stage_tmp = off;   off += sizeof(double) * (size_t)S * kLanes;
    L.n_counters = M + G + (group_good ? G : 0);
    L.counters = off;    off += sizeof(uint32_t) * (size_t)L.n_counters * kLanes;
    L.group_info = off;  off += sizeof(uint32_t) * (size_t)G * kLanes;
    L.model_off = off;   off += sizeof(uint16_t) * (size_t)(M + 1) * kLanes;
    L.model_rep = off;   off += sizeof(uint16_t) * (size_t)P * kLanes;
    L.total = (off + 15) & ~(size_t)15;
    return L;
}

// One candidate's view of its shared-memory state.
struct Lane {
    double *clk;          // [T]  stride kLanes
    double *tmp;          // [S]
    uint32_t *model_good; // [M]
    uint32_t *group_req;  // [G]
    uint32_t *group_good; // [G] or null
    const uint32_t *ginfo;
    const uint16_t *moff;
    const uint16_t *mrep;
    const float *lat;
    int32_t M, C, S;
    uint32_t status;
};

// One request of controller.py:579-622.  Returns finish - arrival (0.0 for a
// dropped request, as the reference stores finish = arrival for those).
template <bool kFull, bool kGroupGood, bool kLegacy>
__device__ __forceinline__ double sim_step(Lane &ln, double ts, int32_t m, float slo_f,
                                           double *finish_out, uint8_t *good_out, int64_t i)
{
    double fin = ts;
    bool ok = false;
    if (m >= 0) {
        if (m >= ln.M) {
            ln.status |= MMS_STATUS_BAD_INDEX;
        } else {
            // :589-598 replica whose last-stage clock is strictly smallest
            const uint32_t lo = ln.moff[(size_t)m * kLanes];
            const uint32_t hi = ln.moff[(size_t)(m + 1) * kLanes];
            double best = kInf;
            uint32_t pick = 0xFFFFFFFFu;
            for (uint32_t e = lo; e < hi; ++e) {
                const uint32_t ent = ln.mrep[(size_t)e * kLanes];
                const double c = ln.clk[(size_t)(ent >> 8) * kLanes];
                if (c < best) { best = c; pick = ent; }
            }
            if (pick != 0xFFFFFFFFu) {
                const uint32_t g = pick & 0xFFu;
                const uint32_t info = ln.ginfo[(size_t)g * kLanes];
                const uint32_t slot = info & 0xFFu;
                const uint32_t col = info >> 16;
                const float *lat = ln.lat + ((size_t)m * ln.C + col) * ln.S;
                double t;
                uint32_t ns;
                if (kLegacy) {
                    // :543-544 one clock per group; lat = {sum, max}
                    ns = 1;
                    const double start = fmax(ln.clk[(size_t)slot * kLanes], ts);
                    t = start + (double)__ldg(lat);
                    ln.tmp[0] = start + (double)__ldg(lat + 1);
                } else {
                    // :605-608 walk the pipeline stages
                    ns = (info >> 8) & 0xFFu;
                    t = ts;
                    for (uint32_t k = 0; k < ns; ++k) {
                        t = fmax(t, ln.clk[(size_t)(slot + k) * kLanes]) + (double)__ldg(lat + k);
                        ln.tmp[(size_t)k * kLanes] = t;
                    }
                }
                const double f = t + kOverhead;                 // :610
                ln.group_req[(size_t)g * kLanes] += 1;          // :611
                if (f - ts <= (double)slo_f) {                  // :613-619
                    fin = f;
                    ok = true;
                    for (uint32_t k = 0; k < ns; ++k)
                        ln.clk[(size_t)(slot + k) * kLanes] = ln.tmp[(size_t)k * kLanes];
                    ln.model_good[(size_t)m * kLanes] += 1;
                    if (kGroupGood) ln.group_good[(size_t)g * kLanes] += 1;
                }
            }
        }
    }
    if (kFull) {
        finish_out[i] = fin;
        good_out[i] = ok ? 1 : 0;
    }
    return fin - ts;
}

template <bool kFull, bool kGroupGood, bool kLegacy>
__global__ void __launch_bounds__(kLanes)
sim_mixed_kernel(const KernelArgs a)
{
    extern __shared__ __align__(16) unsigned char smem[];
    const int lane = threadIdx.x;
    const int64_t b = (int64_t)blockIdx.x * kLanes + lane;
    if (b >= a.B) return;   // lanes never synchronise with each other

    const SmemLayout L = smem_layout(a.M, a.G, a.P, a.T, a.S, kGroupGood);
    Lane ln;
    ln.clk = reinterpret_cast<double *>(smem + L.clocks) + lane;
    ln.tmp = reinterpret_cast<double *>(smem + L.stage_tmp) + lane;
    uint32_t *cnt = reinterpret_cast<uint32_t *>(smem + L.counters) + lane;
    ln.model_good = cnt;
    ln.group_req = cnt + (size_t)a.M * kLanes;
    ln.group_good = kGroupGood ? cnt + (size_t)(a.M + a.G) * kLanes : nullptr;
    uint32_t *ginfo = reinterpret_cast<uint32_t *>(smem + L.group_info) + lane;
    uint16_t *moff = reinterpret_cast<uint16_t *>(smem + L.model_off) + lane;
    uint16_t *mrep = reinterpret_cast<uint16_t *>(smem + L.model_rep) + lane;
    ln.ginfo = ginfo; ln.moff = moff; ln.mrep = mrep;
    ln.lat = a.latency + (size_t)b * a.latency_stride;
    ln.M = a.M; ln.C = a.C; ln.S = a.S;
    ln.status = 0;

    // Bring this candidate's tables on chip, checking every index they hold.
    for (int t = 0; t < a.T; ++t) ln.clk[(size_t)t * kLanes] = 0.0;
    for (int c = 0; c < L.n_counters; ++c) cnt[(size_t)c * kLanes] = 0;
    for (int g = 0; g < a.G; ++g) {
        uint32_t info = a.group_info[(size_t)b * a.G + g];
        const uint32_t slot = info & 0xFFu, ns = (info >> 8) & 0xFFu, col = info >> 16;
        if (slot + ns > (uint32_t)a.T || ns > (uint32_t)a.S || col >= (uint32_t)a.C) {
            ln.status |= MMS_STATUS_BAD_INDEX;
            info = 0;   // zero stages: harmless
        }
        ginfo[(size_t)g * kLanes] = info;
    }
    uint32_t prev = 0;
    for (int m = 0; m <= a.M; ++m) {
        uint32_t o = a.model_off[(size_t)b * (a.M + 1) + m];
        if (o < prev || o > (uint32_t)a.P) { ln.status |= MMS_STATUS_BAD_INDEX; o = prev; }
        moff[(size_t)m * kLanes] = (uint16_t)o;
        prev = o;
    }
    for (uint32_t e = 0; e < prev; ++e) {
        uint32_t ent = a.model_rep[(size_t)b * a.P + e];
        if ((ent & 0xFFu) >= (uint32_t)a.G || (ent >> 8) >= (uint32_t)a.T) {
            ln.status |= MMS_STATUS_BAD_INDEX;
            ent = 0;
        }
        mrep[(size_t)e * kLanes] = (uint16_t)ent;
    }
    if (ln.status & MMS_STATUS_BAD_INDEX) {
        // Tables cannot be trusted: make every model replica-less.
        for (int m = 0; m <= a.M; ++m) moff[(size_t)m * kLanes] = 0;
    }

    double *fin_out = kFull ? a.finish + (size_t)b * a.N : nullptr;
    uint8_t *good_out = kFull ? a.good + (size_t)b * a.N : nullptr;

    // Walk the trace leaf by leaf of numpy's pairwise sum: within a leaf the
    // latency of request j goes to partial sum j mod 8.
    for (int32_t leaf = 0; leaf < a.num_leaves; ++leaf) {
        const int64_t s = a.leaf_start[leaf];
        const int64_t e = a.leaf_start[leaf + 1];
        const int64_t body_end = s + ((e - s) & ~(int64_t)7);
        double p0 = 0.0, p1 = 0.0, p2 = 0.0, p3 = 0.0, p4 = 0.0, p5 = 0.0, p6 = 0.0, p7 = 0.0;
        int64_t i = s;
        for (; i < body_end; i += 8) {
#define MMS_STEP(j, acc)                                                                   \
            acc += sim_step<kFull, kGroupGood, kLegacy>(ln, __ldg(a.arrivals + i + j),     \
                __ldg(a.model_ids + i + j), __ldg(a.slos + i + j), fin_out, good_out, i + j)
            MMS_STEP(0, p0); MMS_STEP(1, p1); MMS_STEP(2, p2); MMS_STEP(3, p3);
            MMS_STEP(4, p4); MMS_STEP(5, p5); MMS_STEP(6, p6); MMS_STEP(7, p7);
#undef MMS_STEP
        }
        double r = ((p0 + p1) + (p2 + p3)) + ((p4 + p5) + (p6 + p7));
        for (; i < e; ++i)
            r += sim_step<kFull, kGroupGood, kLegacy>(ln, __ldg(a.arrivals + i),
                __ldg(a.model_ids + i), __ldg(a.slos + i), fin_out, good_out, i);
        a.leaf_sums[(size_t)leaf * a.B + b] = r;
    }

    for (int m = 0; m < a.M; ++m)
        a.model_num_good[(size_t)b * a.M + m] = (int32_t)ln.model_good[(size_t)m * kLanes];
    for (int g = 0; g < a.G; ++g) {
        a.group_num_requests[(size_t)b * a.G + g] = (int32_t)ln.group_req[(size_t)g * kLanes];
        if (kGroupGood)
            a.group_num_good[(size_t)b * a.G + g] = (int32_t)ln.group_good[(size_t)g * kLanes];
    }
    a.status[b] = ln.status;
}

// Combines the leaf sums in numpy's pairing order and finishes the per-
// candidate totals (controller.py:393-403 consumes them).
__global__ void finalize_kernel(int32_t B, int32_t M, int32_t num_leaves,
                                const uint8_t *leaf_merges, const double *leaf_sums,
                                const int32_t *model_hist, const int32_t *model_num_good,
                                int32_t *model_num_requests, int64_t *good_total,
                                double *latency_sum, uint32_t *status)
{
    const int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= B) return;
    double stack[kMaxSumDepth];
    int sp = 0;
    for (int32_t leaf = 0; leaf < num_leaves; ++leaf) {
        if (sp < kMaxSumDepth) stack[sp] = leaf_sums[(size_t)leaf * B + b];
        ++sp;
        for (int k = leaf_merges[leaf]; k > 0 && sp >= 2; --k) {
            --sp;
            if (sp < kMaxSumDepth) stack[sp - 1] = stack[sp - 1] + stack[sp];
        }
    }
    if (sp > kMaxSumDepth) status[b] |= MMS_STATUS_BAD_INDEX;
    latency_sum[b] = (num_leaves > 0) ? stack[0] : 0.0;
    int64_t total = 0;
    for (int m = 0; m < M; ++m) {
        total += model_num_good[(size_t)b * M + m];
        model_num_requests[(size_t)b * M + m] = model_hist[m];
    }
    good_total[b] = total;
}

__global__ void histogram_kernel(const int32_t *model_ids, int64_t N, int32_t M, int32_t *hist)
{
    extern __shared__ int32_t local[];
    for (int m = threadIdx.x; m < M; m += blockDim.x) local[m] = 0;
    __syncthreads();
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < N; i += stride) {
        const int32_t m = model_ids[i];
        if (m >= 0 && m < M) atomicAdd(&local[m], 1);
    }
    __syncthreads();
    for (int m = threadIdx.x; m < M; m += blockDim.x)
        if (local[m]) atomicAdd(&hist[m], local[m]);
}

// numpy's pairwise split of n elements starting at `base`.
void plan_rec(int64_t base, int64_t n, int32_t *leaf_start, uint8_t *merges, int32_t &count)
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

template <bool kFull, bool kGroupGood, bool kLegacy>
int launch_sim(const KernelArgs &ka, size_t smem, cudaStream_t st)
{
    auto kern = sim_mixed_kernel<kFull, kGroupGood, kLegacy>;
    MMS_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int blocks = (ka.B + kLanes - 1) / kLanes;
    kern<<<blocks, kLanes, smem, st>>>(ka);
    MMS_CUDA(cudaGetLastError());
    return MMS_OK;
}

int check_shape(const mms_placements *c, uint32_t flags, SmemLayout *out)
{
    if (!c || c->num_candidates < 0 || c->num_models < 0 || c->max_groups < 0 ||
        c->max_placed < 0 || c->max_slots < 0 || c->max_stages < 0 || c->num_columns < 0)
        return MMS_ERR_ARG;
    if (c->max_groups > MMS_MAX_GROUPS || c->max_slots > MMS_MAX_SLOTS ||
        c->max_placed > MMS_MAX_PLACED || c->max_stages > MMS_MAX_STAGES ||
        c->num_columns > 65535)
        return MMS_ERR_UNSUPPORTED;
    if ((flags & MMS_FLAG_LEGACY_CLOCK) && c->max_stages != 2) return MMS_ERR_ARG;
    const SmemLayout L = smem_layout(c->num_models, c->max_groups, c->max_placed,
                                     c->max_slots, c->max_stages, true);
    if (L.total > 227 * 1024) return MMS_ERR_UNSUPPORTED;
    if (out) *out = L;
    return MMS_OK;
}

}  // namespace

extern "C" {

int mms_abi_version(void) { return 1; }

const char *mms_last_error(void) { return g_last_error; }

int32_t mms_sum_plan_leaves(int64_t num_requests)
{
    if (num_requests <= 0) return 0;
    if (num_requests > 0x7FFFFFFF) return MMS_ERR_UNSUPPORTED;
    int32_t count = 0;
    plan_rec(0, num_requests, nullptr, nullptr, count);
    return count;
}

int mms_sum_plan_fill(int64_t num_requests, int32_t *leaf_start, uint8_t *leaf_merges)
{
    if (num_requests < 0 || !leaf_start || !leaf_merges) return MMS_ERR_ARG;
    if (num_requests > 0x7FFFFFFF) return MMS_ERR_UNSUPPORTED;
    int32_t count = 0;
    if (num_requests > 0) plan_rec(0, num_requests, leaf_start, leaf_merges, count);
    leaf_start[count] = (int32_t)num_requests;
    return MMS_OK;
}

int mms_trace_model_histogram(const mms_trace *trace, int32_t num_models, int32_t *hist,
                              void *stream)
{
    if (!trace || !hist || num_models < 0 || trace->num_requests < 0) return MMS_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    MMS_CUDA(cudaMemsetAsync(hist, 0, sizeof(int32_t) * (size_t)num_models, st));
    if (trace->num_requests == 0 || num_models == 0) return MMS_OK;
    if (!trace->model_ids) return MMS_ERR_ARG;
    if ((size_t)num_models * sizeof(int32_t) > 48 * 1024) return MMS_ERR_UNSUPPORTED;
    const int threads = 256;
    int64_t want = (trace->num_requests + threads - 1) / threads;
    const int blocks = (int)(want < 592 ? want : 592);   // 4 blocks per SM on 148 SMs
    histogram_kernel<<<blocks, threads, sizeof(int32_t) * (size_t)num_models, st>>>(
        trace->model_ids, trace->num_requests, num_models, hist);
    MMS_CUDA(cudaGetLastError());
    return MMS_OK;
}

size_t mms_sim_workspace_bytes(int64_t num_requests, const mms_placements *cands, uint32_t flags)
{
    (void)flags;
    if (!cands || num_requests < 0) return 0;
    const int32_t leaves = mms_sum_plan_leaves(num_requests);
    if (leaves < 0) return 0;
    size_t bytes = sizeof(double) * (size_t)leaves * (size_t)cands->num_candidates;
    return (bytes + 255) & ~(size_t)255;
}

int mms_sim_mixed(const mms_trace *trace, const mms_placements *cands, const mms_sum_plan *plan,
                  const int32_t *model_hist, const mms_workspace *ws, const mms_results *out,
                  uint32_t flags, void *stream)
{
    if (!trace || !cands || !plan || !ws || !out) return MMS_ERR_ARG;
    if (flags & ~(MMS_FLAG_PER_REQUEST | MMS_FLAG_LEGACY_CLOCK)) return MMS_ERR_ARG;
    SmemLayout L;
    int rc = check_shape(cands, flags, &L);
    if (rc) return rc;
    const int64_t N = trace->num_requests;
    const int32_t B = cands->num_candidates;
    if (N < 0 || N > 0x7FFFFFFF) return N < 0 ? MMS_ERR_ARG : MMS_ERR_UNSUPPORTED;
    if (B == 0) return MMS_OK;
    if (!out->model_num_requests || !out->model_num_good || !out->group_num_requests ||
        !out->good_total || !out->latency_sum || !out->status || !model_hist)
        return MMS_ERR_ARG;
    if (N > 0 && (!trace->arrivals || !trace->model_ids || !trace->slos)) return MMS_ERR_ARG;
    if (!cands->model_off || !cands->group_info || (cands->max_placed > 0 && !cands->model_rep) ||
        !cands->latency)
        return MMS_ERR_ARG;
    const bool full = (flags & MMS_FLAG_PER_REQUEST) != 0;
    if (full && N > 0 && (!out->finish || !out->good)) return MMS_ERR_ARG;
    if (plan->num_leaves != mms_sum_plan_leaves(N)) return MMS_ERR_ARG;
    if (plan->num_leaves > 0 && (!plan->leaf_start || !plan->leaf_merges)) return MMS_ERR_ARG;
    const size_t need = mms_sim_workspace_bytes(N, cands, flags);
    if (need > 0 && (!ws->ptr || ws->bytes < need)) return MMS_ERR_ARG;

    cudaStream_t st = (cudaStream_t)stream;
    KernelArgs ka;
    memset(&ka, 0, sizeof(ka));
    ka.arrivals = trace->arrivals; ka.model_ids = trace->model_ids; ka.slos = trace->slos;
    ka.N = N;
    ka.B = B; ka.M = cands->num_models; ka.G = cands->max_groups; ka.P = cands->max_placed;
    ka.T = cands->max_slots; ka.S = cands->max_stages; ka.C = cands->num_columns;
    ka.model_off = cands->model_off; ka.model_rep = cands->model_rep;
    ka.group_info = cands->group_info; ka.latency = cands->latency;
    ka.latency_stride = cands->latency_stride;
    ka.num_leaves = plan->num_leaves; ka.leaf_start = plan->leaf_start;
    ka.leaf_sums = (double *)ws->ptr;
    ka.model_num_good = out->model_num_good;
    ka.group_num_requests = out->group_num_requests;
    ka.group_num_good = out->group_num_good;
    ka.status = out->status;
    ka.finish = out->finish; ka.good = out->good;

    const bool gg = out->group_num_good != nullptr;
    const bool legacy = (flags & MMS_FLAG_LEGACY_CLOCK) != 0;
    const SmemLayout Lk = smem_layout(ka.M, ka.G, ka.P, ka.T, ka.S, gg);
    const int variant = (full ? 4 : 0) | (gg ? 2 : 0) | (legacy ? 1 : 0);
    switch (variant) {
        case 0: rc = launch_sim<false, false, false>(ka, Lk.total, st); break;
        case 1: rc = launch_sim<false, false, true>(ka, Lk.total, st); break;
        case 2: rc = launch_sim<false, true, false>(ka, Lk.total, st); break;
        case 3: rc = launch_sim<false, true, true>(ka, Lk.total, st); break;
        case 4: rc = launch_sim<true, false, false>(ka, Lk.total, st); break;
        case 5: rc = launch_sim<true, false, true>(ka, Lk.total, st); break;
        case 6: rc = launch_sim<true, true, false>(ka, Lk.total, st); break;
        default: rc = launch_sim<true, true, true>(ka, Lk.total, st); break;
    }
    if (rc) return rc;

    const int threads = 128;
    finalize_kernel<<<(B + threads - 1) / threads, threads, 0, st>>>(
        B, ka.M, plan->num_leaves, plan->leaf_merges, ka.leaf_sums, model_hist,
        out->model_num_good, out->model_num_requests, out->good_total, out->latency_sum,
        out->status);
    MMS_CUDA(cudaGetLastError());
    return MMS_OK;
}

}  // extern "C"
