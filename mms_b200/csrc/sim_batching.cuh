// sim_batching.cuh — the batching simulator.
//
// Restates simulate_requests_mixed_batching
// (alpa_serve/simulator/controller.py:630-798; pure Python in the reference:
// closures, list queues and heapq).  Requests wait in one FIFO queue per
// MODEL; a group serves, when its first stage frees up, the model whose
// oldest queued request arrived first, batching as many of that model's
// queued requests as still meet the head request's deadline.
//
// A model's queue always holds a run of consecutive requests of that model,
// so it is kept as (head index, length) over a per-trace linked list
// next_same[i] = next request with the model of request i; nothing is stored
// per queued request.  The heap of (time, group) events, the queues and the
// clocks are lane-private shared memory, [entry][lane].
//
// Like the unbatched path, the trace is cut into chunks that are simulated
// speculatively at the same time (idle start, a run-in, then the chunk) and
// stitched exactly afterwards (batch_chain_kernel: a chunk is kept if the state
// it started from is equivalent to the state the chunk before it ended in —
// batch_states_equivalent — and re-simulated from the true state otherwise).
// A request that is still queued at a chunk boundary is served by the NEXT
// chunk's run; a speculative run does not write the outputs of such carried
// requests itself (a wrong guess would clobber what the chunk before it
// wrote) but lists them, and the chain kernel applies the list when it
// accepts the chunk.
//
// Two forms of the speculative pass.  batch_simd_kernel runs 32 candidates per
// warp, in step over the arrivals of one chunk; the candidates' tables are
// read from global memory (transposed so that a warp's loads coalesce) and the
// counters are added to global memory without a return value, which leaves
// shared memory to the mutable state alone (clocks, heap, queues: about 1.4 KB
// per candidate).  batch_stream_kernel (one candidate per warp) serves batches
// too small to fill warps.  The repairs — batch_repair_kernel, batch_chain_kernel
// — run one chunk or candidate per warp: what they re-simulate is a dependent
// chain whose latency counts, and a lone lane gets through it fastest.  All of
// them work on the same helpers, templated on the number of lanes L a block
// interleaves.
#pragma once
#include "sim_core.cuh"

namespace mms {

struct BatchArgs {
    const double *arrivals;
    const int32_t *model_ids;
    const float *slos;
    const int32_t *next_same;     // [N]
    int64_t N;
    int32_t B, M, G, P, T, S, C, NB, H;
    int32_t batch_sizes[8];
    int32_t batch_cols[8];        // log2 of the batch size: the column the reference reads
    const uint16_t *model_off;    // [B][M+1]
    const uint32_t *model_rep;    // [B][P]   group | first slot<<8 | stages<<16 | column<<24
    const uint16_t *group_off;    // [B][G+1]
    const uint16_t *group_mod;    // [B][P]   models of each group, ascending
    const uint32_t *group_cfg;    // [B][G]   first slot | stages<<8 | column<<16
    const float *latency;         // [M][C][S][NB]
    int64_t latency_stride;
    int32_t lanes;                // candidates interleaved in one block's shared memory: 32
                                  //   (a warp of candidates) or 1 (one candidate per warp)
    double *finish;               // [B][N]
    uint8_t *good;                // [B][N]
    int32_t *model_num_requests;  // [B][M]
    int32_t *model_num_good;      // [B][M]
    int32_t *group_num_requests;  // [B][G]
    int32_t *group_num_good;      // [B][G]
    uint32_t *status;             // [B]
    // time-parallel execution
    int32_t K;                    // chunks
    int32_t chunk_len;            // arrivals per chunk (the last one takes the rest)
    int32_t warmup;               // run-in arrivals of a speculative chunk
    const int32_t *unsorted;      // != 0: arrival times not sorted / not finite -> one chunk
    unsigned char *snap_start;    // [K][B][state_bytes]: state a speculative chunk started from
    unsigned char *snap_end;      // [K][B][state_bytes]: state after the chunk's last arrival
    uint32_t *chunk_counters;     // [K][B][2M + 2G]
    unsigned char *carry;         // [K][B][carry_bytes]: outputs of carried requests
    int32_t *resimulated;         // [B] or null: chunks the chain kernel re-simulated
    // repair rounds between the speculative pass and the chain kernel
    uint32_t *work_count;         // [rounds]
    uint32_t *work_items;         // [K * B]: chunk * B + candidate
    int32_t round;
    // the candidates' tables as batch_simd_kernel reads them: checked, transposed to
    // [entry][Bp] (Bp = B rounded up to 32), built by batch_tables_kernel
    int32_t Bp;
    uint32_t *t_mrep;             // [P][Bp]
    uint32_t *t_gcfg;             // [G][Bp]
    uint16_t *t_moff;             // [M+1][Bp]
    uint16_t *t_goff;             // [G+1][Bp]
    uint16_t *t_gmod;             // [P][Bp]
    uint32_t *t_status;           // [Bp]: MMS_STATUS_BAD_INDEX where a table index was bad
};

constexpr int kMaxCarry = 120;    // carried requests a speculative chunk may list
constexpr int kBatchBlocksPerSm = 16;   // register budget of the batching kernels: 128 per thread

// Bytes of one saved state: clocks f64[T], idle f64[G], heap times f64[H],
// heap groups u32[H], queue heads i32[M], queue lengths i32[M], heap size.
__host__ __device__ inline size_t batch_state_bytes(int M, int G, int T, int H)
{
    return (8 * (size_t)(T + G + H) + 4 * (size_t)(H + 2 * M) + 8 + 15) & ~(size_t)15;
}

// Bytes of one carry list: count u32 (0xFFFFFFFF = overflowed), the status
// word of the chunk's speculative run, pad, then kMaxCarry x (finish f64) and
// kMaxCarry x (request i32 | good << 31).
__host__ __device__ inline size_t batch_carry_bytes()
{
    return 16 + (size_t)kMaxCarry * 12 + 8;
}

struct BatchSmem {
    size_t clocks, idle, heap_t, qhead, qlen, heap_g, counters, model_rep, group_cfg,
        model_off, group_off, group_mod, total;
};

// Shared memory of a block that interleaves L lanes.  L == 1: everything a
// candidate needs (state, counters, tables).  L == 32: the mutable state only
// (clocks, heap, queues; a group's idle time IS the clock of its first stage —
// controller.py:727 stores tmp[0] in both — and is not kept twice).
__host__ __device__ inline BatchSmem batch_smem(int M, int G, int P, int T, int H, int L)
{
    BatchSmem S;
    size_t off = 0;
    S.clocks = off;    off += sizeof(double) * (size_t)T * L;
    S.idle = off;      off += L == 1 ? sizeof(double) * (size_t)G : 0;
    S.heap_t = off;    off += sizeof(double) * (size_t)H * L;
    S.qhead = off;     off += sizeof(int32_t) * (size_t)M * L;
    S.qlen = off;      off += sizeof(int32_t) * (size_t)M * L;
    S.heap_g = off;    off += (L == 1 ? sizeof(uint32_t) : sizeof(uint8_t)) * (size_t)H * L;
    off = (off + 3) & ~(size_t)3;
    S.counters = off;  off += L == 1 ? sizeof(uint32_t) * (size_t)(2 * M + 2 * G) : 0;
    S.model_rep = off; off += L == 1 ? sizeof(uint32_t) * (size_t)P : 0;
    S.group_cfg = off; off += L == 1 ? sizeof(uint32_t) * (size_t)G : 0;
    S.model_off = off; off += L == 1 ? sizeof(uint16_t) * (size_t)(M + 1) : 0;
    S.group_off = off; off += L == 1 ? sizeof(uint16_t) * (size_t)(G + 1) : 0;
    S.group_mod = off; off += L == 1 ? sizeof(uint16_t) * (size_t)P : 0;
    S.total = (off + 15) & ~(size_t)15;
    return S;
}

// One candidate's state; the shared-memory members are element offsets (lane
// included), entries L elements apart.
struct BLane {
    uint32_t clk, idle, heap_t, heap_g, qhead, qlen;
    uint32_t counters;                   // L == 1: [2M + 2G] in shared memory
    uint32_t mrep, gcfg, moff, goff, gmod;   // L == 1: the tables in shared memory
    const uint32_t *g_mrep, *g_gcfg;     // L == 32: the transposed tables, at this candidate
    const uint16_t *g_moff, *g_goff, *g_gmod;
    uint32_t *g_counters;                // L == 32: this run's [2M + 2G] counters in global memory
    uint32_t heap_n, status;
    const float *lat;
    double *finish;
    uint8_t *good;
    // where outputs go: requests >= own_begin are written directly; older ones (carried over a
    // chunk boundary) only when `direct`, else they are appended to the carry list
    int32_t own_begin;
    bool direct, record;
    uint32_t carry_n;
    double *carry_fin;
    uint32_t *carry_req;
};

// Counter c of the run: [0, M) requests per model, [M, 2M) good per model,
// [2M, 2M + G) requests per group, then good per group.
template <int L>
__device__ __forceinline__ void count_add(const BatchArgs &, BLane &ln, uint32_t c, uint32_t v)
{
    if constexpr (L == 1) SM_U32(ln.counters + c) += v;
    else if (ln.record) atomicAdd(ln.g_counters + c, v);      // no return value: fire and forget
}

template <int L>
__device__ __forceinline__ uint32_t tab_mrep(const BatchArgs &a, const BLane &ln, uint32_t e)
{
    if constexpr (L == 1) return SM_U32(ln.mrep + e);
    else return __ldg(ln.g_mrep + (size_t)e * a.Bp);
}
template <int L>
__device__ __forceinline__ uint32_t tab_gcfg(const BatchArgs &a, const BLane &ln, uint32_t g)
{
    if constexpr (L == 1) return SM_U32(ln.gcfg + g);
    else return __ldg(ln.g_gcfg + (size_t)g * a.Bp);
}
template <int L>
__device__ __forceinline__ uint32_t tab_moff(const BatchArgs &a, const BLane &ln, uint32_t m)
{
    if constexpr (L == 1) return SM_U16(ln.moff + m);
    else return __ldg(ln.g_moff + (size_t)m * a.Bp);
}
template <int L>
__device__ __forceinline__ uint32_t tab_goff(const BatchArgs &a, const BLane &ln, uint32_t g)
{
    if constexpr (L == 1) return SM_U16(ln.goff + g);
    else return __ldg(ln.g_goff + (size_t)g * a.Bp);
}
template <int L>
__device__ __forceinline__ uint32_t tab_gmod(const BatchArgs &a, const BLane &ln, uint32_t e)
{
    if constexpr (L == 1) return SM_U16(ln.gmod + e);
    else return __ldg(ln.g_gmod + (size_t)e * a.Bp);
}
template <int L>
__device__ __forceinline__ uint32_t heap_group(const BLane &ln, uint32_t h)
{
    if constexpr (L == 1) return SM_U32(ln.heap_g + h);
    else return smem[ln.heap_g + h * L];
}
template <int L>
__device__ __forceinline__ void heap_group_set(const BLane &ln, uint32_t h, uint32_t g)
{
    if constexpr (L == 1) SM_U32(ln.heap_g + h) = g;
    else smem[ln.heap_g + h * L] = (uint8_t)g;
}

// Output of request r.
__device__ inline void put(BLane &ln, int32_t r, double fin, bool good)
{
    if (!ln.record) return;
    if (ln.direct || r >= ln.own_begin) {
        ln.finish[r] = fin;
        ln.good[r] = good ? 1 : 0;
    } else if (ln.carry_n < (uint32_t)kMaxCarry) {
        ln.carry_fin[ln.carry_n] = fin;
        ln.carry_req[ln.carry_n] = (uint32_t)r | (good ? 0x80000000u : 0u);
        ++ln.carry_n;
    } else {
        ln.carry_n = 0xFFFFFFFFu;          // too many: the chain kernel re-simulates the chunk
    }
}

// (time, group) ordered like the Python tuples the reference pushes (:728).
__device__ inline bool event_less(double ta, uint32_t ga, double tb, uint32_t gb)
{
    return ta < tb || (ta == tb && ga < gb);
}

template <int L>
__device__ inline void heap_push(const BatchArgs &a, BLane &ln, double t, uint32_t g)
{
    if (ln.heap_n >= (uint32_t)a.H) { ln.status |= MMS_STATUS_HEAP_OVERFLOW; return; }
    uint32_t i = ln.heap_n++;
    while (i > 0) {
        const uint32_t p = (i - 1) >> 1;
        const double tp = SM_F64(ln.heap_t + p * L);
        const uint32_t gp = heap_group<L>(ln, p);
        if (!event_less(t, g, tp, gp)) break;
        SM_F64(ln.heap_t + i * L) = tp;
        heap_group_set<L>(ln, i, gp);
        i = p;
    }
    SM_F64(ln.heap_t + i * L) = t;
    heap_group_set<L>(ln, i, g);
}

template <int L>
__device__ inline void heap_pop(const BatchArgs &, BLane &ln, double &t, uint32_t &g)
{
    t = SM_F64(ln.heap_t);
    g = heap_group<L>(ln, 0);
    const uint32_t n = --ln.heap_n;
    if (n == 0) return;
    const double te = SM_F64(ln.heap_t + n * L);
    const uint32_t ge = heap_group<L>(ln, n);
    uint32_t i = 0;
    for (;;) {
        uint32_t c = 2 * i + 1;
        if (c >= n) break;
        double tc = SM_F64(ln.heap_t + c * L);
        uint32_t gc = heap_group<L>(ln, c);
        if (c + 1 < n) {
            const double tr = SM_F64(ln.heap_t + (c + 1) * L);
            const uint32_t gr = heap_group<L>(ln, c + 1);
            if (event_less(tr, gr, tc, gc)) { c += 1; tc = tr; gc = gr; }
        }
        if (!event_less(tc, gc, te, ge)) break;
        SM_F64(ln.heap_t + i * L) = tc;
        heap_group_set<L>(ln, i, gc);
        i = c;
    }
    SM_F64(ln.heap_t + i * L) = te;
    heap_group_set<L>(ln, i, ge);
}

// select_model, :654-664: the group's model whose queue head arrived first.
template <int L>
__device__ inline int32_t pick_model(const BatchArgs &a, const BLane &ln, uint32_t g)
{
    const uint32_t lo = tab_goff<L>(a, ln, g), hi = tab_goff<L>(a, ln, g + 1);
    double first = kInf;
    int32_t pick = -1;
    for (uint32_t e = lo; e < hi; ++e) {
        const uint32_t m = tab_gmod<L>(a, ln, e);
        if ((int32_t)SM_U32(ln.qlen + m * L) > 0) {
            const double ts = a.arrivals[(int32_t)SM_U32(ln.qhead + m * L)];
            if (ts < first) { first = ts; pick = (int32_t)m; }
        }
    }
    return pick;
}

// check_slo, :666-672.
template <int L>
__device__ inline bool meets_deadline(const BatchArgs &a, const BLane &ln, double ts, uint32_t m,
                                      uint32_t slot, uint32_t ns, uint32_t col, int bcol,
                                      double deadline)
{
    const float *lat = ln.lat + (((size_t)m * a.C + col) * a.S) * a.NB + bcol;
    double t = ts;
    for (uint32_t k = 0; k < ns; ++k)
        t = fmax(SM_F64(ln.clk + (slot + k) * L), t) + (double)__ldg(lat + (size_t)k * a.NB);
    return t + kOverhead <= deadline;
}

template <int L>
__device__ inline int32_t queue_pop(const BatchArgs &a, BLane &ln, uint32_t m)
{
    const int32_t r = (int32_t)SM_U32(ln.qhead + m * L);
    SM_U32(ln.qhead + m * L) = (uint32_t)a.next_same[r];
    SM_U32(ln.qlen + m * L) -= 1;
    return r;
}

// The head request `head` of model m's queue can be served by group g at time
// ts: grows the batch while the HEAD's deadline still holds (:693-702),
// dispatches it (:715-725: overhead first, then the stages; clocks move to the
// new times), and books the group's next idle time and the counters (:727-732).
template <int L>
__device__ inline void dispatch_batch(const BatchArgs &a, BLane &ln, double ts, uint32_t m,
                                      uint32_t g, uint32_t cfg, int32_t head)
{
    const uint32_t slot = cfg & 0xFFu, ns = (cfg >> 8) & 0xFFu, col = cfg >> 16;
    const double deadline = a.arrivals[head] + (double)a.slos[head];
    int32_t bs = 1, bcol = a.batch_cols[0];
    for (int j = 1; j < a.NB; ++j) {
        if (a.batch_sizes[j] - 1 > (int32_t)SM_U32(ln.qlen + m * L)) break;
        if (!meets_deadline<L>(a, ln, ts, m, slot, ns, col, a.batch_cols[j], deadline)) break;
        bs = a.batch_sizes[j];
        bcol = a.batch_cols[j];
    }
    const float *lat = ln.lat + (((size_t)m * a.C + col) * a.S) * a.NB + bcol;
    double t = ts + kOverhead, t_first = 0.0;
    for (uint32_t k = 0; k < ns; ++k) {
        t = fmax(t, SM_F64(ln.clk + (slot + k) * L)) + (double)__ldg(lat + (size_t)k * a.NB);
        SM_F64(ln.clk + (slot + k) * L) = t;   // each stage reads only its own clock
        if (k == 0) t_first = t;
    }
    put(ln, head, t, true);
    for (int32_t k = 1; k < bs; ++k) {
        const int32_t r = queue_pop<L>(a, ln, m);
        put(ln, r, t, true);
    }
    if constexpr (L == 1) SM_F64(ln.idle + g) = t_first;    // L == 32: it is clk[slot]
    heap_push<L>(a, ln, t_first, g);
    count_add<L>(a, ln, 2 * a.M + g, (uint32_t)bs);
    count_add<L>(a, ln, 2 * a.M + a.G + g, (uint32_t)bs);
    count_add<L>(a, ln, a.M + m, (uint32_t)bs);
}

// handle_batched_requests with get_max_batch_under_slo, :674-732.  The
// reference recurses when a model's whole queue was dropped; the loop is the
// same tail call.
template <int L>
__device__ inline void serve_group(const BatchArgs &a, BLane &ln, double ts, int32_t m_in,
                                   uint32_t g)
{
    const uint32_t cfg = tab_gcfg<L>(a, ln, g);
    const uint32_t slot = cfg & 0xFFu, ns = (cfg >> 8) & 0xFFu, col = cfg >> 16;
    int32_t m = m_in;
    while (m >= 0) {
        // :677-686 drop queue heads that cannot make their deadline even alone
        int32_t head = -1;
        while ((int32_t)SM_U32(ln.qlen + m * L) > 0) {
            const int32_t r = queue_pop<L>(a, ln, m);
            const double dl = a.arrivals[r] + (double)a.slos[r];
            if (meets_deadline<L>(a, ln, ts, m, slot, ns, col, a.batch_cols[0], dl)) { head = r; break; }
            count_add<L>(a, ln, 2 * a.M + g, 1u);
            put(ln, r, a.arrivals[r], false);
        }
        if (head < 0) { m = pick_model<L>(a, ln, g); continue; }      // :709-713
        dispatch_batch<L>(a, ln, ts, (uint32_t)m, g, cfg, head);
        return;
    }
}

// This lane's view of candidate b with ONE lane per block: offsets of the
// state, and the candidate's tables copied on chip, every index checked (a
// bad one is reported in ln.status).
__device__ inline void batch_setup(const BatchArgs &a, BLane &ln, int64_t b)
{
    const BatchSmem S = batch_smem(a.M, a.G, a.P, a.T, a.H, 1);
    ln.clk = (uint32_t)(S.clocks / 8);
    ln.idle = (uint32_t)(S.idle / 8);
    ln.heap_t = (uint32_t)(S.heap_t / 8);
    ln.heap_g = (uint32_t)(S.heap_g / 4);
    ln.qhead = (uint32_t)(S.qhead / 4);
    ln.qlen = (uint32_t)(S.qlen / 4);
    ln.counters = (uint32_t)(S.counters / 4);
    ln.mrep = (uint32_t)(S.model_rep / 4);
    ln.gcfg = (uint32_t)(S.group_cfg / 4);
    ln.moff = (uint32_t)(S.model_off / 2);
    ln.goff = (uint32_t)(S.group_off / 2);
    ln.gmod = (uint32_t)(S.group_mod / 2);
    ln.g_mrep = ln.g_gcfg = nullptr;
    ln.g_moff = ln.g_goff = ln.g_gmod = nullptr;
    ln.g_counters = nullptr;
    ln.heap_n = 0;
    ln.status = 0;
    ln.lat = a.latency + (size_t)b * a.latency_stride;
    ln.finish = a.finish + (size_t)b * a.N;
    ln.good = a.good + (size_t)b * a.N;
    ln.own_begin = 0; ln.direct = true; ln.record = true;
    ln.carry_n = 0; ln.carry_fin = nullptr; ln.carry_req = nullptr;

    for (int g = 0; g < a.G; ++g) {
        uint32_t cfg = a.group_cfg[(size_t)b * a.G + g];
        const uint32_t slot = cfg & 0xFFu, ns = (cfg >> 8) & 0xFFu;
        if (slot + ns > (uint32_t)a.T || ns > (uint32_t)a.S || (cfg >> 16) >= (uint32_t)a.C) {
            ln.status |= MMS_STATUS_BAD_INDEX;
            cfg = 0;
        }
        SM_U32(ln.gcfg + g) = cfg;
    }
    uint32_t prev = 0;
    for (int m = 0; m <= a.M; ++m) {
        uint32_t o = a.model_off[(size_t)b * (a.M + 1) + m];
        if (o < prev || o > (uint32_t)a.P) { ln.status |= MMS_STATUS_BAD_INDEX; o = prev; }
        SM_U16(ln.moff + m) = (uint16_t)o;
        prev = o;
    }
    for (uint32_t e = 0; e < (uint32_t)a.P; ++e) {
        uint32_t ent = e < prev ? a.model_rep[(size_t)b * a.P + e] : 0u;
        if (e < prev) {
            const uint32_t g = ent & 0xFFu;
            if (g >= (uint32_t)a.G || ((ent >> 8) & 0xFFFFu) != (SM_U32(ln.gcfg + g) & 0xFFFFu))
                ln.status |= MMS_STATUS_BAD_INDEX;
        }
        SM_U32(ln.mrep + e) = ent;
    }
    prev = 0;
    for (int g = 0; g <= a.G; ++g) {
        uint32_t o = a.group_off[(size_t)b * (a.G + 1) + g];
        if (o < prev || o > (uint32_t)a.P) { ln.status |= MMS_STATUS_BAD_INDEX; o = prev; }
        SM_U16(ln.goff + g) = (uint16_t)o;
        prev = o;
    }
    for (uint32_t e = 0; e < (uint32_t)a.P; ++e) {
        uint32_t m = e < prev ? a.group_mod[(size_t)b * a.P + e] : 0u;
        if (m >= (uint32_t)a.M) { ln.status |= MMS_STATUS_BAD_INDEX; m = 0; }
        SM_U16(ln.gmod + e) = (uint16_t)m;
    }
}

// The same checks, one thread per candidate, writing the tables transposed
// ([entry][Bp]) for batch_simd_kernel.
__global__ void batch_tables_kernel(const BatchArgs a)
{
    const int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= a.Bp) return;
    const size_t Bp = (size_t)a.Bp;
    uint32_t status = 0;
    if (b >= a.B) {                         // padding lanes: empty tables
        for (int g = 0; g < a.G; ++g) a.t_gcfg[g * Bp + b] = 0;
        for (int m = 0; m <= a.M; ++m) a.t_moff[m * Bp + b] = 0;
        for (int g = 0; g <= a.G; ++g) a.t_goff[g * Bp + b] = 0;
        for (int e = 0; e < a.P; ++e) { a.t_mrep[e * Bp + b] = 0; a.t_gmod[e * Bp + b] = 0; }
        a.t_status[b] = 0;
        return;
    }
    for (int g = 0; g < a.G; ++g) {
        uint32_t cfg = a.group_cfg[(size_t)b * a.G + g];
        const uint32_t slot = cfg & 0xFFu, ns = (cfg >> 8) & 0xFFu;
        if (slot + ns > (uint32_t)a.T || ns > (uint32_t)a.S || (cfg >> 16) >= (uint32_t)a.C) {
            status |= MMS_STATUS_BAD_INDEX;
            cfg = 0;
        }
        a.t_gcfg[g * Bp + b] = cfg;
    }
    uint32_t prev = 0;
    for (int m = 0; m <= a.M; ++m) {
        uint32_t o = a.model_off[(size_t)b * (a.M + 1) + m];
        if (o < prev || o > (uint32_t)a.P) { status |= MMS_STATUS_BAD_INDEX; o = prev; }
        a.t_moff[m * Bp + b] = (uint16_t)o;
        prev = o;
    }
    for (uint32_t e = 0; e < (uint32_t)a.P; ++e) {
        uint32_t ent = e < prev ? a.model_rep[(size_t)b * a.P + e] : 0u;
        if (e < prev) {
            const uint32_t g = ent & 0xFFu;
            if (g >= (uint32_t)a.G || ((ent >> 8) & 0xFFFFu) != (a.t_gcfg[g * Bp + b] & 0xFFFFu))
                status |= MMS_STATUS_BAD_INDEX;
        }
        a.t_mrep[e * Bp + b] = ent;
    }
    prev = 0;
    for (int g = 0; g <= a.G; ++g) {
        uint32_t o = a.group_off[(size_t)b * (a.G + 1) + g];
        if (o < prev || o > (uint32_t)a.P) { status |= MMS_STATUS_BAD_INDEX; o = prev; }
        a.t_goff[g * Bp + b] = (uint16_t)o;
        prev = o;
    }
    for (uint32_t e = 0; e < (uint32_t)a.P; ++e) {
        uint32_t m = e < prev ? a.group_mod[(size_t)b * a.P + e] : 0u;
        if (m >= (uint32_t)a.M) { status |= MMS_STATUS_BAD_INDEX; m = 0; }
        a.t_gmod[e * Bp + b] = (uint16_t)m;
    }
    a.t_status[b] = status;
}

__device__ inline void batch_zero_counters(const BatchArgs &a, BLane &ln)
{
    for (int c = 0; c < 2 * a.M + 2 * a.G; ++c) SM_U32(ln.counters + c) = 0;
}

// Idle clocks, empty queues, empty heap.
template <int L>
__device__ inline void batch_zero_state(const BatchArgs &a, BLane &ln)
{
    for (int t = 0; t < a.T; ++t) SM_F64(ln.clk + t * L) = 0.0;
    if constexpr (L == 1)
        for (int g = 0; g < a.G; ++g) SM_F64(ln.idle + g) = 0.0;
    for (int m = 0; m < a.M; ++m) { SM_U32(ln.qhead + m * L) = 0; SM_U32(ln.qlen + m * L) = 0; }
    ln.heap_n = 0;
}

// :759-773 for arrival i of model m with replicas [lo, hi): the replica whose
// last-stage clock is strictly smallest; the request joins its MODEL's queue.
// Returns the chosen replica entry, `found` false when no replica qualifies.
template <int L>
__device__ inline uint32_t choose_and_enqueue(const BatchArgs &a, BLane &ln, int64_t i, int32_t m,
                                              uint32_t lo, uint32_t hi, bool &found)
{
    double best = kInf;
    uint32_t pick = 0;
    found = false;
    for (uint32_t e = lo; e < hi; ++e) {
        const uint32_t ent = tab_mrep<L>(a, ln, e);
        const uint32_t last = ((ent >> 8) & 0xFFu) + ((ent >> 16) & 0xFFu) - 1;
        const double c = SM_F64(ln.clk + last * L);
        if (c < best) { best = c; pick = ent; found = true; }
    }
    if ((int32_t)SM_U32(ln.qlen + m * L) == 0) SM_U32(ln.qhead + m * L) = (uint32_t)i;
    SM_U32(ln.qlen + m * L) += 1;
    count_add<L>(a, ln, (uint32_t)m, 1u);
    return pick;
}

// Arrival i, :736-778.
template <int L>
__device__ inline void batch_arrival(const BatchArgs &a, BLane &ln, int64_t i)
{
    const double ts = a.arrivals[i];
    // :739-744 groups whose first stage became free before this arrival
    while (ln.heap_n > 0 && SM_F64(ln.heap_t) <= ts) {
        double te; uint32_t ge;
        heap_pop<L>(a, ln, te, ge);
        const int32_t pm = pick_model<L>(a, ln, ge);
        if (pm < 0) break;                     // the reference breaks here, not continues
        serve_group<L>(a, ln, te, pm, ge);
    }
    int32_t m = a.model_ids[i];
    if (m >= a.M) { ln.status |= MMS_STATUS_BAD_INDEX; m = -1; }
    uint32_t lo = 0, hi = 0;
    if (m >= 0) { lo = tab_moff<L>(a, ln, m); hi = tab_moff<L>(a, ln, m + 1); }
    if (lo == hi) {                            // :748-757 unknown model or no replica
        put(ln, (int32_t)i, ts, false);
        return;
    }
    bool found;
    const uint32_t pick = choose_and_enqueue<L>(a, ln, i, m, lo, hi, found);
    const uint32_t g = pick & 0xFFu;
    // a group's idle time is the clock of its first stage (kept twice only with L == 1)
    const double idle = L == 1 ? SM_F64(ln.idle + g) : SM_F64(ln.clk + ((pick >> 8) & 0xFFu) * L);
    if (found && ts >= idle)                   // :776-778
        serve_group<L>(a, ln, ts, m, g);
}

// After the last arrival, :781-790.
template <int L>
__device__ inline void batch_drain(const BatchArgs &a, BLane &ln)
{
    while (ln.heap_n > 0) {
        double te; uint32_t ge;
        heap_pop<L>(a, ln, te, ge);
        const int32_t pm = pick_model<L>(a, ln, ge);
        if (pm < 0) continue;
        serve_group<L>(a, ln, te, pm, ge);
    }
    for (int m = 0; m < a.M; ++m)
        if ((int32_t)SM_U32(ln.qlen + m * L) != 0) ln.status |= MMS_STATUS_QUEUE_LEFT;
}

// A saved state, see batch_state_bytes.
struct StateView {
    double *clk, *idle, *heap_t;
    uint32_t *heap_g;
    int32_t *qhead, *qlen;
    uint32_t *heap_n;
};

__device__ inline StateView state_view(const BatchArgs &a, unsigned char *p)
{
    StateView v;
    v.clk = reinterpret_cast<double *>(p);
    v.idle = v.clk + a.T;
    v.heap_t = v.idle + a.G;
    v.heap_g = reinterpret_cast<uint32_t *>(v.heap_t + a.H);
    v.qhead = reinterpret_cast<int32_t *>(v.heap_g + a.H);
    v.qlen = v.qhead + a.M;
    v.heap_n = reinterpret_cast<uint32_t *>(v.qlen + a.M);
    return v;
}

template <int L>
__device__ inline void state_save(const BatchArgs &a, const BLane &ln, unsigned char *p)
{
    const StateView v = state_view(a, p);
    for (int t = 0; t < a.T; ++t) v.clk[t] = SM_F64(ln.clk + t * L);
    for (int g = 0; g < a.G; ++g) {
        if constexpr (L == 1) {
            v.idle[g] = SM_F64(ln.idle + g);
        } else {        // the clock of the group's first stage; 0 for a row of padding
            const uint32_t cfg = tab_gcfg<L>(a, ln, g);
            v.idle[g] = ((cfg >> 8) & 0xFFu) ? SM_F64(ln.clk + (cfg & 0xFFu) * L) : 0.0;
        }
    }
    for (uint32_t h = 0; h < ln.heap_n; ++h) {
        v.heap_t[h] = SM_F64(ln.heap_t + h * L);
        v.heap_g[h] = heap_group<L>(ln, h);
    }
    for (int m = 0; m < a.M; ++m) {
        v.qhead[m] = (int32_t)SM_U32(ln.qhead + m * L);
        v.qlen[m] = (int32_t)SM_U32(ln.qlen + m * L);
    }
    *v.heap_n = ln.heap_n;
}

__device__ inline void state_load(const BatchArgs &a, BLane &ln, unsigned char *p)
{
    const StateView v = state_view(a, p);
    for (int t = 0; t < a.T; ++t) SM_F64(ln.clk + t) = v.clk[t];
    for (int g = 0; g < a.G; ++g) SM_F64(ln.idle + g) = v.idle[g];
    ln.heap_n = *v.heap_n;
    for (uint32_t h = 0; h < ln.heap_n; ++h) {
        SM_F64(ln.heap_t + h) = v.heap_t[h];
        SM_U32(ln.heap_g + h) = v.heap_g[h];
    }
    for (int m = 0; m < a.M; ++m) {
        SM_U32(ln.qhead + m) = (uint32_t)v.qhead[m];
        SM_U32(ln.qlen + m) = (uint32_t)v.qlen[m];
    }
}

// The state X on chip (true) and a saved state Y, both taken just before the
// arrival at time tau, lead to identical futures when
//  - every queue has the same length and, if not empty, the same head (a
//    queue is a run of consecutive requests of its model);
//  - the heaps hold the same events: compared as arrays, which is stricter
//    than as sets (two runs that pushed and popped the same events in the
//    same order have identical arrays);
//  - a group's idle time is equal in both or <= tau in both (it is only
//    compared with arrival times >= tau, :776);
//  - every clock is equal in both or < theta in both, theta = the earlier of
//    tau and the first pending event: a clock only ever enters max(clock, t)
//    with t an arrival time or a pending event's time (:669, :719);
//  - the last-stage clocks that differ (both < theta) of groups serving a
//    replicated model are in the same order (ties included) relative to all
//    such groups' last-stage clocks: dispatch compares them with '<' (:764).
// Sufficient, not necessary: a failed check only costs a re-simulation.
// X, Y: anything with heap_n(), heap_t(h), heap_g(h), qlen(m), qhead(m), idle(g),
// clk(t); moff(m) / mrep(e): the candidate's replica lists.
template <typename XS, typename YS, typename Moff, typename Mrep>
__device__ inline bool batch_equivalent(const BatchArgs &a, const XS &x, const YS &y, double tau,
                                        Moff moff, Mrep mrep)
{
    if (y.heap_n() != x.heap_n()) return false;
    double theta = tau;
    for (uint32_t h = 0; h < x.heap_n(); ++h) {
        const double t = x.heap_t(h);
        if (t != y.heap_t(h) || x.heap_g(h) != y.heap_g(h)) return false;
        if (t < theta) theta = t;
    }
    for (int m = 0; m < a.M; ++m) {
        const int32_t n = x.qlen(m);
        if (n != y.qlen(m)) return false;
        if (n > 0 && x.qhead(m) != y.qhead(m)) return false;
    }
    for (int g = 0; g < a.G; ++g) {
        const double u = x.idle(g), v = y.idle(g);
        if (!(u == v || (u <= tau && v <= tau))) return false;
    }
    for (int t = 0; t < a.T; ++t) {
        const double u = x.clk(t), v = y.clk(t);
        if (!(u == v || (u < theta && v < theta))) return false;
    }
    // order of differing last-stage clocks among groups that share a model
    for (int m = 0; m < a.M; ++m) {
        const uint32_t lo = moff(m), hi = moff(m + 1);
        for (uint32_t e = lo; e + 1 < hi; ++e) {
            const uint32_t eu = mrep(e);
            const uint32_t su = ((eu >> 8) & 0xFFu) + ((eu >> 16) & 0xFFu) - 1;
            const double xu = x.clk(su), yu = y.clk(su);
            for (uint32_t f = e + 1; f < hi; ++f) {
                const uint32_t ev = mrep(f);
                const uint32_t sv = ((ev >> 8) & 0xFFu) + ((ev >> 16) & 0xFFu) - 1;
                const double xv = x.clk(sv), yv = y.clk(sv);
                if ((xu < xv) != (yu < yv) || (xu > xv) != (yu > yv)) return false;
            }
        }
    }
    return true;
}

// A saved state as batch_equivalent reads it.
struct SavedState {
    StateView v;
    __device__ uint32_t heap_n() const { return *v.heap_n; }
    __device__ double heap_t(uint32_t h) const { return v.heap_t[h]; }
    __device__ uint32_t heap_g(uint32_t h) const { return v.heap_g[h]; }
    __device__ int32_t qlen(int m) const { return v.qlen[m]; }
    __device__ int32_t qhead(int m) const { return v.qhead[m]; }
    __device__ double idle(int g) const { return v.idle[g]; }
    __device__ double clk(int t) const { return v.clk[t]; }
};

// The state of a one-lane block on chip.
struct ChipState {
    const BLane &ln;
    __device__ uint32_t heap_n() const { return ln.heap_n; }
    __device__ double heap_t(uint32_t h) const { return SM_F64(ln.heap_t + h); }
    __device__ uint32_t heap_g(uint32_t h) const { return SM_U32(ln.heap_g + h); }
    __device__ int32_t qlen(int m) const { return (int32_t)SM_U32(ln.qlen + m); }
    __device__ int32_t qhead(int m) const { return (int32_t)SM_U32(ln.qhead + m); }
    __device__ double idle(int g) const { return SM_F64(ln.idle + g); }
    __device__ double clk(int t) const { return SM_F64(ln.clk + t); }
};

__device__ inline bool batch_states_equivalent(const BatchArgs &a, const BLane &ln,
                                               unsigned char *saved, double tau)
{
    const ChipState x{ln};
    const SavedState y{state_view(a, saved)};
    return batch_equivalent(a, x, y, tau, [&](int m) { return (uint32_t)SM_U16(ln.moff + m); },
                            [&](uint32_t e) { return SM_U32(ln.mrep + e); });
}

__device__ inline void counters_store(const BatchArgs &a, const BLane &ln, uint32_t *dst)
{
    for (int c = 0; c < 2 * a.M + 2 * a.G; ++c) dst[c] = SM_U32(ln.counters + c);
}

// First arrival of chunk j (j == K: one past the last arrival).
__device__ inline int64_t chunk_first(const BatchArgs &a, int32_t j)
{
    const int64_t at = (int64_t)j * a.chunk_len;
    return j >= a.K || at > a.N ? a.N : at;
}

__device__ inline bool batch_can_chunk(const BatchArgs &a) { return a.K > 1 && *a.unsorted == 0; }

// One candidate per warp (thread 0 of the block alone, so that a candidate's
// branches are not serialised against 31 others'): one thread per (candidate,
// chunk).  Chunk 0 starts from the true (idle) state; the others start idle
// `warmup` arrivals early and store the state they have at their first arrival.
__global__ void __launch_bounds__(kLanes, kBatchBlocksPerSm)
batch_stream_kernel(const BatchArgs a)
{
    if (threadIdx.x != 0) return;
    const int64_t stream = blockIdx.x;
    if (stream >= (int64_t)a.B * a.K) return;
    const int32_t j = (int32_t)(stream / a.B);
    const int64_t b = stream % a.B;
    const bool chunked = batch_can_chunk(a);
    if (!chunked && j > 0) return;
    BLane ln;
    batch_setup(a, ln, b);
    batch_zero_state<1>(a, ln);
    batch_zero_counters(a, ln);
    const size_t sb = batch_state_bytes(a.M, a.G, a.T, a.H);
    const size_t cell = (size_t)j * a.B + b;
    const int64_t first = chunked ? chunk_first(a, j) : 0;
    const int64_t end = chunked ? chunk_first(a, j + 1) : a.N;
    if (!(ln.status & MMS_STATUS_BAD_INDEX)) {
        if (j > 0) {
            unsigned char *carry = a.carry + cell * batch_carry_bytes();
            ln.carry_fin = reinterpret_cast<double *>(carry + 16);
            ln.carry_req = reinterpret_cast<uint32_t *>(carry + 16 + (size_t)kMaxCarry * 8);
            ln.own_begin = (int32_t)first;
            ln.direct = false;
            ln.record = false;
            for (int64_t i = first - a.warmup > 0 ? first - a.warmup : 0; i < first; ++i)
                batch_arrival<1>(a, ln, i);
            ln.record = true;
            ln.status &= MMS_STATUS_BAD_INDEX;       // overflows of the run-in are not the chunk's
            batch_zero_counters(a, ln);
            state_save<1>(a, ln, a.snap_start + cell * sb);
        }
        for (int64_t i = first; i < end; ++i) batch_arrival<1>(a, ln, i);
        if (end == a.N) batch_drain<1>(a, ln);
        if (chunked) state_save<1>(a, ln, a.snap_end + cell * sb);
    }
    counters_store(a, ln, a.chunk_counters + cell * (size_t)(2 * a.M + 2 * a.G));
    if (chunked) {
        // the chain kernel decides whether this run, and with it its status word, counts
        uint32_t *hdr = reinterpret_cast<uint32_t *>(a.carry + cell * batch_carry_bytes());
        hdr[0] = ln.carry_n;
        hdr[1] = ln.status;
    } else if (ln.status) {
        atomicOr(&a.status[b], ln.status);
    }
}

// 32 candidates per warp, one block per (32 consecutive candidates, chunk); the
// counters of the chunk (a.chunk_counters) must be zero on entry.  The lanes go
// through the chunk's arrivals in step — the trace values are one broadcast
// load per warp — and each runs the sequential code for its candidate; where
// their control flow differs (events to pop, heads to drop, batch sizes,
// pipeline depths) the warp serialises, and it is whole again at the next
// arrival.  What this form shares with the one-candidate-per-warp kernels is
// every helper above; what differs is where tables and counters live.
__global__ void __launch_bounds__(kLanes)
batch_simd_kernel(const BatchArgs a)
{
    constexpr int L = kLanes;
    const int lane = threadIdx.x;
    const int32_t Bw = a.Bp / kLanes;
    const int32_t j = (int32_t)(blockIdx.x / Bw);
    const int64_t b = (int64_t)(blockIdx.x % Bw) * kLanes + lane;
    const bool chunked = batch_can_chunk(a);
    if (!chunked && j > 0) return;              // the whole block
    const BatchSmem S = batch_smem(a.M, a.G, a.P, a.T, a.H, L);
    BLane ln;
    ln.clk = (uint32_t)(S.clocks / 8) + lane;
    ln.heap_t = (uint32_t)(S.heap_t / 8) + lane;
    ln.heap_g = (uint32_t)S.heap_g + lane;           // bytes
    ln.qhead = (uint32_t)(S.qhead / 4) + lane;
    ln.qlen = (uint32_t)(S.qlen / 4) + lane;
    ln.idle = ln.counters = ln.mrep = ln.gcfg = ln.moff = ln.goff = ln.gmod = 0;
    const bool valid = b < a.B;
    const int64_t bb = valid ? b : 0;
    ln.g_mrep = a.t_mrep + bb; ln.g_gcfg = a.t_gcfg + bb;
    ln.g_moff = a.t_moff + bb; ln.g_goff = a.t_goff + bb; ln.g_gmod = a.t_gmod + bb;
    const size_t cell = (size_t)j * a.B + bb;
    ln.g_counters = a.chunk_counters + cell * (size_t)(2 * a.M + 2 * a.G);
    ln.heap_n = 0;
    ln.status = valid ? a.t_status[b] : 0;
    ln.lat = a.latency + (size_t)bb * a.latency_stride;
    ln.finish = a.finish + (size_t)bb * a.N;
    ln.good = a.good + (size_t)bb * a.N;
    ln.own_begin = 0; ln.direct = true; ln.record = true;
    ln.carry_n = 0; ln.carry_fin = nullptr; ln.carry_req = nullptr;
    batch_zero_state<L>(a, ln);
    // a lane simulates when it has a candidate and the candidate's tables are sound
    const bool run = valid && !(ln.status & MMS_STATUS_BAD_INDEX);

    const size_t sb = batch_state_bytes(a.M, a.G, a.T, a.H);
    const int64_t first = chunked ? chunk_first(a, j) : 0;
    const int64_t end = chunked ? chunk_first(a, j + 1) : a.N;
    if (j > 0) {
        unsigned char *carry = a.carry + cell * batch_carry_bytes();
        ln.carry_fin = reinterpret_cast<double *>(carry + 16);
        ln.carry_req = reinterpret_cast<uint32_t *>(carry + 16 + (size_t)kMaxCarry * 8);
        ln.own_begin = (int32_t)first;
        ln.direct = false;
        ln.record = false;                           // run-in
        for (int64_t i = first - a.warmup > 0 ? first - a.warmup : 0; i < first; ++i) {
            if (run) batch_arrival<L>(a, ln, i);
            __syncwarp();
        }
        ln.record = true;
        ln.status &= MMS_STATUS_BAD_INDEX;           // overflows of the run-in are not the chunk's
        if (run) state_save<L>(a, ln, a.snap_start + cell * sb);
    }
    for (int64_t i = first; i < end; ++i) {
        if (run) batch_arrival<L>(a, ln, i);
        __syncwarp();
    }
    if (run && end == a.N) batch_drain<L>(a, ln);
    if (!valid) return;
    if (chunked) {
        if (run) state_save<L>(a, ln, a.snap_end + cell * sb);
        // the chain kernel decides whether this run, and with it its status word, counts
        uint32_t *hdr = reinterpret_cast<uint32_t *>(a.carry + cell * batch_carry_bytes());
        hdr[0] = ln.carry_n;
        hdr[1] = ln.status;
    } else if (ln.status) {
        atomicOr(&a.status[b], ln.status);
    }
}

// Repair rounds.  One thread per (candidate, chunk j >= 1): does the state the
// chunk's stored run started from (snap_start[j]) continue the state the run
// of the chunk before it ended in (snap_end[j - 1])?  If not, that end state
// becomes the chunk's start state and the chunk goes on the round's work list.
// The end state may itself be wrong still (its chunk is on the list too);
// then the next round, or the chain kernel, catches what follows from it.
__global__ void batch_validate_kernel(const BatchArgs a)
{
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (!batch_can_chunk(a) || t >= (int64_t)a.B * (a.K - 1)) return;
    if (a.round > 0 && a.work_count[a.round - 1] == 0) return;      // nothing changed since
    const int32_t j = (int32_t)(t / a.B) + 1;
    const int64_t b = t % a.B;
    const int64_t first = chunk_first(a, j);
    if (first >= a.N) return;
    const size_t sb = batch_state_bytes(a.M, a.G, a.T, a.H);
    const size_t cell = (size_t)j * a.B + b;
    unsigned char *end_prev = a.snap_end + (cell - a.B) * sb;
    unsigned char *start = a.snap_start + cell * sb;
    const uint32_t *hdr_prev = reinterpret_cast<const uint32_t *>(a.carry + (cell - a.B) * batch_carry_bytes());
    // tables with a bad index: nothing was simulated, the chain kernel reports it
    if (hdr_prev[1] & MMS_STATUS_BAD_INDEX) return;
    const SavedState x{state_view(a, end_prev)}, y{state_view(a, start)};
    const uint16_t *moff = a.model_off + (size_t)b * (a.M + 1);
    const uint32_t *mrep = a.model_rep + (size_t)b * a.P;
    if (batch_equivalent(a, x, y, a.arrivals[first], [&](int m) { return (uint32_t)moff[m]; },
                         [&](uint32_t e) { return mrep[e]; }))
        return;
    // the heap is saved up to its size only: copy field by field
    const StateView src = x.v, dst = y.v;
    for (int k = 0; k < a.T; ++k) dst.clk[k] = src.clk[k];
    for (int g = 0; g < a.G; ++g) dst.idle[g] = src.idle[g];
    const uint32_t n = *src.heap_n;
    for (uint32_t h = 0; h < n && h < (uint32_t)a.H; ++h) { dst.heap_t[h] = src.heap_t[h]; dst.heap_g[h] = src.heap_g[h]; }
    for (int m = 0; m < a.M; ++m) { dst.qhead[m] = src.qhead[m]; dst.qlen[m] = src.qlen[m]; }
    *dst.heap_n = n;
    a.work_items[atomicAdd(&a.work_count[a.round], 1u)] = (uint32_t)((int64_t)j * a.B + b);
}

// One listed chunk per warp (thread 0 alone): re-simulated from the start state
// batch_validate_kernel copied in.  That state is not known to be the true one
// yet, so the outputs of carried requests are listed, not written, like in a
// speculative run.
__global__ void __launch_bounds__(kLanes, kBatchBlocksPerSm)
batch_repair_kernel(const BatchArgs a)
{
    if (threadIdx.x != 0 || !batch_can_chunk(a)) return;
    if (blockIdx.x >= a.work_count[a.round]) return;
    const uint32_t item = a.work_items[blockIdx.x];
    const int32_t j = (int32_t)(item / (uint32_t)a.B);
    const int64_t b = item % (uint32_t)a.B;
    BLane ln;
    batch_setup(a, ln, b);
    if (ln.status & MMS_STATUS_BAD_INDEX) return;
    const size_t sb = batch_state_bytes(a.M, a.G, a.T, a.H);
    const size_t cell = (size_t)j * a.B + b;
    const int64_t first = chunk_first(a, j), end = chunk_first(a, j + 1);
    unsigned char *carry = a.carry + cell * batch_carry_bytes();
    ln.carry_fin = reinterpret_cast<double *>(carry + 16);
    ln.carry_req = reinterpret_cast<uint32_t *>(carry + 16 + (size_t)kMaxCarry * 8);
    ln.own_begin = (int32_t)first;
    ln.direct = false;
    state_load(a, ln, a.snap_start + cell * sb);
    batch_zero_counters(a, ln);
    for (int64_t i = first; i < end; ++i) batch_arrival<1>(a, ln, i);
    if (end == a.N) batch_drain<1>(a, ln);
    state_save<1>(a, ln, a.snap_end + cell * sb);
    counters_store(a, ln, a.chunk_counters + cell * (size_t)(2 * a.M + 2 * a.G));
    uint32_t *hdr = reinterpret_cast<uint32_t *>(carry);
    hdr[0] = ln.carry_n;
    hdr[1] = ln.status;
    if (a.resimulated) atomicAdd(&a.resimulated[b], 1);
}

// One thread per candidate (one candidate per warp): walks the chunk
// boundaries in order; a chunk whose start state is equivalent to the true
// state is kept (and the outputs of the requests it carried over are
// written), any other is re-simulated from the true state.
__global__ void __launch_bounds__(kLanes, kBatchBlocksPerSm)
batch_chain_kernel(const BatchArgs a)
{
    if (threadIdx.x != 0) return;
    const int64_t b = blockIdx.x;
    if (b >= a.B || !batch_can_chunk(a)) return;
    BLane ln;
    batch_setup(a, ln, b);
    if (ln.status & MMS_STATUS_BAD_INDEX) {             // bad tables: nothing was simulated
        atomicOr(&a.status[b], ln.status);
        return;
    }
    const size_t sb = batch_state_bytes(a.M, a.G, a.T, a.H);
    const size_t n_counters = (size_t)(2 * a.M + 2 * a.G);
    state_load(a, ln, a.snap_end + (size_t)b * sb);     // chunk 0 ran from the true state
    uint32_t status = reinterpret_cast<const uint32_t *>(a.carry + (size_t)b * batch_carry_bytes())[1];
    int32_t redone = 0;
    for (int32_t j = 1; j < a.K; ++j) {
        const size_t cell = (size_t)j * a.B + b;
        const int64_t first = chunk_first(a, j), end = chunk_first(a, j + 1);
        if (first >= a.N) break;
        unsigned char *carry = a.carry + cell * batch_carry_bytes();
        const uint32_t carried = reinterpret_cast<const uint32_t *>(carry)[0];
        if (carried != 0xFFFFFFFFu &&
            batch_states_equivalent(a, ln, a.snap_start + cell * sb, a.arrivals[first])) {
            const double *fin = reinterpret_cast<const double *>(carry + 16);
            const uint32_t *req = reinterpret_cast<const uint32_t *>(carry + 16 + (size_t)kMaxCarry * 8);
            for (uint32_t k = 0; k < carried; ++k) {
                ln.finish[req[k] & 0x7FFFFFFFu] = fin[k];
                ln.good[req[k] & 0x7FFFFFFFu] = (uint8_t)(req[k] >> 31);
            }
            status |= reinterpret_cast<const uint32_t *>(carry)[1];
            state_load(a, ln, a.snap_end + cell * sb);
            continue;
        }
        ++redone;                          // the speculative run of chunk j is dropped, status and all
        batch_zero_counters(a, ln);
        ln.status = 0;
        for (int64_t i = first; i < end; ++i) batch_arrival<1>(a, ln, i);
        if (end == a.N) batch_drain<1>(a, ln);
        counters_store(a, ln, a.chunk_counters + cell * n_counters);
        status |= ln.status;
    }
    if (a.resimulated && redone) atomicAdd(&a.resimulated[b], redone);
    if (status) atomicOr(&a.status[b], status);
}

// Adds the per-chunk counters: one thread per (counter, candidate).
__global__ void batch_sum_kernel(const BatchArgs a)
{
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int n_counters = 2 * a.M + 2 * a.G;
    if (t >= (int64_t)a.B * n_counters) return;
    const int c = (int)(t % n_counters);
    const int64_t b = t / n_counters;
    const int32_t chunks = batch_can_chunk(a) ? a.K : 1;
    uint32_t v = 0;
    for (int32_t j = 0; j < chunks; ++j) v += a.chunk_counters[((size_t)j * a.B + b) * n_counters + c];
    if (c < a.M) a.model_num_requests[(size_t)b * a.M + c] = (int32_t)v;
    else if (c < 2 * a.M) a.model_num_good[(size_t)b * a.M + (c - a.M)] = (int32_t)v;
    else if (c < 2 * a.M + a.G) a.group_num_requests[(size_t)b * a.G + (c - 2 * a.M)] = (int32_t)v;
    else a.group_num_good[(size_t)b * a.G + (c - 2 * a.M - a.G)] = (int32_t)v;
}

// Number of positions where the arrival times are not finite or go backwards.
__global__ void unsorted_kernel(const double *arrivals, int64_t N, int32_t *count)
{
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    int32_t bad = 0;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < N; i += stride) {
        const double t = arrivals[i];
        if (!(t - t == 0.0) || (i > 0 && !(arrivals[i - 1] <= t))) ++bad;
    }
    if (bad) atomicAdd(count, bad);
}

// next_same[i] = next request with request i's model, -1 if none; one thread
// per model walks the trace backwards.
__global__ void next_same_kernel(const int32_t *model_ids, int64_t N, int32_t M, int32_t *next_same)
{
    const int m = blockIdx.x * blockDim.x + threadIdx.x;
    if (m >= M) return;
    int32_t last = -1;
    for (int64_t i = N - 1; i >= 0; --i) {
        if (model_ids[i] == m) { next_same[i] = last; last = (int32_t)i; }
    }
}

// Sum of finish - arrival over one leaf of numpy's pairwise order, read back
// from the per-request outputs: one thread per (leaf, candidate).
__global__ void leaf_sums_from_finish_kernel(const double *finish, const double *arrivals,
                                             int64_t N, int32_t B,
                                             int32_t num_leaves, const int32_t *leaf_start,
                                             double *leaf_sums)
{
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= (int64_t)B * num_leaves) return;
    const int32_t leaf = (int32_t)(t % num_leaves);
    const int64_t b = t / num_leaves;
    const int64_t s = leaf_start[leaf], e = leaf_start[leaf + 1];
    const int64_t body_end = s + ((e - s) & ~(int64_t)7);
    const double *f = finish + (size_t)b * N;
    double p[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    int64_t i = s;
    for (; i < body_end; i += 8)
#pragma unroll
        for (int j = 0; j < 8; ++j) p[j] += f[i + j] - arrivals[i + j];
    double r = ((p[0] + p[1]) + (p[2] + p[3])) + ((p[4] + p[5]) + (p[6] + p[7]));
    for (; i < e; ++i) r += f[i] - arrivals[i];
    leaf_sums[(size_t)leaf * B + b] = r;
}

}  // namespace mms
