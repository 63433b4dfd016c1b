// mms_sim.cu — sm_100a kernels of the placement-evaluation simulator.
//
// What is simulated: AlpaServe's per-request FIFO pipeline model with SLO
// dropping (alpa_serve/simulator/controller.py:561-628, and :506-558 for the
// one-clock-per-group variant) for a batch of candidate placements against
// one request trace, followed by the fast_stats reductions of
// controller.py:393-403.
//
// The recurrence over requests is sequential per candidate.  Parallelism
// comes from (a) the candidates of the batch and (b) cutting each candidate's
// trace into chunks that are simulated SPECULATIVELY at the same time:
//
//   stream kernel   one thread per (candidate, chunk).  A chunk starts from
//                   idle clocks a few thousand requests before its first
//                   request (run-in, nothing recorded), stores the clock
//                   vector it has when the chunk proper begins and after
//                   every segment, and records its decisions and latency sums.
//                   A MIRROR candidate (a copy of a candidate with
//                   interchangeable groups) exchanges those groups' clocks
//                   after the run-in: a second guess at the state.
//   validate kernel one thread per stored run and chunk boundary: which
//                   stored runs of the next chunk start from a state
//                   EQUIVALENT to the one this run ended in
//                   (states_equivalent: equal futures, provably)?
//   resolve kernel  one warp per candidate follows the chain of chunks
//                   through those answers; where no stored run continues
//                   the chain, the true state is copied in and the chunk
//                   goes on a work list.
//   repair kernel   one thread per listed chunk re-simulates it from the true
//                   state, segment by segment, until its state is equivalent
//                   to what a stored run had at that point; the rest of the
//                   chunk is taken from that run.  32 chunks to a warp, or,
//                   for a short list, one (with a step that branches).
//                   validate + resolve + repair run a few rounds (a repaired
//                   chunk can end differently and invalidate its successor).
//   chain kernel    one thread per candidate that is still unsettled walks
//                   all boundaries in order and repairs in place whatever the
//                   rounds left — it makes the result exact whatever the
//                   chunking and the rounds.
//   count kernel    tallies the recorded decisions of the selected runs into
//                   the counters and combines the per-leaf latency sums in
//                   numpy's pairwise order.
//
// The 32 lanes of a warp are 32 candidates on the same chunk (one broadcast
// load per trace element) whenever the batch has 32 or more candidates.
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "mms_sim.h"
#include "sim_batching.cuh"
#include "sim_chunk.cuh"

namespace mms {

constexpr int kMaxSumDepth = 48;        // pair-sum stack of the numpy order
constexpr int kLatSmemBytes = 32 * 1024;
constexpr int kMaxRepairRounds = 16;
constexpr int kDefaultRepairRounds = 4;
constexpr int kDefaultRepairSegments = -1;   // no cap: measured best on the benchmark shape

// What a call clears before its kernels run, in one launch (grid-stride): the
// work lists and run selections of the time-parallel machinery, the outputs
// the tally adds into, the status words — and the kernels' own copy of
// group_info, bounds-checked (a bad entry becomes an empty group) and with the
// "contested" bit (bit 16) cleared: build_tables_kernel derives that bit from
// the replica lists, so exactness never rests on what the caller put there.
struct ClearArgs {
    const uint32_t *group_info_in;    // the caller's [B][G]
    uint32_t *group_info;             // scratch copy the kernels read
    int32_t *model_num_good;          // [Bs][M]
    int32_t *group_num_requests;      // [Bs][G]
    int32_t *group_num_good;          // [Bs][G] or null
    int64_t *good_total;              // [Bs]
};

__device__ inline bool group_info_valid(const KernelArgs &a, uint32_t info)
{
    const uint32_t slot = info & 0xFFu, ns = (info >> 8) & 0xFFu;
    return slot + ns <= (uint32_t)a.T && ns <= (uint32_t)a.S;
}

__global__ void clear_kernel(const KernelArgs a, const ClearArgs c)
{
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t nth = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = tid; i < (int64_t)a.NS * a.B; i += nth) a.seg_src[i] = -1;
    for (int64_t i = tid; i < (int64_t)a.K * a.B; i += nth) {
        a.repair_from[i] = -1;
        a.own_rewritten[i] = 0;
    }
    for (int64_t i = tid; i < (int64_t)a.B * a.G; i += nth) {
        const uint32_t info = c.group_info_in[i];
        c.group_info[i] = group_info_valid(a, info) ? (info & ~0x10000u) : 0u;
    }
    for (int64_t i = tid; i < (int64_t)a.Bs * a.M; i += nth) c.model_num_good[i] = 0;
    for (int64_t i = tid; i < (int64_t)a.Bs * a.G; i += nth) {
        c.group_num_requests[i] = 0;
        if (c.group_num_good) c.group_num_good[i] = 0;
    }
    for (int64_t i = tid; i < a.Bs; i += nth) {
        c.good_total[i] = 0;
        a.status[i] = 0;
        if (a.resimulated) a.resimulated[i] = 0;
    }
    for (int64_t i = tid; i <= kMaxRepairRounds; i += nth) a.work_count[i] = 0;
}

// Builds, in one launch behind clear_kernel, the tables the simulation kernels
// read: (1) one thread per (candidate, model or the extra empty row) checks the
// model's replica list, writes its two 16-byte rows (see Lane::rows) and marks
// the groups of a list with more than one replica as contested; a list with a
// bad index is reported in the status word and emptied.  (2) One thread per
// (candidate, group) reports a group_info entry that clear_kernel had to empty.
// (3) One thread per segment finds the segment's first leaf.
__global__ void build_tables_kernel(const KernelArgs a, const ClearArgs c)
{
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t nth = (int64_t)gridDim.x * blockDim.x;
    for (int64_t q = tid; q <= a.NS; q += nth)
        a.seg_first_leaf[q] = q == 0 ? 0 : q == a.NS ? a.num_leaves
            : leaf_lower_bound(a.leaf_start, a.num_leaves, q * a.seg_len);
    for (int64_t i = tid; i < (int64_t)a.B * a.G; i += nth)
        if (!group_info_valid(a, c.group_info_in[i]))
            atomicOr(&a.status[status_row(a, i / a.G)], MMS_STATUS_BAD_INDEX);
    for (int64_t t = tid; t < (int64_t)a.B * (a.M + 1); t += nth) {
        const int64_t b = t / (a.M + 1);
        const int m = (int)(t % (a.M + 1));
        uint32_t e[8] = {kNoReplica, kNoReplica, kNoReplica, kNoReplica,
                         kNoReplica, kNoReplica, kNoReplica, kNoReplica};
        if (m < a.M) {
            const uint32_t lo = a.model_off[(size_t)b * (a.M + 1) + m];
            const uint32_t hi = a.model_off[(size_t)b * (a.M + 1) + m + 1];
            bool bad = lo > hi || hi > (uint32_t)a.P;
            if (!bad) {
                for (uint32_t r = lo; r < hi; ++r) {
                    const uint32_t ent = a.model_rep[(size_t)b * a.P + r];
                    const uint32_t ns = (ent >> 16) & 0xFFu, first = (ent >> 8) & 0xFFu;
                    if ((ent & 0xFFu) >= (uint32_t)a.G || ns == 0 || first + ns > (uint32_t)a.T ||
                        ns > (uint32_t)a.S || (ent >> 24) >= (uint32_t)a.C)
                        bad = true;
                    else if (r - lo < 8)
                        e[r - lo] = rep_to_last(ent);
                }
                if (hi - lo > 8) e[7] = kMoreReplicas;
            }
            if (bad) {
                atomicOr(&a.status[status_row(a, b)], MMS_STATUS_BAD_INDEX);
                for (int k = 0; k < 8; ++k) e[k] = kNoReplica;
            } else if (hi - lo > 1) {
                // dispatch compares the last-stage clocks of these groups with '<'
                for (uint32_t r = lo; r < hi; ++r)
                    atomicOr(&c.group_info[(size_t)b * a.G + (a.model_rep[(size_t)b * a.P + r] & 0xFFu)],
                             0x10000u);
            }
        }
        uint4 *rows = reinterpret_cast<uint4 *>(a.rep_rows);
        rows[row_index(a, b, m)] = make_uint4(e[0], e[1], e[2], e[3]);
        rows[row_plane(a) + row_index(a, b, m)] = make_uint4(e[4], e[5], e[6], e[7]);
    }
}

// This lane's view of candidate b: offsets of its shared-memory state (clocks
// zeroed) and pointers to its tables in global memory.
template <bool kGroupGood>
__device__ inline Lane setup_lane(const KernelArgs &a, int64_t b, int lane, int warp = 0)
{
    const SmemLayout L = smem_layout(a.M, a.G, a.P, a.T, a.S, kGroupGood, a.lat_smem_elems, a.lat_f64 != 0);
    const size_t base = L.warp0 + (size_t)warp * L.warp_bytes;
    Lane ln;
    ln.clk = (uint32_t)((base + L.clocks) / sizeof(double)) + lane;
    ln.tmp = (uint32_t)((base + L.stage_tmp) / sizeof(double)) + lane;
    ln.lat_sm = (uint32_t)(L.latency / sizeof(float));
    ln.dec_wide = a.dec_wide;
    ln.dec = a.dec_wide ? static_cast<void *>(static_cast<uint16_t *>(a.decisions) + 4 * b)
                        : static_cast<void *>(static_cast<uint8_t *>(a.decisions) + 4 * b);
    ln.dec_pitch = (uint32_t)a.dec_pitch;
    ln.dec_word = 0;
    ln.rows = reinterpret_cast<const uint4 *>(a.rep_rows) + row_index(a, b, 0);
    ln.rows_b = ln.rows + row_plane(a);
    ln.rep_raw = a.model_rep + (size_t)b * a.P;
    ln.rep_off = a.model_off + (size_t)b * (a.M + 1);
    ln.lat_gl = a.latency + (size_t)b * a.latency_stride;
    ln.lat_on_chip = a.lat_smem_elems != 0;
    ln.lat_f64 = a.lat_f64 != 0;
    ln.M = a.M; ln.C = a.C; ln.S = a.S;
    ln.status = 0;
    ln.staging = 0;
    for (int t = 0; t < a.T + kClockPad; ++t) SM_F64(ln.clk + t * kLanes) = 0.0;
    return ln;
}

// The batch's shared latency table goes on chip (f32; widened to f64, exactly,
// when it is used), loaded by all threads of the block: call it before any
// thread returns.
__device__ inline void stage_latency_table(const KernelArgs &a, const SmemLayout &L)
{
    if (a.lat_smem_elems) {
        const int real = a.M * a.C * a.S;
        if (a.lat_f64) {        // widened once here instead of at every use
            const uint32_t base = (uint32_t)(L.latency / sizeof(double));
            for (int i = threadIdx.x; i < a.lat_smem_elems; i += blockDim.x)
                SM_F64(base + i) = i < real ? (double)__ldg(a.latency + i) : 0.0;
        } else {
            const uint32_t base = (uint32_t)(L.latency / sizeof(float));
            for (int i = threadIdx.x; i < a.lat_smem_elems; i += blockDim.x)
                SM_F32(base + i) = i < real ? __ldg(a.latency + i) : 0.0f;
        }
    }
    __syncthreads();
}

__device__ inline void init_pipe(const KernelArgs &a, Pipe &p, int64_t b)
{
    const size_t base = trace_base(a, b);
    p.arrivals = a.arrivals + base; p.model_ids = a.model_ids + base; p.slos = a.slos + base;
    p.pitch = (uint32_t)a.trace_pitch;
    p.last = (int32_t)(a.N - 1);
}

// What the slim form of the narrow step (sim_step, kSlim) takes for granted.
__device__ inline bool slim_shape(const KernelArgs &a)
{
    return a.lat_smem_elems != 0 && a.lat_f64 != 0 && !a.dec_wide;
}

// Byte offset of the decoded-request records behind the repair scratch.
__host__ __device__ inline size_t staging_offset(size_t layout_total, int T, int G)
{
    return (layout_total + (sizeof(double) * (size_t)T + (size_t)G) * kLanes + 15) & ~(size_t)15;
}

// What the step that decodes ahead (staged_step) takes for granted, beyond the slim step:
// every shared-memory index fits 16 bits, and no model of candidate b has more than eight
// replicas.  Called by all 32 lanes of a warp; the answer is the same in all of them.
__device__ inline bool staged_shape(const KernelArgs &a, const SmemLayout &L, int64_t b)
{
    if (!slim_shape(a) || a.trace_pitch < 1) return false;
    if ((staging_offset(L.total, a.T, a.G) + kStagedBytes) / sizeof(double) >= 65536) return false;
    const uint16_t *off = a.model_off + (size_t)b * (a.M + 1);
    bool many = false;
    for (int m = threadIdx.x & (kLanes - 1); m < a.M; m += kLanes) many |= off[m + 1] - off[m] > 8;
    return !__any_sync(0xFFFFFFFFu, many);
}

// Extra shared memory of the kernels that repair: the state the previous run
// stored (f64 [T]) and the scratch list of states_equivalent (u8 [G]).
__device__ inline void repair_scratch(const KernelArgs &a, const SmemLayout &L, int lane,
                                      uint32_t &old_state, uint32_t &stale_buf)
{
    old_state = (uint32_t)(L.total / sizeof(double)) + lane;
    stale_buf = (uint32_t)(L.total + sizeof(double) * (size_t)a.T * kLanes) + lane;
}

// Blocks of block_warps warps (they share the latency table and nothing else).
template <bool kFull, bool kGroupGood, bool kLegacy>
__global__ void __launch_bounds__(kLanes * kMaxBlockWarps, 1)
sim_stream_kernel(const KernelArgs a)
{
    const int lane = threadIdx.x & (kLanes - 1);
    const int warp = threadIdx.x / kLanes;
    stage_latency_table(a, smem_layout(a.M, a.G, a.P, a.T, a.S, kGroupGood, a.lat_smem_elems, a.lat_f64 != 0));
    const bool chunked = can_chunk(a);
    const int64_t stream = ((int64_t)blockIdx.x * a.block_warps + warp) * kLanes + lane;
    if (stream >= (int64_t)a.B * a.K) return;   // lanes never wait for each other below
    const int32_t j = (int32_t)(stream / a.B);
    const int64_t b = stream % a.B;
    if (a.N == 0 || (!chunked && j > 0)) return;
    // a mirror only runs the speculative chunks
    const bool mirror = b >= a.Bs;
    if (mirror && (j == 0 || !chunked)) return;
    const uint64_t swap = (mirror && a.mirror_swap)
                              ? ((uint64_t)a.mirror_swap[2 * b + 1] << 32) | a.mirror_swap[2 * b]
                              : ~0ull;

    Lane ln = setup_lane<kGroupGood>(a, b, lane, warp);
    Pipe p;
    init_pipe(a, p, b);
    // not chunked: one chunk holding every segment, plain sequential simulation
    KernelArgs ka = a;
    int32_t begin = 0;
    if (!chunked) {
        ka.seg_per_chunk = a.NS;
    } else if (j > 0) {
        const int32_t first = a.leaf_start[seg_leaf(a, j * a.seg_per_chunk)];
        begin = first - a.warmup > 0 ? first - a.warmup : 0;
    }
    run_chunk<kFull, kGroupGood, kLegacy>(ka, ln, p, b, j, begin, false,
                                          chunked, 0, 0, -1, 0, swap);
    if (ln.status) atomicOr(&a.status[status_row(a, b)], ln.status);
}

// One thread per (array u, chunk j >= 1), u a scored candidate or a mirror:
// which stored runs of chunk j start from a state that continues the state
// array u holds at the end of chunk j-1 (states_equivalent: equal futures,
// provably)?  Bit 0: the array of the candidate itself, bit 1 + i: its i-th
// mirror.
__global__ void validate_kernel(const KernelArgs a)
{
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (!can_chunk(a) || t >= (int64_t)a.B * (a.K - 1)) return;
    // a round that repaired nothing left every state, and so every mask, as it was
    if (a.round > 0 && a.work_count[a.round - 1] == 0) return;
    if (t == 0) a.work_count[kMaxRepairRounds] = 0;   // resolve_kernel counts the unsettled there
    const int32_t j = (int32_t)(t / a.B) + 1;
    const int64_t u = t % a.B;
    const int64_t b = status_row(a, u);                // the scored candidate u belongs to
    if (u >= a.Bs && (j == 1 || a.partner[u] != b)) return;   // a mirror has no chunk 0
    int64_t m_end;
    const int64_t m_first = mirrors_of(a, b, m_end);
    const int32_t q_prev = j * a.seg_per_chunk - 1;
    const double tau = arrival_at(a, b, a.leaf_start[seg_leaf(a, q_prev + 1)]);
    const size_t B = (size_t)a.B;
    const double *X = a.seg_end + (size_t)q_prev * a.T * B + u;
    uint8_t stale[MMS_MAX_GROUPS];
    uint32_t mask = 0;
    for (int64_t r = 0; r <= m_end - m_first && r < 16; ++r) {
        const double *Y = a.chunk_start + (size_t)j * a.T * B + (r == 0 ? b : m_first + r - 1);
        if (states_equivalent(a, b, [&](uint32_t s) { return X[s * B]; },
                              [&](uint32_t s) { return Y[s * B]; }, tau,
                              [&](int w) -> uint8_t & { return stale[w]; }))
            mask |= 1u << r;
    }
    a.compat[(size_t)j * B + u] = (uint16_t)mask;
}

// Chunk j of candidate b is about to be re-simulated from a NEW start state
// while an earlier, capped repair of it (from an older start state) is still
// unfinished: that repair left its own end-of-segment states in the segments it
// got through, and behind them the records are still those of the speculative
// run, which it never matched.  The new repair must not settle against those
// left-over states (it would then keep the unmatched rest), so they are made
// unequal to everything: a NaN in clock slot 0 fails both "equal" and "in the
// past".  The segments behind them hold states of runs that go on to the end
// of the chunk, which a repair may settle against as usual.
__device__ inline void forget_capped_repair(const KernelArgs &a, int64_t b, int32_t j)
{
    const int32_t pending = a.repair_from[(size_t)j * a.B + b];
    const double nan = __longlong_as_double(0x7FF8000000000000LL);
    for (int32_t q = j * a.seg_per_chunk; q < pending; ++q)
        a.seg_end[(size_t)q * a.T * a.B + b] = nan;
    a.repair_from[(size_t)j * a.B + b] = -1;
}

// One warp per scored candidate: follows the chain of chunks through the
// masks of validate_kernel.  A chunk keeps the run selected for it when that
// one continues the chunk before it; else it is taken from the first mirror
// that does; else the true state is copied into the candidate's own array and
// the chunk goes on the work list.  Behind a listed chunk the walk goes on
// with the old data; the next round (or the chain kernel) sees the new one.
// A candidate whose walk lists nothing is settled: every chunk continues the
// one before it.  That is noted in row 0 of the masks (no boundary uses it)
// and lets the chain kernel skip the candidate.
__global__ void resolve_kernel(const KernelArgs a)
{
    // a warp per candidate: lane 0 walks, all lanes copy a state when one is to be copied
    const int lane = threadIdx.x & (kLanes - 1);
    const int64_t b = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / kLanes;
    if (!can_chunk(a) || b >= a.Bs) return;
    if (a.round > 0 && a.work_count[a.round - 1] == 0) return;    // same masks, same answer
    bool settled = true;
    int64_t m_end;
    const int64_t m_first = mirrors_of(a, b, m_end);
    const size_t B = (size_t)a.B;
    int32_t redone = 0;
    // A candidate nearly all of whose boundaries fail (a placement under sustained overload:
    // no state ever settles, a repaired chunk only moves the failure to the next boundary)
    // gains nothing from the rounds: every chunk would be re-simulated in each of them and
    // once more by the chain kernel.  It is left to the chain kernel as it is.
    {
        int32_t fails = 0;
        for (int32_t j = 1 + lane; j < a.K; j += kLanes) {
            const int32_t q0 = j * a.seg_per_chunk;
            const int32_t e = a.seg_src[(size_t)(q0 - 1) * B + b];
            const int32_t s0 = a.seg_src[(size_t)q0 * B + b];
            const uint32_t mask = a.compat[(size_t)j * B + (e < 0 ? b : e)];
            const uint32_t bit = s0 < 0 ? 0u : (uint32_t)(s0 - m_first + 1);
            fails += !((bit < 16 && ((mask >> bit) & 1u)) || mask != 0);
        }
        fails = __reduce_add_sync(0xFFFFFFFFu, fails);
        if (a.K > 8 && (int64_t)fails * 8 >= (int64_t)(a.K - 1) * 7) {
            if (lane == 0) {
                a.compat[b] = 0;
                atomicAdd(&a.work_count[kMaxRepairRounds], 1u);
            }
            return;
        }
    }
    for (int32_t j = 1; j < a.K; ++j) {
        const int32_t q0 = j * a.seg_per_chunk;
        const int32_t q1 = q0 + a.seg_per_chunk < a.NS ? q0 + a.seg_per_chunk : a.NS;
        int64_t copy_from = -1;          // candidate whose end state becomes chunk j's start
        if (lane == 0) {
            const int32_t e = a.seg_src[(size_t)(q0 - 1) * B + b];     // whose end of chunk j-1 counts
            const int32_t s0 = a.seg_src[(size_t)q0 * B + b];          // whose start of chunk j
            const uint32_t mask = a.compat[(size_t)j * B + (e < 0 ? b : e)];
            const uint32_t bit = s0 < 0 ? 0u : (uint32_t)(s0 - m_first + 1);
            if (bit < 16 && ((mask >> bit) & 1u)) {
                if (s0 < 0 && a.repair_from[(size_t)j * B + b] >= 0) {   // a capped repair goes on
                    const uint32_t slot = atomicAdd(&a.work_count[a.round], 1u);
                    a.work_items[slot] = (uint32_t)((int64_t)j * a.B + b) | 0x80000000u;
                    settled = false;
                }
            } else if (s0 >= 0 && (mask & 1u) && !a.own_rewritten[(size_t)j * B + b]) {
                // a mirror's run was selected, but it is the candidate's own speculative
                // run — untouched so far — that continues the chunk before
                for (int32_t q = q0; q < q1; ++q) a.seg_src[(size_t)q * B + b] = -1;
                a.repair_from[(size_t)j * B + b] = -1;
            } else if (mask >> 1) {
                const int32_t v = (int32_t)m_first + (__ffs((int)(mask >> 1)) - 1);
                for (int32_t q = q0; q < q1; ++q) a.seg_src[(size_t)q * B + b] = v;
                a.repair_from[(size_t)j * B + b] = -1;
            } else {
                copy_from = e < 0 ? b : e;
                // The whole chunk is redone.  Its run selection stays as it is until the
                // repair has compared its state with the selected run's, segment by
                // segment (run_chunk then makes each segment it ran the candidate's own):
                // the selected runs of consecutive segments continue one another, which a
                // selection changed here by hand would not.
                forget_capped_repair(a, b, j);
                const uint32_t slot = atomicAdd(&a.work_count[a.round], 1u);
                a.work_items[slot] = (uint32_t)((int64_t)j * a.B + b);
                ++redone;
                settled = false;
            }
        }
        copy_from = __shfl_sync(0xFFFFFFFFu, copy_from, 0);
        if (copy_from >= 0) {
            const double *X = a.seg_end + (size_t)(q0 - 1) * a.T * B + copy_from;
            double *Y = a.chunk_start + (size_t)j * a.T * B + b;
            for (int s = lane; s < a.T; s += kLanes) Y[s * B] = X[s * B];
        }
    }
    if (lane != 0) return;
    a.compat[b] = settled ? 1 : 0;
    if (!settled) atomicAdd(&a.work_count[kMaxRepairRounds], 1u);
    if (a.resimulated && redone) atomicAdd(&a.resimulated[b], redone);
}

// One thread per chunk on the work list of this round.  A long list is
// worked 32 chunks to a warp (kNarrow false).  A short one — the late rounds,
// where what is left is a few long dependent repairs and the GPU is otherwise
// idle — one chunk to a warp, with the step that branches (kNarrow): the
// duration of a round is that of its longest repair, and a lone lane gets
// through a request in a quarter fewer instructions.  Both kernels are
// launched every round; the one whose turn it is not returns at once.
template <bool kFull, bool kGroupGood, bool kLegacy, bool kNarrow>
__global__ void __launch_bounds__(kLanes, 1)
sim_repair_kernel(const KernelArgs a)
{
    const int lane = kNarrow ? 0 : threadIdx.x;
    const uint32_t count = a.work_count[a.round];
    if ((count <= (uint32_t)a.narrow_limit) != kNarrow) return;
    if ((uint64_t)blockIdx.x * (kNarrow ? 1 : kLanes) >= count) return;
    const SmemLayout L = smem_layout(a.M, a.G, a.P, a.T, a.S, kGroupGood, a.lat_smem_elems, a.lat_f64 != 0);
    stage_latency_table(a, L);
    const uint32_t w = kNarrow ? blockIdx.x : blockIdx.x * kLanes + lane;
    if (w >= count) return;
    const uint32_t item = a.work_items[w] & 0x7FFFFFFFu;
    const bool resume = (a.work_items[w] >> 31) != 0;
    const int32_t j = (int32_t)(item / (uint32_t)a.B);
    const int64_t b = item % (uint32_t)a.B;
    // one chunk to a warp: the lone lane, or — where the step that decodes ahead applies —
    // all 32 lanes as copies of it
    constexpr bool kCanSlim = kNarrow && !kFull && !kLegacy;
    bool staged = false;
    if constexpr (kCanSlim) staged = staged_shape(a, L, b);
    if (kNarrow && !staged && threadIdx.x != 0) return;

    Lane ln = setup_lane<kGroupGood>(a, b, lane);
    ln.staging = staged ? (uint32_t)staging_offset(L.total, a.T, a.G) : 0u;
    uint32_t old_state, stale_buf;
    repair_scratch(a, L, lane, old_state, stale_buf);
    // start of the chunk from the copied-in true state, or where a capped
    // repair stopped, from the state it left after the segment before
    const int32_t q_begin = resume ? a.repair_from[(size_t)j * a.B + b] : j * a.seg_per_chunk;
    const double *src = resume ? a.seg_end + (size_t)(q_begin - 1) * a.T * a.B
                               : a.chunk_start + (size_t)j * a.T * a.B;
    for (int t = 0; t < a.T; ++t) SM_F64(ln.clk + t * kLanes) = src[(size_t)t * a.B + b];
    Pipe p;
    init_pipe(a, p, b);
    const int32_t first = a.leaf_start[seg_leaf(a, q_begin)];
    int64_t m_end;
    const int64_t m_first = mirrors_of(a, b, m_end);
    const bool own_pure = !a.own_rewritten[(size_t)j * a.B + b];
    if (staged) __syncwarp();            // every copy has read the flag before one sets it
    a.own_rewritten[(size_t)j * a.B + b] = 1;
    if (kCanSlim && staged)
        a.repair_from[(size_t)j * a.B + b] =
            run_chunk<kFull, kGroupGood, kLegacy, kNarrow, kCanSlim, kCanSlim>(
                a, ln, p, b, j, first, true, true, old_state, stale_buf, q_begin,
                a.repair_cap, ~0ull, m_first, m_end, own_pure);
    else if (kCanSlim && slim_shape(a))
        a.repair_from[(size_t)j * a.B + b] =
            run_chunk<kFull, kGroupGood, kLegacy, kNarrow, kCanSlim>(
                a, ln, p, b, j, first, true, true, old_state, stale_buf, q_begin,
                a.repair_cap, ~0ull, m_first, m_end, own_pure);
    else
        a.repair_from[(size_t)j * a.B + b] = run_chunk<kFull, kGroupGood, kLegacy, kNarrow>(
            a, ln, p, b, j, first, true, true, old_state, stale_buf, q_begin,
            a.repair_cap, ~0ull, m_first, m_end, own_pure);
    if (ln.status) atomicOr(&a.status[b], ln.status);
}

// One thread per scored candidate: walks the chunk boundaries in order.  A
// chunk keeps the run selected for it when that one continues the chunk
// before it, else takes the first mirror's run that does, else is repaired in
// place in the candidate's own array.  After it, every segment that counts
// was simulated from a state equivalent to the true one.  Like the repairs, it
// comes in two forms, 32 candidates to a warp or (kNarrow, when few are left
// unsettled) one.
template <bool kFull, bool kGroupGood, bool kLegacy, bool kNarrow>
__global__ void __launch_bounds__(kLanes, 1)
sim_chain_kernel(const KernelArgs a)
{
    const int lane = kNarrow ? 0 : threadIdx.x;
    if (!can_chunk(a) || a.N == 0) return;
    if ((a.work_count[kMaxRepairRounds] <= (uint32_t)a.narrow_limit) != kNarrow) return;
    if (kNarrow && a.compat[blockIdx.x]) return;          // whole block: nothing to stage for
    const SmemLayout L = smem_layout(a.M, a.G, a.P, a.T, a.S, kGroupGood, a.lat_smem_elems, a.lat_f64 != 0);
    stage_latency_table(a, L);
    const int64_t b = kNarrow ? (int64_t)blockIdx.x : (int64_t)blockIdx.x * kLanes + lane;
    if (b >= a.Bs) return;
    if (a.compat[b]) return;             // settled by the last walk of resolve_kernel
    // one candidate to a warp: the lone lane, or all 32 lanes as copies of it (see
    // sim_repair_kernel)
    constexpr bool kCanSlim = kNarrow && !kFull && !kLegacy;
    bool staged = false;
    if constexpr (kCanSlim) staged = staged_shape(a, L, b);
    if (kNarrow && !staged && threadIdx.x != 0) return;
    int64_t m_end;
    const int64_t m_first = mirrors_of(a, b, m_end);

    Lane ln = setup_lane<kGroupGood>(a, b, lane);
    ln.staging = staged ? (uint32_t)staging_offset(L.total, a.T, a.G) : 0u;
    uint32_t old_state, stale_buf;
    repair_scratch(a, L, lane, old_state, stale_buf);
    Pipe p;
    init_pipe(a, p, b);
    int32_t redone = 0;
    for (int32_t j = 1; j < a.K; ++j) {
        const int32_t q0 = j * a.seg_per_chunk;
        const int32_t q1 = q0 + a.seg_per_chunk < a.NS ? q0 + a.seg_per_chunk : a.NS;
        const int64_t first = a.leaf_start[seg_leaf(a, q0)];
        const double tau = arrival_at(a, b, first);
        const int32_t e = a.seg_src[(size_t)(q0 - 1) * a.B + b];
        const int32_t s0 = a.seg_src[(size_t)q0 * a.B + b];
        for (int t = 0; t < a.T; ++t)
            SM_F64(ln.clk + t * kLanes) =
                a.seg_end[((size_t)(q0 - 1) * a.T + t) * a.B + (e < 0 ? b : e)];
        auto continues = [&](int64_t v) {
            for (int t = 0; t < a.T; ++t)
                SM_F64(old_state + t * kLanes) = a.chunk_start[((size_t)j * a.T + t) * a.B + v];
            return states_equivalent(
                a, b, [&](uint32_t s) { return SM_F64(ln.clk + s * kLanes); },
                [&](uint32_t s) { return SM_F64(old_state + s * kLanes); }, tau,
                [&](int u) -> uint8_t & { return smem[stale_buf + u * kLanes]; });
        };
        int32_t q_begin = q0;
        int32_t begin = (int32_t)first;
        if (continues(s0 < 0 ? b : s0)) {
            // the chunk continues its predecessor; finish a repair a round left capped
            q_begin = s0 < 0 ? a.repair_from[(size_t)j * a.B + b] : -1;
            if (q_begin < 0) continue;
            begin = a.leaf_start[seg_leaf(a, q_begin)];
            for (int t = 0; t < a.T; ++t)
                SM_F64(ln.clk + t * kLanes) = a.seg_end[((size_t)(q_begin - 1) * a.T + t) * a.B + b];
        } else {
            const bool own_pure = !a.own_rewritten[(size_t)j * a.B + b];
            if (s0 >= 0 && own_pure && continues(b)) {     // back to the own speculative run
                for (int32_t q = q0; q < q1; ++q) a.seg_src[(size_t)q * a.B + b] = -1;
                continue;
            }
            int64_t found = -1;
            for (int64_t m = m_first; m < m_end && found < 0; ++m)
                if (m != s0 && continues(m)) found = m;
            if (found >= 0) {
                for (int32_t q = q0; q < q1; ++q) a.seg_src[(size_t)q * a.B + b] = (int32_t)found;
                continue;
            }
            if (staged) __syncwarp();    // the comparisons above read what is written now
            for (int t = 0; t < a.T; ++t)
                a.chunk_start[((size_t)j * a.T + t) * a.B + b] = SM_F64(ln.clk + t * kLanes);
            forget_capped_repair(a, b, j);
        }
        ++redone;
        const bool own_pure = !a.own_rewritten[(size_t)j * a.B + b];
        if (staged) __syncwarp();        // every copy has read the flag before one sets it
        a.own_rewritten[(size_t)j * a.B + b] = 1;
        if (kCanSlim && staged)
            run_chunk<kFull, kGroupGood, kLegacy, kNarrow, kCanSlim, kCanSlim>(
                a, ln, p, b, j, begin, true, true, old_state, stale_buf, q_begin, 0, ~0ull,
                m_first, m_end, own_pure);
        else if (kCanSlim && slim_shape(a))
            run_chunk<kFull, kGroupGood, kLegacy, kNarrow, kCanSlim>(
                a, ln, p, b, j, begin, true, true, old_state, stale_buf, q_begin, 0, ~0ull,
                m_first, m_end, own_pure);
        else
            run_chunk<kFull, kGroupGood, kLegacy, kNarrow>(a, ln, p, b, j, begin, true, true,
                                                           old_state, stale_buf, q_begin, 0, ~0ull,
                                                           m_first, m_end, own_pure);
        a.repair_from[(size_t)j * a.B + b] = -1;
    }
    if (a.resimulated && redone && (!kNarrow || threadIdx.x == 0))
        atomicAdd(&a.resimulated[b], redone);
    if (ln.status) atomicOr(&a.status[b], ln.status);
}

// Combines the leaf sums of candidate b in numpy's pairing order
// (controller.py:402 consumes the mean).  Leaf sums are fetched eight at a
// time so that the loads overlap.  With seg_src == nullptr every leaf sum is
// the candidate's own.
__device__ inline void sum_leaves(const KernelArgs &a, int64_t b, const uint8_t *leaf_merges,
                                  double *latency_sum)
{
    const int32_t num_leaves = a.num_leaves;
    double stack[kMaxSumDepth];
    int sp = 0;
    int32_t q = -1, seg_stop = 0;        // leaves [.., seg_stop) belong to segment q
    int64_t from = b;
    for (int32_t base = 0; base < num_leaves; base += 8) {
        double v[8];
        uint8_t mg[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int32_t leaf = base + u < num_leaves ? base + u : num_leaves - 1;
            while (leaf >= seg_stop) {
                if (!a.seg_src) { seg_stop = num_leaves; break; }
                ++q;
                const int32_t src = a.seg_src[(size_t)q * a.B + b];
                from = src >= 0 ? src : b;
                seg_stop = seg_leaf(a, q + 1);
            }
            v[u] = a.leaf_sums[(size_t)leaf * a.B + from];
            mg[u] = leaf_merges[leaf];
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            if (base + u >= num_leaves) break;
            if (sp < kMaxSumDepth) stack[sp] = v[u];
            ++sp;
            for (int k = mg[u]; k > 0 && sp >= 2; --k) {
                --sp;
                if (sp < kMaxSumDepth) stack[sp - 1] = stack[sp - 1] + stack[sp];
            }
        }
    }
    if (sp > kMaxSumDepth) atomicOr(&a.status[b], MMS_STATUS_BAD_INDEX);
    latency_sum[b] = (num_leaves > 0) ? stack[0] : 0.0;
}

// One thread per scored candidate: the latency sum, and the total of the good
// requests (controller.py:401) from the per-model counts.
__global__ void finalize_kernel(const KernelArgs a, const uint8_t *leaf_merges,
                                const int32_t *model_num_good, int64_t *good_total,
                                double *latency_sum)
{
    const int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= a.Bs) return;
    sum_leaves(a, b, leaf_merges, latency_sum);
    int64_t total = 0;
    for (int m = 0; m < a.M; ++m) total += model_num_good[(size_t)b * a.M + m];
    good_total[b] = total;
}

// Tallies the recorded decisions of the runs that count (controller.py:587,
// 611, 617-618).  A warp handles 32 consecutive scored candidates (one per
// lane, so their decisions of one request are one 64-byte access) over a
// range of at most 32 segments (fewer than 65 536 requests); each lane counts
// in its own 16-bit shared-memory histograms and adds them to the
// outputs (good_total among them), which must be zero on entry.  One more row
// of blocks (blockIdx.y == 0, so that it starts first) forms the candidates'
// latency sums beside the tally: that walk is one dependent chain per
// candidate and hides under it.
template <typename Dec>
__global__ void __launch_bounds__(kLanes)
count_kernel(const KernelArgs a, int32_t seg_per_block, bool group_good, int32_t *model_num_good,
             int32_t *group_num_requests, int32_t *group_num_good, int64_t *good_total,
             const uint8_t *leaf_merges, double *latency_sum)
{
    if (blockIdx.y == 0) {
        const int64_t c = (int64_t)blockIdx.x * kLanes + threadIdx.x;
        if (c < a.Bs) sum_leaves(a, c, leaf_merges, latency_sum);
        return;
    }
    constexpr int kAcceptedBit = 8 * sizeof(Dec) - 1;
    constexpr uint32_t kAccepted = 1u << kAcceptedBit;
    // per lane: a 32-bit word per group (requests in the low half, good ones in
    // the high half: one update per record) at [group][lane], and 16-bit counts
    // of good requests per model at [model / 2][lane][model % 2] — every lane
    // stays in a bank of its own whatever it counts
    extern __shared__ uint32_t hist[];
    uint32_t *grp = hist;
    uint32_t *modw = hist + (size_t)a.G * kLanes;          // two 16-bit counts to a word
    uint16_t *mod = reinterpret_cast<uint16_t *>(modw);
    const int lane = threadIdx.x;
    const int64_t b = (int64_t)blockIdx.x * kLanes + lane;
    for (int g = 0; g < a.G; ++g) grp[g * kLanes + lane] = 0;
    for (int h = 0; h < (a.M + 1) / 2; ++h)
        reinterpret_cast<uint32_t *>(mod)[h * kLanes + lane] = 0;
    if (b >= a.Bs || a.num_leaves == 0) return;
    const size_t tb = trace_base(a, b);
    const int32_t q0 = (blockIdx.y - 1) * seg_per_block;
    const int32_t q1 = q0 + seg_per_block < a.NS ? q0 + seg_per_block : a.NS;
    for (int32_t q = q0; q < q1; ++q) {
        const int32_t src = a.seg_src[(size_t)q * a.B + b];
        // four consecutive requests of a candidate are one aligned group of records
        struct alignas(4 * sizeof(Dec)) Quad { Dec r[4]; };
        const Quad *col = static_cast<const Quad *>(a.decisions) + (src >= 0 ? src : b);
        const int32_t i_begin = a.leaf_start[seg_leaf(a, q)];
        const int32_t i1 = seg_leaf(a, q + 1) < a.num_leaves ? a.leaf_start[seg_leaf(a, q + 1)]
                                                             : (int32_t)a.N;
        // four groups (sixteen requests) at a time, so that their loads are in flight
        // together; segments start at multiples of 8
        constexpr int kQuads = 4;
        for (int32_t i0 = i_begin; i0 < i1; i0 += 4 * kQuads) {
            Quad d[kQuads];
            int32_t m[4 * kQuads];
#pragma unroll
            for (int u = 0; u < kQuads; ++u) {
                const int32_t i = i0 + 4 * u < i1 ? i0 + 4 * u : i0;
                d[u] = col[(size_t)(i >> 2) * a.dec_pitch];
            }
#pragma unroll
            for (int u = 0; u < 4 * kQuads; ++u) {
                const int32_t i = i0 + u < i1 ? i0 + u : i1 - 1;
                m[u] = a.model_ids[(size_t)i * a.trace_pitch + tb];
            }
            const int32_t valid = i1 - i0;
#pragma unroll
            for (int u = 0; u < 4 * kQuads; ++u) {
                const uint32_t rec = d[u >> 2].r[u & 3];
                if (u >= valid || rec == 0) continue;
                const uint32_t g = (rec & (kAccepted - 1)) - 1;
                const uint32_t accepted = rec >> kAcceptedBit;
                // shared-memory atomics whose result nobody reads: one instruction each and
                // nothing to wait for, where load + add + store was a dependent chain (a lane
                // only ever meets its own words, so there is no contention)
                atomicAdd(&grp[g * kLanes + lane], 1u + (accepted << 16));
                if (accepted)
                    atomicAdd(&modw[((uint32_t)m[u] >> 1) * kLanes + lane], 1u << (16 * (m[u] & 1)));
            }
        }
    }
    uint32_t accepted = 0;
    for (int m = 0; m < a.M; ++m) {
        const uint32_t k = mod[((m >> 1) * kLanes + lane) * 2 + (m & 1)];
        if (k) {
            atomicAdd(&model_num_good[(size_t)b * a.M + m], (int32_t)k);
            accepted += k;
        }
    }
    if (accepted)
        atomicAdd(reinterpret_cast<unsigned long long *>(good_total + b), (unsigned long long)accepted);
    for (int g = 0; g < a.G; ++g) {
        const uint32_t r = grp[g * kLanes + lane] & 0xFFFFu, k = grp[g * kLanes + lane] >> 16;
        if (r) atomicAdd(&group_num_requests[(size_t)b * a.G + g], (int32_t)r);
        if (group_good && k) atomicAdd(&group_num_good[(size_t)b * a.G + g], (int32_t)k);
    }
}

// model_num_requests (controller.py:587) does not depend on the placement:
// one thread per (candidate, model) copies the trace's histogram.
__global__ void model_requests_kernel(const KernelArgs a, int32_t *model_num_requests)
{
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= (int64_t)a.Bs * a.M) return;
    const int64_t b = t / a.M;
    const int m = (int)(t % a.M);
    model_num_requests[t] = a.model_hist[(a.trace_pitch > 1 ? (size_t)b * (a.M + 1) : 0) + m];
}

// Per-model request counts, plus the number of positions where the arrival
// times are not finite or go backwards (hist[M]).
__global__ void histogram_kernel(const double *arrivals, const int32_t *model_ids, int64_t N,
                                 int32_t M, int32_t *hist)
{
    extern __shared__ int32_t local[];
    for (int m = threadIdx.x; m <= M; m += blockDim.x) local[m] = 0;
    __syncthreads();
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < N; i += stride) {
        const int32_t m = model_ids[i];
        if (m >= 0 && m < M) atomicAdd(&local[m], 1);
        const double t = arrivals[i];
        const bool bad = !(t - t == 0.0) || (i > 0 && !(arrivals[i - 1] <= t));
        if (bad) atomicAdd(&local[M], 1);
    }
    __syncthreads();
    for (int m = threadIdx.x; m <= M; m += blockDim.x)
        if (local[m]) atomicAdd(&hist[m], local[m]);
}

// The same for T traces stored request-major ([N][T]): hist[t][M + 1], and the
// total of the bad positions of all traces in hist[T * (M + 1)].  A block
// covers 32 traces (threadIdx.x) and a slice of the requests (blockIdx.y).
__global__ void histogram_traces_kernel(const double *arrivals, const int32_t *model_ids, int64_t N,
                                        int32_t T, int32_t M, int32_t *hist)
{
    extern __shared__ int32_t local[];      // [32][M + 1]
    const int lane = threadIdx.x, row = threadIdx.y;
    for (int k = row * 32 + lane; k < 32 * (M + 1); k += 32 * blockDim.y) local[k] = 0;
    __syncthreads();
    const int64_t t = (int64_t)blockIdx.x * 32 + lane;
    const int64_t step = (int64_t)gridDim.y * blockDim.y;
    if (t < T) {
        for (int64_t i = (int64_t)blockIdx.y * blockDim.y + row; i < N; i += step) {
            const int32_t m = model_ids[(size_t)i * T + t];
            if (m >= 0 && m < M) atomicAdd(&local[lane * (M + 1) + m], 1);
            const double x = arrivals[(size_t)i * T + t];
            const bool bad = !(x - x == 0.0) || (i > 0 && !(arrivals[(size_t)(i - 1) * T + t] <= x));
            if (bad) atomicAdd(&local[lane * (M + 1) + M], 1);
        }
    }
    __syncthreads();
    for (int k = row * 32 + lane; k < 32 * (M + 1); k += 32 * blockDim.y) {
        const int64_t tt = (int64_t)blockIdx.x * 32 + k / (M + 1);
        if (local[k] && tt < T) {
            atomicAdd(&hist[tt * (M + 1) + k % (M + 1)], local[k]);
            if (k % (M + 1) == M) atomicAdd(&hist[(size_t)T * (M + 1)], local[k]);
        }
    }
}

// T traces given one after the other (trace t = elements [offsets[t],
// offsets[t + 1]) of the three arrays) -> the request-major batch the kernels
// read ([N][T], see mms_trace.num_traces), shorter traces padded with requests
// of model -1 that repeat the trace's last arrival time.  A block moves a tile
// of 32 requests x 32 traces through shared memory, so that both the reads
// (along a trace) and the writes (across traces) are coalesced.
__global__ void __launch_bounds__(32 * 8)
pack_traces_kernel(const double *arrivals, const int32_t *model_ids, const float *slos,
                   const int64_t *offsets, int64_t T, int64_t N, double *out_arrivals,
                   int32_t *out_model_ids, float *out_slos)
{
    __shared__ double s_arr[32][33];
    __shared__ int32_t s_mid[32][33];
    __shared__ float s_slo[32][33];
    const int64_t i0 = (int64_t)blockIdx.x * 32, t0 = (int64_t)blockIdx.y * 32;
    for (int r = threadIdx.y; r < 32; r += 8) {          // row r of the tile: trace t0 + r
        const int64_t t = t0 + r, i = i0 + threadIdx.x;
        double a = 0.0;
        int32_t m = -1;
        float s = 0.0f;
        if (t < T) {
            const int64_t lo = offsets[t], n = offsets[t + 1] - lo;
            if (i < n) { a = arrivals[lo + i]; m = model_ids[lo + i]; s = slos[lo + i]; }
            else if (n > 0) a = arrivals[lo + n - 1];
        }
        s_arr[r][threadIdx.x] = a; s_mid[r][threadIdx.x] = m; s_slo[r][threadIdx.x] = s;
    }
    __syncthreads();
    for (int r = threadIdx.y; r < 32; r += 8) {          // request i0 + r, trace t0 + threadIdx.x
        const int64_t i = i0 + r, t = t0 + threadIdx.x;
        if (i < N && t < T) {
            out_arrivals[i * T + t] = s_arr[threadIdx.x][r];
            out_model_ids[i * T + t] = s_mid[threadIdx.x][r];
            out_slos[i * T + t] = s_slo[threadIdx.x][r];
        }
    }
}

// The search's selection over one shard of candidates: the score of
// base_policy.py:225-226 from the reductions (goodput - latency_mean / 10000 +
// num_replicas / 1000000, the same fp64 operations in the same order as the
// host forms it), and the FIRST maximum as np.argmax returns it
// (model_parallelism.py:349-351).  One block; best = {score, global index as a
// double}.  With `accumulate` the pair already in `best` competes too (a batch
// scored in several calls), the smaller index winning a tie.
constexpr int kArgmaxThreads = 256;

__global__ void __launch_bounds__(kArgmaxThreads)
argmax_scores_kernel(const int64_t *good_total, const double *latency_sum,
                     const int64_t *num_replicas, int64_t N, int32_t B, const int64_t *index_map,
                     int64_t index_base, bool accumulate, double *best)
{
    __shared__ double s_score[kArgmaxThreads];
    __shared__ double s_index[kArgmaxThreads];
    double top = -kInf, top_i = 9007199254740992.0;     // 2^53: behind every real index
    for (int32_t b = threadIdx.x; b < B; b += kArgmaxThreads) {
        const double n = (double)N;
        const double goodput = (double)good_total[b] / n;
        const double latency_mean = latency_sum[b] / n;
        double score = goodput - latency_mean / 10000.0;
        if (num_replicas) score = score + (double)num_replicas[b] / 1000000.0;
        const double idx = (double)(index_base + (index_map ? index_map[b] : (int64_t)b));
        if (score > top || (score == top && idx < top_i)) { top = score; top_i = idx; }
    }
    s_score[threadIdx.x] = top;
    s_index[threadIdx.x] = top_i;
    __syncthreads();
    for (int w = kArgmaxThreads / 2; w > 0; w >>= 1) {
        if ((int)threadIdx.x < w) {
            const double o = s_score[threadIdx.x + w], oi = s_index[threadIdx.x + w];
            if (o > s_score[threadIdx.x] || (o == s_score[threadIdx.x] && oi < s_index[threadIdx.x])) {
                s_score[threadIdx.x] = o;
                s_index[threadIdx.x] = oi;
            }
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        double sc = s_score[0], si = s_index[0];
        if (accumulate && (best[0] > sc || (best[0] == sc && best[1] < si))) { sc = best[0]; si = best[1]; }
        best[0] = sc;
        best[1] = si;
    }
}

}  // namespace mms

#include "mms_abi.inl"
