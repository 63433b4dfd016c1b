// sim_chunk.cuh — kernel arguments, trace geometry and the chunk runner.
//
// Geometry.  The trace is cut at leaf boundaries of numpy's pairwise sum into
// SEGMENTS of about seg_len requests (the last one takes the remainder); a
// CHUNK is seg_per_chunk consecutive segments.  Per (candidate, segment) the
// kernels keep the clock vector at the segment's end and the decisions of the
// segment; per (candidate, chunk) the clock vector the chunk was started
// from.  All of it is laid out [..][entry][candidate] so that the 32
// candidates of a warp touch consecutive addresses.
#pragma once
#include "sim_core.cuh"

namespace mms {

struct KernelArgs {
    // trace
    const double *arrivals;
    const int32_t *model_ids;
    const float *slos;
    int64_t N;
    int32_t trace_pitch;          // 1: one trace for all candidates; T > 1: T traces stored
                                  //   request-major ([N][T]), candidate b simulates trace b
    const int32_t *model_hist;    // [M + 1] request counts per model ([T][M + 1] with T traces)
    const int32_t *unsorted;      // number of unsorted / non-finite positions in the trace(s)
    // placements
    int32_t B, M, G, P, T, S, C;
    int32_t Bs;                   // candidates with outputs; [Bs, B) are mirrors
    const int32_t *partner;       // [B] or null
    const uint32_t *mirror_swap;  // [B][2] or null
    const uint16_t *model_off;
    const uint32_t *model_rep;
    const uint32_t *group_info;
    const float *latency;
    int64_t latency_stride;
    int32_t lat_smem_elems;
    int32_t lat_f64;              // the on-chip latency table holds doubles (the f32 values widened)
    int32_t block_warps;          // warps per block of the stream kernel
    // geometry
    int32_t K;                    // chunks
    int32_t NS;                   // segments
    int32_t seg_len;              // requests per segment (nominal)
    int32_t seg_per_chunk;
    int32_t warmup;               // run-in requests before a speculative chunk
    // summation plan
    int32_t num_leaves;
    const int32_t *leaf_start;
    // scratch
    uint32_t *rep_rows;           // [2][ceil(B/32)][M + 1][32][4]: replica rows built from
                                  //   model_off/model_rep (first four replicas of each model,
                                  //   then the next four), see row_index()
    double *leaf_sums;            // [num_leaves][B]
    double *seg_end;              // [NS][T][B]   clock vector after each segment
    double *chunk_start;          // [K][T][B]    clock vector each chunk started from
    int64_t dec_pitch;            // elements per request row of `decisions`: B rounded up to 32,
                                  //   so that a warp's records of one request fill whole sectors
    void *decisions;              // [ceil(N/4)][dec_pitch][4] u8 (up to 126 groups) or u16: 0 = not
                                  //   dispatched, else (group + 1) | accepted << 7 (or << 15),
                                  //   see count_kernel
    bool dec_wide;
    uint32_t *work_count;         // [rounds]
    uint32_t *work_items;         // [B * K]: chunk * B + candidate; bit 31 = continue a repair
    int32_t *repair_from;         // [K][B]: segment a capped repair of chunk j stopped at, or -1
    int32_t *seg_src;             // [NS][B]: whose run of segment q counts for candidate b (its
                                  //          own or one of its mirrors'); -1 = its own
    uint8_t *own_rewritten;       // [K][B]: a repair has written into candidate b's own arrays of
                                  //         chunk j (they are no longer its speculative run from
                                  //         the chunk's first segment to its last)
    uint16_t *compat;             // [K][B]: for run u of chunk j-1, the runs of chunk j whose
                                  //         start continues u's end (bit 0: the candidate's own
                                  //         array, bit 1 + i: its i-th mirror)
    int32_t *seg_first_leaf;      // [NS + 1]: first leaf of each segment
    int32_t narrow_limit;         // repairs of at most this many chunks (or candidates) run one
                                  //   per warp, see sim_repair_kernel
    int32_t repair_cap;           // segments a repair may run per round
    int32_t round;
    // outputs
    uint32_t *status;             // [B]
    double *finish;               // [B][N] or null
    uint8_t *good;                // [B][N] or null
    int32_t *resimulated;         // [B] or null
};

// First leaf whose first request is at or after request index `pos`.
__device__ inline int32_t leaf_lower_bound(const int32_t *leaf_start, int32_t num_leaves,
                                           int64_t pos)
{
    int32_t lo = 0, hi = num_leaves;
    while (lo < hi) {
        const int32_t mid = (lo + hi) >> 1;
        if ((int64_t)leaf_start[mid] < pos) lo = mid + 1; else hi = mid;
    }
    return lo;
}

// First leaf of segment q (q == NS: one past the last leaf).
__device__ inline int32_t seg_leaf(const KernelArgs &a, int32_t q)
{
    if (q <= 0) return 0;
    if (q >= a.NS) return a.num_leaves;
    return a.seg_first_leaf[q];
}

// Where the replica row of (candidate b, model m) is, in 16-byte units: the
// rows of 32 consecutive candidates for one model are contiguous.
__device__ inline size_t row_index(const KernelArgs &a, int64_t b, int m)
{
    return ((size_t)(b / kLanes) * (a.M + 1) + m) * kLanes + (size_t)(b % kLanes);
}

// 16-byte units between a model's first and second replica row.
__device__ inline size_t row_plane(const KernelArgs &a)
{
    return (size_t)((a.B + kLanes - 1) / kLanes) * (a.M + 1) * kLanes;
}

// The mirrors of scored candidate b are candidates [first, end): returns
// first and sets end (first == end: none).
__device__ inline int64_t mirrors_of(const KernelArgs &a, int64_t b, int64_t &end)
{
    end = 0;
    if (!a.partner || a.Bs == a.B) return 0;
    const int64_t first = a.partner[b];
    if (first < a.Bs || first >= a.B) return 0;
    int64_t m = first;
    while (m < a.B && a.partner[m] == b) ++m;
    end = m;
    return first;
}

// Row of the status output candidate b reports to: its own, or for a mirror
// the row of the candidate it mirrors (outputs have Bs rows).
__device__ inline int64_t status_row(const KernelArgs &a, int64_t b)
{
    if (b < a.Bs) return b;
    const int32_t p = a.partner ? a.partner[b] : 0;
    return (p >= 0 && p < a.Bs) ? p : 0;
}

// True when the trace can be cut (sorted, finite arrival times).
__device__ inline bool can_chunk(const KernelArgs &a)
{
    return a.K > 1 && *a.unsorted == 0;
}

// Offset of request 0 of the trace candidate b simulates (a mirror: the trace
// of the candidate it mirrors).
__device__ inline size_t trace_base(const KernelArgs &a, int64_t b)
{
    return a.trace_pitch > 1 ? (size_t)status_row(a, b) : 0;
}

// Arrival time of request i in candidate b's trace.
__device__ inline double arrival_at(const KernelArgs &a, int64_t b, int64_t i)
{
    return a.arrivals[(size_t)i * a.trace_pitch + trace_base(a, b)];
}

// Two clock vectors X and Y, taken at a point where every later arrival is
// >= tau, lead to identical futures (every later finish time, good flag and
// counter) when
//  (1) each slot holds the same value in both, or a value < tau in both — a
//      clock that is already in the past only ever enters max(t, clock) with
//      t >= tau, so its exact value cannot matter — EXCEPT
//  (2) the last-stage clock of a group that serves a model with several
//      replicas: dispatch compares those clocks with '<' (controller.py:595-598),
//      so for the ones in the past the ORDER among them (ties included) must
//      agree as well.  A clock in the past is below every clock that is not,
//      in both vectors, so mixed comparisons agree by (1).
// Each accepted request overwrites clocks with values >= tau that are equal
// in both runs, so the relation is preserved step by step, and it is
// transitive.  LoadX / LoadY map a clock slot to its value.
template <typename LoadX, typename LoadY, typename Stale>
__device__ inline bool states_equivalent(const KernelArgs &a, int64_t b, LoadX X, LoadY Y,
                                         double tau, Stale stale)
{
    int n_stale = 0;
    for (int g = 0; g < a.G; ++g) {
        const uint32_t info = a.group_info[(size_t)b * a.G + g];
        const uint32_t slot = info & 0xFFu, ns = (info >> 8) & 0xFFu;
        const bool contested = (info >> 16) & 1u;
        for (uint32_t k = 0; k < ns; ++k) {
            const double x = X(slot + k), y = Y(slot + k);
            const bool past = x < tau && y < tau;
            if (!(x == y || past)) return false;
            if (past && contested && k == ns - 1 && x != y) stale(n_stale++) = (uint8_t)(slot + k);
        }
    }
    // Order of every past last-stage clock that differs between X and Y
    // against the last-stage clocks of all contested groups.
    for (int u = 0; u < n_stale; ++u) {
        const uint32_t su = stale(u);
        const double xu = X(su), yu = Y(su);
        for (int g = 0; g < a.G; ++g) {
            const uint32_t info = a.group_info[(size_t)b * a.G + g];
            const uint32_t ns = (info >> 8) & 0xFFu;
            if (ns == 0 || !((info >> 16) & 1u)) continue;
            const uint32_t sv = (info & 0xFFu) + ns - 1;
            const double xv = X(sv), yv = Y(sv);
            if ((xu < xv) != (yu < yv) || (xu > xv) != (yu > yv)) return false;
        }
    }
    return true;
}

// Runs chunk j of candidate b on this lane: requests [begin, first) as run-in
// (nothing recorded; `first` is the chunk's first request), then the chunk's
// segments, recording decisions, per-request outputs (kFull) and one latency
// sum per leaf.  Within a leaf the latency of request k goes to partial sum
// k mod 8, as numpy's pairwise sum does: the eight partial sums rotate
// through p0 so that the loop holds ONE copy of the step.
//
//   speculative (repair == false): the clock vector after the run-in is
//       stored as the chunk's start state, and every segment's end state.
//   repair: the lane's clocks already hold the true state at `first`.  After
//       each segment the new state is compared with the states stored runs
//       had at that point (the run selected for the segment so far, the
//       mirrors [m_first, m_end) of the candidate and, with own_pure, the
//       candidate's own speculative run where another run is selected); once
//       it is equivalent to one, the rest of the chunk is taken from that run
//       (seg_src) and the lane stops.  own_pure: no repair has written into
//       the candidate's own arrays of this chunk before this one, so behind
//       the segment being compared they still hold the speculative run.
//       The segments a repair runs become the candidate's own.  A repair
//       may start at a later segment q_begin of the chunk (its clocks then
//       hold the state after segment q_begin - 1) and may be capped at `cap`
//       segments (0 = no cap).
// Returns -1 when the chunk is finished (ran to its end, or settled), else
// the segment at which the capped repair has to be continued.
//
// kStaged (with kSlim): the step that lets the warp decode ahead (staged_step);
// every lane of the warp must be here, set up as lane 0 (see sim_core.cuh).
template <bool kFull, bool kGroupGood, bool kLegacy, bool kNarrow = false, bool kSlim = false,
          bool kStaged = false>
__device__ inline int32_t run_chunk(const KernelArgs &a, Lane &ln, Pipe &p,
                                    int64_t b, int32_t j, int32_t begin,
                                    bool repair, bool snapshots, uint32_t old_state,
                                    uint32_t stale_buf, int32_t q_begin = -1, int32_t cap = 0,
                                    uint64_t swap_pairs = ~0ull, int64_t m_first = 0,
                                    int64_t m_end = 0, bool own_pure = false)
{
    double *fin_out = kFull ? a.finish + (size_t)b * a.N : nullptr;
    uint8_t *good_out = kFull ? a.good + (size_t)b * a.N : nullptr;
    const int32_t q0 = q_begin >= 0 ? q_begin : j * a.seg_per_chunk;
    const int32_t q1 = (j + 1) * a.seg_per_chunk < a.NS ? (j + 1) * a.seg_per_chunk : a.NS;
    int32_t q = q0;
    int32_t leaf = seg_leaf(a, q0);
    int32_t seg_stop = seg_leaf(a, q0 + 1);
    const int32_t first = leaf < a.num_leaves ? a.leaf_start[leaf] : (int32_t)a.N;
    leaf -= 1;                      // the run-in counts as a leaf that is not recorded
    int32_t i = begin, span_end = first;
    bool record = false;
    int32_t done = 0;
    static_assert(!kStaged || kSlim, "the staged step is a form of the slim step");
    Staged st;
    if constexpr (kStaged) st = staged_init(ln); else pipe_prime(ln, p, begin);
    for (;;) {
        // Within a leaf the latency of request k goes to partial sum k mod 8
        // (leaves start at multiples of 8).  The latencies of eight requests
        // are parked in the eight spare clock slots behind the lane's clock
        // vector (read only as don't-care stages otherwise) and added to the
        // partial sums together.
        const int32_t body_end = record ? i + ((span_end - i) & ~7) : i;
        const uint32_t ring = ln.clk + (uint32_t)a.T * kLanes;
        double p0 = 0.0, p1 = 0.0, p2 = 0.0, p3 = 0.0, p4 = 0.0, p5 = 0.0, p6 = 0.0, p7 = 0.0;
        double r = 0.0;
        auto one = [&](int32_t ii) {
            double d;
            if constexpr (kStaged)
                d = staged_step(ln, p, st, ii, record);
            else
                d = sim_step<kFull, kGroupGood, kLegacy, kNarrow, kSlim>(ln, p, ii, record,
                                                                         fin_out, good_out);
            if (ii < body_end) {
                SM_F64(ring + (uint32_t)(ii & 7) * kLanes) = d;
                if ((ii & 7) == 7) {
                    p0 += SM_F64(ring); p1 += SM_F64(ring + kLanes);
                    p2 += SM_F64(ring + 2 * kLanes); p3 += SM_F64(ring + 3 * kLanes);
                    p4 += SM_F64(ring + 4 * kLanes); p5 += SM_F64(ring + 5 * kLanes);
                    p6 += SM_F64(ring + 6 * kLanes); p7 += SM_F64(ring + 7 * kLanes);
                    if (ii + 1 == body_end)
                        r = ((p0 + p1) + (p2 + p3)) + ((p4 + p5) + (p6 + p7));
                }
            } else {
                r += d;
            }
        };
#ifndef MMS_SLIM_UNROLL
#define MMS_SLIM_UNROLL 1
#endif
#ifndef MMS_WIDE_UNROLL
#define MMS_WIDE_UNROLL 1
#endif
        if constexpr ((kSlim && !kStaged && MMS_SLIM_UNROLL) || (!kNarrow && MMS_WIDE_UNROLL)) {
            // three requests per turn: the values fetched ahead rotate through three sets of
            // registers, and after three steps every set is back where it was — no moves (two
            // dozen per request otherwise; in the 32-candidate kernels as well: stream kernel
            // 17.0 -> 16.1 ms)
            for (; i + 3 <= span_end; i += 3) { one(i); one(i + 1); one(i + 2); }
        }
#pragma unroll 1
        for (; i < span_end; ++i) one(i);
        if (!record) {
            // a mirror starts its chunk with interchangeable groups exchanged
            for (int k = 0; k < 4 && swap_pairs != ~0ull; ++k) {
                const uint32_t ga = (uint32_t)(swap_pairs >> (16 * k)) & 0xFFu;
                const uint32_t gb = (uint32_t)(swap_pairs >> (16 * k + 8)) & 0xFFu;
                if (ga >= (uint32_t)a.G || gb >= (uint32_t)a.G) continue;
                const uint32_t ia = a.group_info[(size_t)b * a.G + ga];
                const uint32_t ib = a.group_info[(size_t)b * a.G + gb];
                const uint32_t ns = (ia >> 8) & 0xFFu;
                if (ns != ((ib >> 8) & 0xFFu)) continue;
                for (uint32_t t = 0; t < ns; ++t) {
                    const uint32_t sa = ln.clk + ((ia & 0xFFu) + t) * kLanes;
                    const uint32_t sb = ln.clk + ((ib & 0xFFu) + t) * kLanes;
                    const double va = SM_F64(sa);
                    SM_F64(sa) = SM_F64(sb);
                    SM_F64(sb) = va;
                }
            }
            if (!repair && snapshots)   // the state this speculative chunk starts from
                for (int t = 0; t < a.T; ++t)
                    a.chunk_start[((size_t)j * a.T + t) * a.B + b] = SM_F64(ln.clk + t * kLanes);
        } else {
            a.leaf_sums[(size_t)leaf * a.B + b] = r;
            if (leaf + 1 == seg_stop) {             // segment q is complete
                ++done;
                // A repair stops when its state is equivalent to the state some
                // stored run had at this point: the run currently selected for
                // this segment, or a mirror's.  The rest of the chunk is then
                // taken from that run.
                bool settled = false, reselect = false;
                int32_t settle_src = -1;
                if (repair && snapshots && span_end < a.N) {
                    const double tau = arrival_at(a, b, span_end);
                    const int32_t cur = a.seg_src[(size_t)q * a.B + b];
                    // r == 0: the selected run; r == 1: the own speculative run, where
                    // another is selected; r >= 2: the mirrors
                    for (int64_t r = 0; r <= m_end - m_first + 1 && !settled; ++r) {
                        int64_t v;
                        if (r == 0) v = cur < 0 ? b : cur;
                        else if (r == 1) { if (cur < 0 || !own_pure) continue; v = b; }
                        else { v = m_first + r - 2; if (v == cur) continue; }
                        for (int t = 0; t < a.T; ++t)
                            SM_F64(old_state + t * kLanes) =
                                a.seg_end[((size_t)q * a.T + t) * a.B + v];
                        settled = states_equivalent(
                            a, b, [&](uint32_t s) { return SM_F64(ln.clk + s * kLanes); },
                            [&](uint32_t s) { return SM_F64(old_state + s * kLanes); }, tau,
                            [&](int u) -> uint8_t & { return smem[stale_buf + u * kLanes]; });
                        if (settled && r > 0) { reselect = true; settle_src = v == b ? -1 : (int32_t)v; }
                    }
                }
                // (all lanes of a staged warp run this code as copies of one another: none
                // may overwrite what another has yet to compare)
                if constexpr (kStaged) __syncwarp();
                if (snapshots) {
                    for (int t = 0; t < a.T; ++t)
                        a.seg_end[((size_t)q * a.T + t) * a.B + b] = SM_F64(ln.clk + t * kLanes);
                    if (repair) a.seg_src[(size_t)q * a.B + b] = -1;
                }
                if (settled) {
                    if (reselect)
                        for (int32_t r = q + 1; r < q1; ++r)
                            a.seg_src[(size_t)r * a.B + b] = settle_src;
                    return -1;
                }
                if (++q >= q1) return -1;
                if (cap > 0 && done >= cap) return q;
                seg_stop = seg_leaf(a, q + 1);
            }
        }
        ++leaf;
        if (leaf >= a.num_leaves) return -1;        // only an empty trace gets here
        record = true;
        span_end = a.leaf_start[leaf + 1];
    }
}

}  // namespace mms
