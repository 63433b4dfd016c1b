// latency_stats.cu — Workload.compute_stats on the device.
//
// alpa_serve/simulator/workload.py:308-354 turns the per-request outputs of a
// simulation (finish time and good flag of every request) into per-model
// statistics: request count, goodput, throughput, mean / standard deviation /
// 90th / 99th percentile of the latency of the good requests, plus the overall
// goodput and mean latency, all over the trace with `warmup` seconds cut off at
// both ends.  The reference does it with numpy on the host, which for this
// library means downloading 9 bytes per request and candidate first.  These
// kernels produce the same numbers, bit for bit, from the arrays where the
// simulator left them:
//
//   window_hist_kernel      requests of each model inside the window
//   window_offsets_kernel   where each model's latencies go in scratch
//   compact_latency_kernel  one block per (model, candidate): finish - start of
//                           the model's good requests, in request order (the
//                           order numpy's fancy indexing gives them)
//   latency_moments_kernel  one block per (model or whole window, candidate):
//                           the sums in numpy's pairwise order (blocks of at
//                           most 128 elements with eight partial sums, halves
//                           rounded down to multiples of eight: numpy/_core/
//                           src/umath/loops_utils.h.src), mean and standard
//                           deviation as np.mean / np.std form them, and the
//                           two order statistics by a radix selection over the
//                           bit patterns (sorted[int(0.90 * n)] needs no sort)
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>

#include "mms_sim.h"

namespace mms {

extern thread_local char g_last_error[256];

constexpr int kStatsThreads = 256;
constexpr int kStatsItems = 8;                     // requests per thread and tile
constexpr int kStatsSmemBins = 4096;               // models counted in shared memory
constexpr int kStatsDepth = 48;                    // pair-sum stack

struct StatsArgs {
    const double *arrivals;
    const int32_t *model_ids;
    const double *finish;
    const uint8_t *good;
    int64_t row_stride;        // elements between two candidates' rows of finish / good
    int64_t first, window;     // requests [first, first + window)
    int32_t M, B;
    // scratch
    int32_t *counts;           // [M]
    int64_t *offsets;          // [M + 1] start of each model's latencies inside a row of lat
    int64_t *leaf_off;         // [M + 2] start of each unit's leaves (unit M: the whole window)
    double *lat;               // [B][window]
    int32_t *leaf_start;       // [B][leaf_cap]
    uint8_t *leaf_merges;      // [B][leaf_cap]
    double *leaf_sums;         // [B][leaf_cap]
    int32_t *node_n;           // [B][leaf_cap] second buffers of the leaf planner
    uint8_t *node_m;           // [B][leaf_cap]
    int64_t leaf_cap;
    mms_stats_out out;
};

__global__ void __launch_bounds__(kStatsThreads)
window_hist_kernel(const int32_t *model_ids, int64_t first, int64_t window, int32_t M,
                   int32_t *counts)
{
    __shared__ int32_t s_bins[kStatsSmemBins];
    const bool in_smem = M <= kStatsSmemBins;
    if (in_smem) {
        for (int m = threadIdx.x; m < M; m += blockDim.x) s_bins[m] = 0;
        __syncthreads();
    }
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < window; i += step) {
        const int32_t m = model_ids[first + i];
        if (m < 0 || m >= M) continue;
        if (in_smem) atomicAdd(&s_bins[m], 1); else atomicAdd(&counts[m], 1);
    }
    if (in_smem) {
        __syncthreads();
        for (int m = threadIdx.x; m < M; m += blockDim.x)
            if (s_bins[m]) atomicAdd(&counts[m], s_bins[m]);
    }
}

// Leaves of numpy's pairwise split never have fewer than 64 elements unless the
// whole array is one leaf, so n / 64 + 2 entries hold the leaf starts of n
// elements and the end mark behind them.
__host__ __device__ inline int64_t leaf_room(int64_t n) { return n / 64 + 2; }

__global__ void window_offsets_kernel(StatsArgs a)
{
    if (blockIdx.x || threadIdx.x) return;
    int64_t at = 0, leaves = 0;
    for (int32_t m = 0; m < a.M; ++m) {
        a.offsets[m] = at;
        a.leaf_off[m] = leaves;
        at += a.counts[m];
        leaves += leaf_room(a.counts[m]);
        if (a.out.num_requests) a.out.num_requests[m] = a.counts[m];
    }
    a.offsets[a.M] = at;
    a.leaf_off[a.M] = leaves;
    a.leaf_off[a.M + 1] = leaves + leaf_room(a.window);
}

// Block (m, b): the latencies of model m's good requests of candidate b, in
// request order, into lat[b][offsets[m] ..]; their number; the arrival times
// of the first and the last of them.
__global__ void __launch_bounds__(kStatsThreads)
compact_latency_kernel(StatsArgs a)
{
    const int32_t m = blockIdx.x;
    const int64_t b = blockIdx.y;
    __shared__ int32_t s_warp[kStatsThreads / 32];
    __shared__ long long s_first, s_last;
    if (threadIdx.x == 0) { s_first = INT64_MAX; s_last = -1; }
    __syncthreads();
    const double *fin = a.finish + (size_t)b * a.row_stride + a.first;
    const uint8_t *good = a.good + (size_t)b * a.row_stride + a.first;
    const double *arr = a.arrivals + a.first;
    const int32_t *ids = a.model_ids + a.first;
    double *dst = a.lat + (size_t)b * a.window + a.offsets[m];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int64_t written = 0, mine_first = INT64_MAX, mine_last = -1;
    constexpr int64_t kTile = (int64_t)kStatsThreads * kStatsItems;
    for (int64_t base = 0; base < a.window; base += kTile) {
        const int64_t i0 = base + (int64_t)threadIdx.x * kStatsItems;
        bool take[kStatsItems];
        int mine = 0;
#pragma unroll
        for (int k = 0; k < kStatsItems; ++k) {
            const int64_t i = i0 + k;
            // both loads issued whatever the first one returns
            const int32_t id = i < a.window ? ids[i] : -1;
            const uint8_t ok = i < a.window ? good[i] : (uint8_t)0;
            take[k] = (id == m) & (ok != 0);
            mine += take[k];
        }
        int incl = mine;                                  // inclusive scan inside the warp
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int o = __shfl_up_sync(0xFFFFFFFFu, incl, d);
            if (lane >= d) incl += o;
        }
        if (lane == 31) s_warp[warp] = incl;
        __syncthreads();
        int before = 0, total = 0;
#pragma unroll
        for (int w = 0; w < kStatsThreads / 32; ++w) {
            const int c = s_warp[w];
            if (w < warp) before += c;
            total += c;
        }
        int64_t pos = written + before + incl - mine;
#pragma unroll
        for (int k = 0; k < kStatsItems; ++k)
            if (take[k]) {
                const int64_t i = i0 + k;
                dst[pos++] = fin[i] - arr[i];
                if (i < mine_first) mine_first = i;
                mine_last = i;
            }
        written += total;
        __syncthreads();                                  // s_warp is rewritten next tile
    }
    if (mine_last >= 0) {
        atomicMin(&s_first, (long long)mine_first);
        atomicMax(&s_last, (long long)mine_last);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const size_t cell = (size_t)b * a.M + m;
        a.out.num_good[cell] = (int32_t)written;
        a.out.first_start[cell] = written ? arr[s_first] : 0.0;
        a.out.last_start[cell] = written ? arr[s_last] : 0.0;
    }
}

// Exclusive prefix sum of one value per thread over the block; `total` gets the sum.
__device__ inline int block_exclusive_scan(int v, int &total)
{
    __shared__ int s_part[kStatsThreads / 32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int incl = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int o = __shfl_up_sync(0xFFFFFFFFu, incl, d);
        if (lane >= d) incl += o;
    }
    if (lane == 31) s_part[warp] = incl;
    __syncthreads();
    int before = 0;
    total = 0;
#pragma unroll
    for (int w = 0; w < kStatsThreads / 32; ++w) {
        const int c = s_part[w];
        if (w < warp) before += c;
        total += c;
    }
    __syncthreads();                                   // s_part is rewritten by the next call
    return before + incl - v;
}

// numpy's split of n elements into leaves, by the whole block: leaf_start[0 ..
// count] (the last entry is n) and, per leaf, how many pair sums follow it.
// The recursion (halves rounded down to multiples of eight until at most 128
// elements are left) is unrolled level by level: every node of a level that is
// still too long is replaced by its two halves, in place in the sequence, so
// the sequence stays in element order; a right half inherits its parent's pair
// sums and adds one.  node_n / node_m: a second pair of buffers of the same
// size as leaf_start / merges.
__device__ inline int32_t block_plan_leaves(int64_t n, int32_t *leaf_start, uint8_t *merges,
                                            int32_t *node_n, uint8_t *node_m)
{
    __shared__ int s_any;
    int32_t *src_n = leaf_start, *dst_n = node_n;
    uint8_t *src_m = merges, *dst_m = node_m;
    if (threadIdx.x == 0) { src_n[0] = (int32_t)n; src_m[0] = 0; s_any = 0; }
    __syncthreads();
    int32_t count = 1;
    for (int level = 0; level < 40; ++level) {
        int32_t made = 0;
        bool split_any = false;
        for (int32_t base = 0; base < count; base += kStatsThreads) {
            const int32_t k = base + threadIdx.x;
            const int32_t v = k < count ? src_n[k] : 0;
            const bool split = v > 128;
            int total;
            const int pos = made + block_exclusive_scan(k < count ? (split ? 2 : 1) : 0, total);
            if (k < count) {
                const uint8_t m = src_m[k];
                if (split) {
                    int32_t half = v / 2;
                    half -= half % 8;
                    dst_n[pos] = half;         dst_m[pos] = 0;
                    dst_n[pos + 1] = v - half; dst_m[pos + 1] = (uint8_t)(m + 1);
                    split_any = true;
                } else {
                    dst_n[pos] = v; dst_m[pos] = m;
                }
            }
            made += total;
        }
        if (split_any) s_any = 1;
        __syncthreads();
        const bool again = s_any != 0;
        __syncthreads();
        if (threadIdx.x == 0) s_any = 0;
        if (!again) break;                              // src already holds the leaves
        int32_t *tn = src_n; src_n = dst_n; dst_n = tn;
        uint8_t *tm = src_m; src_m = dst_m; dst_m = tm;
        count = made;
        __syncthreads();
    }
    // sizes -> starts (in place when the leaves ended up in leaf_start's own buffer: every
    // thread reads its entry before it writes it)
    int32_t at = 0;
    for (int32_t base = 0; base < count; base += kStatsThreads) {
        const int32_t k = base + threadIdx.x;
        const int32_t v = k < count ? src_n[k] : 0;
        const uint8_t m = k < count ? src_m[k] : 0;
        int total;
        const int start = at + block_exclusive_scan(v, total);
        if (k < count) { leaf_start[k] = start; merges[k] = m; }
        at += total;
    }
    if (threadIdx.x == 0) leaf_start[count] = (int32_t)n;
    __syncthreads();
    return count;
}

// One leaf the way numpy adds it up: eight partial sums over the multiples of
// eight, paired, then the rest one by one.
template <typename F>
__device__ inline double leaf_sum(int64_t s, int64_t e, F value)
{
    const int64_t body_end = s + ((e - s) & ~(int64_t)7);
    double p[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    int64_t i = s;
    for (; i < body_end; i += 8)
#pragma unroll
        for (int j = 0; j < 8; ++j) p[j] += value(i + j);
    double r = ((p[0] + p[1]) + (p[2] + p[3])) + ((p[4] + p[5]) + (p[6] + p[7]));
    for (; i < e; ++i) r += value(i);
    return r;
}

// Leaves [lo, hi) combined by the pair sums that fall inside them (a subtree of
// numpy's recursion: the pair sums its last leaf owes to nodes above it stay
// undone).
__device__ inline double merge_leaves(int32_t lo, int32_t hi, const double *sums,
                                      const uint8_t *merges)
{
    double stack[kStatsDepth];
    int sp = 0;
    for (int32_t k = lo; k < hi; ++k) {
        stack[sp++] = sums[k];
        for (int g = merges[k]; g > 0 && sp >= 2; --g) {
            --sp;
            stack[sp - 1] = stack[sp - 1] + stack[sp];
        }
    }
    return hi > lo ? stack[0] : 0.0;
}

// First leaf that starts at element `at` (leaf_start is ascending; the entry exists).
__device__ inline int32_t leaf_at(const int32_t *leaf_start, int32_t num_leaves, int64_t at)
{
    int32_t lo = 0, hi = num_leaves;
    while (lo < hi) {
        const int32_t mid = (lo + hi) >> 1;
        if (leaf_start[mid] < at) lo = mid + 1; else hi = mid;
    }
    return lo;
}

// Block-wide numpy-ordered sum of value(0 .. n-1); every thread gets the result.
// The leaves are added up one per thread.  The pair sums above them follow
// numpy's recursion tree: its nodes at depth D (2^D of them, D chosen so that
// every node above is still split) go one to a thread, which combines its
// node's leaves; the 2^D results are then paired level by level, left + right.
template <typename F>
__device__ inline double block_numpy_sum(int32_t num_leaves, const int32_t *leaf_start,
                                         const uint8_t *merges, double *sums, F value)
{
    __shared__ double s_node[kStatsThreads];
    for (int32_t k = threadIdx.x; k < num_leaves; k += blockDim.x)
        sums[k] = leaf_sum(leaf_start[k], leaf_start[k + 1], value);
    __syncthreads();
    const int64_t n = num_leaves > 0 ? leaf_start[num_leaves] : 0;
    int depth = 0;                      // nodes at depth < `depth` have more than 256 elements
    while ((1 << (depth + 1)) <= kStatsThreads && (n >> (depth + 1)) >= 256) ++depth;
    const int nodes = 1 << depth;
    if ((int)threadIdx.x < nodes) {
        int64_t base = 0, len = n;
        for (int d = depth - 1; d >= 0; --d) {          // the path to node threadIdx.x
            int64_t half = len / 2;
            half -= half % 8;
            if ((threadIdx.x >> d) & 1) { base += half; len -= half; } else { len = half; }
        }
        const int32_t lo = leaf_at(leaf_start, num_leaves, base);
        const int32_t hi = leaf_at(leaf_start, num_leaves, base + len);
        s_node[threadIdx.x] = merge_leaves(lo, hi, sums, merges);
    }
    __syncthreads();
    for (int width = nodes >> 1; width >= 1; width >>= 1) {
        double pair = 0.0;
        if ((int)threadIdx.x < width) pair = s_node[2 * threadIdx.x] + s_node[2 * threadIdx.x + 1];
        __syncthreads();
        if ((int)threadIdx.x < width) s_node[threadIdx.x] = pair;
        __syncthreads();
    }
    const double total = s_node[0];
    __syncthreads();
    return total;
}

// Bit pattern of a double as an unsigned number that orders like the double.
__device__ inline uint64_t order_key(double x)
{
    const uint64_t u = (uint64_t)__double_as_longlong(x);
    return (u >> 63) ? ~u : (u | 0x8000000000000000ull);
}

__device__ inline double key_value(uint64_t k)
{
    const uint64_t u = (k >> 63) ? (k & 0x7FFFFFFFFFFFFFFFull) : ~k;
    return __longlong_as_double((long long)u);
}

// The element of rank `rank` (0-based, ascending) of x[0 .. n): eight passes
// over the data, one byte of the key per pass, most significant first.
__device__ inline double block_select(const double *x, int64_t n, int64_t rank)
{
    __shared__ unsigned int s_hist[256];
    __shared__ unsigned long long s_prefix;
    __shared__ long long s_rank;
    if (threadIdx.x == 0) { s_prefix = 0; s_rank = rank; }
    for (int shift = 56; shift >= 0; shift -= 8) {
        for (int k = threadIdx.x; k < 256; k += blockDim.x) s_hist[k] = 0;
        __syncthreads();
        const uint64_t prefix = s_prefix;
        const uint64_t above = shift == 56 ? 0 : (~0ull << (shift + 8));
        for (int64_t base = 0; base < n; base += 4 * (int64_t)blockDim.x) {
            double v[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {                // four loads in flight per thread
                const int64_t i = base + (int64_t)q * blockDim.x + threadIdx.x;
                v[q] = i < n ? x[i] : 0.0;
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int64_t i = base + (int64_t)q * blockDim.x + threadIdx.x;
                const uint64_t k = order_key(v[q]);
                const bool in = i < n && (k & above) == prefix;
                const unsigned int byte = (unsigned int)(k >> shift) & 255u;
                // equal bytes of a warp go in with one addition
                const unsigned int live = __ballot_sync(0xFFFFFFFFu, in);
                if (in) {
                    const unsigned int same = __match_any_sync(live, byte);
                    if ((int)(threadIdx.x & 31) == __ffs(same) - 1)
                        atomicAdd(&s_hist[byte], __popc(same));
                }
            }
        }
        __syncthreads();
        // the bin that holds the rank: thread t looks at bin t
        const long long want = s_rank;
        const int mine = threadIdx.x < 256 ? (int)s_hist[threadIdx.x] : 0;
        int total;
        const long long before = block_exclusive_scan(mine, total);
        if (threadIdx.x < 256 && before <= want && want < before + mine) {
            s_rank = want - before;
            s_prefix = prefix | ((unsigned long long)threadIdx.x << shift);
        }
        __syncthreads();
    }
    const double v = key_value(s_prefix);
    __syncthreads();
    return v;
}

// Block (u, b, part): u < M is model u, u == M the whole window; part 0 forms
// the sums, parts 1 and 2 select the 90th and the 99th percentile.
__global__ void __launch_bounds__(kStatsThreads)
latency_moments_kernel(StatsArgs a)
{
    const int32_t u = blockIdx.x;
    const int64_t b = blockIdx.y;
    const int part = blockIdx.z;
    if (u == a.M && part != 0) return;
    const size_t region = (size_t)b * a.leaf_cap + a.leaf_off[u];
    int32_t *leaf_start = a.leaf_start + region;
    uint8_t *merges = a.leaf_merges + region;
    double *sums = a.leaf_sums + region;
    int32_t *node_n = a.node_n + region;
    uint8_t *node_m = a.node_m + region;
    if (u == a.M) {
        // np.mean(good) and np.mean(finish - start) over the window (workload.py:352)
        const double *fin = a.finish + (size_t)b * a.row_stride + a.first;
        const uint8_t *good = a.good + (size_t)b * a.row_stride + a.first;
        const double *arr = a.arrivals + a.first;
        const int32_t num_leaves =
            a.window > 0 ? block_plan_leaves(a.window, leaf_start, merges, node_n, node_m) : 0;
        const double total = block_numpy_sum(num_leaves, leaf_start, merges, sums,
                                             [&](int64_t i) { return fin[i] - arr[i]; });
        __shared__ unsigned long long s_good;
        if (threadIdx.x == 0) s_good = 0;
        __syncthreads();
        unsigned long long mine = 0;
        for (int64_t i = threadIdx.x; i < a.window; i += blockDim.x) mine += good[i] != 0;
        atomicAdd(&s_good, mine);
        __syncthreads();
        if (threadIdx.x == 0) {
            a.out.latency_sum[b] = total;
            a.out.good_total[b] = (int64_t)s_good;
        }
        return;
    }
    const size_t cell = (size_t)b * a.M + u;
    const int64_t n = a.out.num_good[cell];
    if (n == 0) {            // the reference puts latency = [0] here (workload.py:339-341)
        if (threadIdx.x == 0 && part == 0) {
            a.out.latency_mean[cell] = 0.0; a.out.latency_std[cell] = 0.0;
            a.out.latency_p90[cell] = 0.0; a.out.latency_p99[cell] = 0.0;
        }
        return;
    }
    const double *x = a.lat + (size_t)b * a.window + a.offsets[u];
    if (part != 0) {
        // sorted[int(0.90 * n)], sorted[int(0.99 * n)] (workload.py:344-345)
        const double frac = part == 1 ? 0.90 : 0.99;
        const double v = block_select(x, n, (int64_t)(frac * (double)n));
        if (threadIdx.x == 0) (part == 1 ? a.out.latency_p90 : a.out.latency_p99)[cell] = v;
        return;
    }
    const int32_t num_leaves = block_plan_leaves(n, leaf_start, merges, node_n, node_m);
    // np.mean: the pairwise sum divided by the count
    const double mean = block_numpy_sum(num_leaves, leaf_start, merges, sums,
                                        [&](int64_t i) { return x[i]; }) / (double)n;
    // np.std: sqrt(sum((x - mean) * (x - mean)) / n), the sum pairwise again
    const double sq = block_numpy_sum(num_leaves, leaf_start, merges, sums,
                                      [&](int64_t i) { const double d = x[i] - mean; return d * d; });
    if (threadIdx.x == 0) {
        a.out.latency_mean[cell] = mean;
        a.out.latency_std[cell] = sqrt(sq / (double)n);
    }
}

static size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

struct StatsGeometry {
    int64_t leaf_cap;
    size_t off_counts, off_offsets, off_leaf_off, off_lat, off_leaf_start, off_leaf_merges,
        off_leaf_sums, off_node_n, off_node_m, total;
};

static int plan_stats(int64_t window, int32_t M, int32_t B, StatsGeometry *g)
{
    if (window < 0 || M < 0 || B < 0) return MMS_ERR_ARG;
    if (window > 0x7FFFFFFF || M > 65535 || B > 65535) return MMS_ERR_UNSUPPORTED;
    // every model's leaves and end mark, then the whole window's
    g->leaf_cap = window / 64 + 2 * (int64_t)M + leaf_room(window);
    size_t at = 0;
    g->off_counts = at;      at = align256(at + (size_t)(M + 1) * 4);
    g->off_offsets = at;     at = align256(at + (size_t)(M + 1) * 8);
    g->off_leaf_off = at;    at = align256(at + (size_t)(M + 2) * 8);
    g->off_lat = at;         at = align256(at + (size_t)B * window * 8);
    g->off_leaf_start = at;  at = align256(at + (size_t)B * g->leaf_cap * 4);
    g->off_leaf_merges = at; at = align256(at + (size_t)B * g->leaf_cap);
    g->off_leaf_sums = at;   at = align256(at + (size_t)B * g->leaf_cap * 8);
    g->off_node_n = at;      at = align256(at + (size_t)B * g->leaf_cap * 4);
    g->off_node_m = at;      at = align256(at + (size_t)B * g->leaf_cap);
    g->total = at;
    return MMS_OK;
}

}  // namespace mms

extern "C" {

size_t mms_compute_stats_workspace_bytes(int64_t window, int32_t num_models, int32_t num_candidates)
{
    mms::StatsGeometry g;
    if (mms::plan_stats(window, num_models, num_candidates, &g) != MMS_OK) return 0;
    return g.total;
}

int mms_compute_stats(const double *arrivals, const int32_t *model_ids, int32_t num_models,
                      const double *finish, const uint8_t *good, int64_t row_stride,
                      int32_t num_candidates, int64_t first, int64_t window,
                      const mms_workspace *ws, const mms_stats_out *out, void *stream)
{
    mms::StatsGeometry g;
    const int rc = mms::plan_stats(window, num_models, num_candidates, &g);
    if (rc != MMS_OK) return rc;
    if (first < 0 || row_stride < first + window || !out) return MMS_ERR_ARG;
    const int32_t M = num_models, B = num_candidates;
    if (B == 0) return MMS_OK;
    if (!out->good_total || !out->latency_sum) return MMS_ERR_ARG;
    if (M > 0 && (!out->num_good || !out->first_start || !out->last_start || !out->latency_mean ||
                  !out->latency_std || !out->latency_p90 || !out->latency_p99))
        return MMS_ERR_ARG;
    if (window > 0 && (!arrivals || !model_ids || !finish || !good)) return MMS_ERR_ARG;
    if (!ws || !ws->ptr || ws->bytes < g.total) {
        snprintf(mms::g_last_error, sizeof(mms::g_last_error),
                 "mms_compute_stats needs %zu bytes of workspace", g.total);
        return MMS_ERR_ARG;
    }
    cudaStream_t st = (cudaStream_t)stream;
    unsigned char *scratch = (unsigned char *)ws->ptr;
    mms::StatsArgs a;
    a.arrivals = arrivals; a.model_ids = model_ids; a.finish = finish; a.good = good;
    a.row_stride = row_stride; a.first = first; a.window = window; a.M = M; a.B = B;
    a.counts = (int32_t *)(scratch + g.off_counts);
    a.offsets = (int64_t *)(scratch + g.off_offsets);
    a.leaf_off = (int64_t *)(scratch + g.off_leaf_off);
    a.lat = (double *)(scratch + g.off_lat);
    a.leaf_start = (int32_t *)(scratch + g.off_leaf_start);
    a.leaf_merges = (uint8_t *)(scratch + g.off_leaf_merges);
    a.leaf_sums = (double *)(scratch + g.off_leaf_sums);
    a.node_n = (int32_t *)(scratch + g.off_node_n);
    a.node_m = (uint8_t *)(scratch + g.off_node_m);
    a.leaf_cap = g.leaf_cap;
    a.out = *out;
#define MMS_STATS_CUDA(call)                                                              \
    do {                                                                                  \
        cudaError_t e_ = (call);                                                          \
        if (e_ != cudaSuccess) {                                                          \
            snprintf(mms::g_last_error, sizeof(mms::g_last_error), "%s: %s", #call,       \
                     cudaGetErrorString(e_));                                             \
            return MMS_ERR_CUDA;                                                          \
        }                                                                                 \
    } while (0)
    MMS_STATS_CUDA(cudaMemsetAsync(a.counts, 0, (size_t)(M + 1) * 4, st));
    if (window > 0 && M > 0) {
        const unsigned blocks = (unsigned)((window + 256 * 16 - 1) / (256 * 16));
        mms::window_hist_kernel<<<blocks < 1024 ? blocks : 1024, mms::kStatsThreads, 0, st>>>(
            model_ids, first, window, M, a.counts);
        MMS_STATS_CUDA(cudaGetLastError());
    }
    mms::window_offsets_kernel<<<1, 32, 0, st>>>(a);
    MMS_STATS_CUDA(cudaGetLastError());
    if (M > 0) {
        mms::compact_latency_kernel<<<dim3((unsigned)M, (unsigned)B), mms::kStatsThreads, 0, st>>>(a);
        MMS_STATS_CUDA(cudaGetLastError());
    }
    mms::latency_moments_kernel<<<dim3((unsigned)M + 1, (unsigned)B, 3), mms::kStatsThreads, 0, st>>>(a);
    MMS_STATS_CUDA(cudaGetLastError());
#undef MMS_STATS_CUDA
    return MMS_OK;
}

}  // extern "C"
