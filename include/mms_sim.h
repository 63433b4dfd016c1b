/*
 * mms_sim.h — C ABI of the B200 placement-evaluation simulator.
 *
 * One call scores a BATCH of candidate placements against ONE request trace
 * on the current CUDA device.  It replaces, for that path, what AlpaServe's
 * PlacementEvaluator does one candidate at a time
 * (alpa_serve/placement_policy/base_policy.py:175-189 calling
 * alpa_serve/simulator/controller.py:308 approximate_one_case).
 *
 * Conventions
 *  - every pointer in the structs below is a DEVICE pointer unless its
 *    comment says "host"; the caller owns all buffers;
 *  - calls are stream-ordered on `stream` (a cudaStream_t passed as void*);
 *    no call synchronises the device, none allocates device memory;
 *  - the return value is 0 or a negative MMS_ERR_* code; per-candidate
 *    conditions found on the device are reported in `status[b]`;
 *  - results are bit-identical to the reference's numba/Python simulator on
 *    the same inputs (fp64, same operation order).
 */
#ifndef MMS_SIM_H_
#define MMS_SIM_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MMS_OK 0
#define MMS_ERR_ARG (-1)          /* null pointer, negative size, bad flag       */
#define MMS_ERR_UNSUPPORTED (-2)  /* shape outside the limits listed below       */
#define MMS_ERR_CUDA (-3)         /* a CUDA runtime call failed (see last_error) */
#define MMS_ERR_NO_DEVICE (-4)

/* Shape limits of the kernels (checked, never assumed). */
#define MMS_MAX_GROUPS 255        /* groups per candidate                        */
#define MMS_MAX_SLOTS 256         /* sum of pipeline stages over a candidate     */
#define MMS_MAX_PLACED 65535      /* (group, model) pairs per candidate          */
#define MMS_MAX_STAGES 255        /* stages of one group                         */
#define MMS_MAX_COLUMNS 254       /* columns of the latency table                */

/* status[b] bits */
#define MMS_STATUS_OK 0u
#define MMS_STATUS_HEAP_OVERFLOW 1u   /* batching: event heap capacity exceeded  */
#define MMS_STATUS_QUEUE_LEFT 2u      /* batching: a request stayed queued       */
#define MMS_STATUS_BAD_INDEX 4u       /* a table index was out of range          */

/* flags */
#define MMS_FLAG_PER_REQUEST 1u   /* also write finish[b][i] and good[b][i]      */
#define MMS_FLAG_LEGACY_CLOCK 2u  /* one clock per group: controller.py:506-558  */
#define MMS_FLAG_NO_GROUP_GOOD 4u /* group_num_good is not wanted (not written);
                                     pass the same flags to the workspace query  */
#define MMS_FLAG_CROWDED 8u       /* a hint, results do not depend on it: another
                                     launch is expected to fill most of the GPU
                                     while this one repairs its chunks, so its
                                     repairs stay packed 32 to a warp unless only
                                     a handful are left                          */

/* The request trace: what controller.py:323-339 caches per Workload
 * (model_ids, slos) plus Workload.arrivals (simulator/workload.py:272). */
typedef struct {
    int64_t num_requests;          /* N */
    const double *arrivals;        /* f64[N]                                     */
    const int32_t *model_ids;      /* i32[N]; -1 = model not registered          */
    const float *slos;             /* f32[N]                                     */
    int64_t num_traces;            /* 0 or 1: one trace, shared by all candidates.
                                      T > 1: T traces of N requests each, stored
                                      request-major (element i of trace t at
                                      [i * T + t], so that 32 candidates read
                                      consecutive addresses); candidate b is
                                      simulated on trace b (mms_sim_mixed only;
                                      num_scored <= T).  Traces of different
                                      lengths are padded at the end with
                                      requests of model -1 that repeat the last
                                      arrival time: such a request changes no
                                      clock and no counter, only latency_sum is
                                      then the pairwise sum over the padded
                                      length.                                    */
} mms_trace;

/* B candidate placements, the tables of controller.py:418-476 in a compact
 * form.  Group g of a candidate owns the clock slots
 * [slot, slot + stages) of that candidate's clock vector.
 *
 *  model_off  u16[B][M+1]  CSR offsets into model_rep
 *  model_rep  u32[B][P]    for model m, its groups in ascending group id
 *                          (row order of m_id2g_id, controller.py:418-422):
 *                          bits 0-7 group id, 8-15 the group's first clock
 *                          slot, 16-23 its stages (pp), 24-31 its column in
 *                          the latency table
 *  group_info u32[B][G]    bits 0-7 first clock slot, 8-15 stages (0 = row
 *                          padding).  Bit 16 ("serves a model that has more
 *                          than one replica") may be set by the caller but is
 *                          not relied on: the library derives it from
 *                          model_off / model_rep on the device, and checks
 *                          slot + stages <= T (MMS_STATUS_BAD_INDEX, the
 *                          group is then treated as padding)
 *  latency    f32[M][C][S] seconds per stage, already rounded to f32 the way
 *                          controller.py:467-476 does; column = parallel
 *                          config.  With latency_stride != 0 candidate b
 *                          reads its own table at latency + b*stride (the
 *                          dense per-group table of the reference: C == G).
 *  With MMS_FLAG_LEGACY_CLOCK: S == 2 and latency[m][c] = {sum, max} of
 *  controller.py:440-441, every group has 1 stage.
 *
 * Mirrors (optional, a speed-up only; nothing in the reference corresponds).
 * Groups with the same parallel config and the same models are
 * interchangeable, and a chunk simulated speculatively (see mms_sim_options)
 * often comes out with their roles permuted, which the exact chain pass
 * then has to re-simulate.  The caller may append, behind the num_scored
 * candidates it wants results for, MIRROR candidates: a copy of a scored
 * candidate's tables whose speculative chunks start with the clock vectors
 * of some groups exchanged.  The chain pass takes each chunk from the
 * candidate's own run or from one of its mirrors', whichever started from a
 * state equivalent to the true one, so results stay exact.
 *   num_scored   candidates [0, num_scored) get outputs (every output array
 *                has num_scored rows); 0 means all
 *   partner      i32[B] or NULL: for a scored candidate its first mirror (or
 *                -1), for a mirror the candidate it mirrors; the mirrors of
 *                one candidate are consecutive
 *   mirror_swap  u32[B][2] or NULL: for a mirror, up to four exchanges of two
 *                groups, applied in order; each is two bytes (group ids a, b),
 *                0xFF = unused
 */
typedef struct {
    int32_t num_candidates;        /* B */
    int32_t num_models;            /* M */
    int32_t max_groups;            /* G: row length of group_info and outputs    */
    int32_t max_placed;            /* P: row length of model_rep                 */
    int32_t max_slots;             /* T: clock slots per candidate (<= 256)      */
    int32_t max_stages;            /* S: last axis of latency                    */
    int32_t num_columns;           /* C (<= 254)                                 */
    int32_t num_scored;            /* 0 = num_candidates (no mirrors)            */
    const uint16_t *model_off;
    const uint32_t *model_rep;
    const uint32_t *group_info;
    const float *latency;
    int64_t latency_stride;        /* elements; 0 = one table for all candidates */
    const int32_t *partner;        /* see "Mirrors" above; may be NULL           */
    const uint32_t *mirror_swap;   /* may be NULL                                */
} mms_placements;

/* How the trace is cut for time-parallel execution.  A candidate's requests
 * are split into chunks of about chunk_requests; every chunk is simulated
 * speculatively from idle clocks after warmup_requests of run-in, then a
 * chain pass keeps a chunk only if the state it started from is equivalent
 * to the true state at that point and re-simulates it otherwise, so results
 * never depend on these two numbers.  Zero = let the library choose;
 * chunk_requests < 0 = one chunk (plain sequential simulation). */
typedef struct {
    int32_t chunk_requests;
    int32_t warmup_requests;
    int32_t repair_rounds;         /* validate+repair rounds before the chain pass (0 = default) */
    int32_t repair_segments;       /* segments (of 1024 requests) one repair may run per round;
                                      it goes on in the next round (0 = default, <0 = no cap) */
} mms_sim_options;

/* How numpy sums N doubles (pairwise, blocks of <= 128, eight interleaved
 * partial sums): the order np.mean(finish - start) uses at
 * controller.py:402.  The plan depends on N only. */
typedef struct {
    int32_t num_leaves;
    int32_t reserved;
    const int32_t *leaf_start;     /* i32[num_leaves + 1], leaf_start[0] == 0    */
    const uint8_t *leaf_merges;    /* u8[num_leaves]: pair-sums after each leaf  */
} mms_sum_plan;

/* Scratch the caller provides (size from mms_sim_workspace_bytes). */
typedef struct {
    void *ptr;
    size_t bytes;
} mms_workspace;

/* Outputs.  B below is num_scored when the batch has mirror candidates. */
typedef struct {
    int32_t *model_num_requests;   /* i32[B][M]                                  */
    int32_t *model_num_good;       /* i32[B][M]                                  */
    int32_t *group_num_requests;   /* i32[B][G]                                  */
    int32_t *group_num_good;       /* i32[B][G] or NULL                          */
    int64_t *good_total;           /* i64[B]: sum(good)                          */
    double *latency_sum;           /* f64[B]: numpy-ordered sum(finish - start)  */
    uint32_t *status;              /* u32[B]                                     */
    double *finish;                /* f64[B][N] with MMS_FLAG_PER_REQUEST        */
    uint8_t *good;                 /* u8[B][N]  with MMS_FLAG_PER_REQUEST        */
    int32_t *resimulated;          /* i32[B] or NULL: chunks the chain pass redid */
} mms_results;

/* Library and device -------------------------------------------------------*/
int mms_abi_version(void);
/* Text of the last failing CUDA call on this thread ("" if none). */
const char *mms_last_error(void);

/* Timing of the dominant kernels, for benchmarks (nothing in the reference
 * corresponds).  After mms_profile_begin(), every mms_sim_mixed and
 * mms_sim_batching call of this process brackets the launches named below
 * with two CUDA events on the caller's stream (up to 2048 spans; later ones
 * are not recorded).  mms_profile_end() stops recording, waits for the
 * recorded events and returns the number of spans and, for the first
 * `capacity` of them in call order, their duration and which launch they
 * bracket.  Off by default; events are created on first use, on the device
 * current then.  For benchmarks only: the recording state is process-wide and
 * unsynchronised, so use it from ONE host thread with no other thread inside
 * the library, and on one device. */
#define MMS_PROFILE_STREAM 0        /* sim_stream_kernel                          */
#define MMS_PROFILE_CHAIN 1         /* sim_chain_kernel (both forms, one span)    */
#define MMS_PROFILE_BATCH_STREAM 2  /* batch_stream_kernel                        */
#define MMS_PROFILE_BATCH_CHAIN 3   /* batch_chain_kernel                         */
#define MMS_PROFILE_CALL 4          /* a whole mms_sim_mixed call                 */
#define MMS_PROFILE_BATCH_REPAIR 5  /* the repair rounds of mms_sim_batching      */
int mms_profile_begin(void);
int mms_profile_end(int32_t *launches, float *each_ms, int32_t *each_tag, int32_t capacity);

/* Summation plan (host side; replaces nothing in the reference — it restates
 * numpy's reduction order, reached from controller.py:402). */
int32_t mms_sum_plan_leaves(int64_t num_requests);
int mms_sum_plan_fill(int64_t num_requests, int32_t *leaf_start /*host*/,
                      uint8_t *leaf_merges /*host*/);

/* Per-model request counts of a trace (model_num_requests of
 * controller.py:587 does not depend on the placement).  hist: i32[M+1]; the
 * last entry counts positions where the arrival times are not finite or
 * decrease — the time-parallel path needs it to be 0 and the kernels fall
 * back to one chunk per candidate when it is not. */
/* With T > 1 traces: hist is i32[T][M+1] followed by ONE more entry, the
 * total of the bad positions of all traces; pass the whole array as model_hist. */
int mms_trace_model_histogram(const mms_trace *trace, int32_t num_models,
                              int32_t *hist, void *stream);

/* Builds the request-major trace batch (an mms_trace with num_traces > 1) on the
 * device from T traces stored one after the other, as a caller has them when it
 * uploads each workload's cached arrays (controller.py:335-339) as they are:
 * trace t is elements [offsets[t], offsets[t+1]) of arrivals / model_ids / slos
 * (offsets: i64[T+1], device).  out_*: [padded_requests][T]; traces shorter
 * than padded_requests (>= the longest) are padded as mms_trace describes.
 * Nothing in the reference corresponds (it simulates one trace per call). */
int mms_trace_pack(const double *arrivals, const int32_t *model_ids, const float *slos,
                   const int64_t *offsets, int64_t num_traces, int64_t padded_requests,
                   double *out_arrivals, int32_t *out_model_ids, float *out_slos, void *stream);

/* Bytes of scratch mms_sim_mixed needs for this shape and these options. */
size_t mms_sim_workspace_bytes(int64_t num_requests, const mms_placements *cands,
                               const mms_sim_options *opts, uint32_t flags);

/* simulate_requests_mixed (controller.py:561-628) — or simulate_requests
 * (controller.py:506-558) with MMS_FLAG_LEGACY_CLOCK — for every candidate,
 * followed by the fast_stats reductions of controller.py:393-403. */
int mms_sim_mixed(const mms_trace *trace, const mms_placements *cands,
                  const mms_sum_plan *plan, const int32_t *model_hist,
                  const mms_sim_options *opts, const mms_workspace *ws,
                  const mms_results *out, uint32_t flags, void *stream);

/* ---- mms_sim_mixed for callers that must not allocate -------------------
 * No counterpart in the reference.
 *
 * Some hosts cannot give mms_sim_mixed a workspace: a plugin running inside a
 * serving process whose framework has already reserved the GPU's memory for
 * its own pool (a cudaMalloc there fails or is forbidden by the host), or a
 * latency-critical loop that must not take the driver's allocation lock and
 * the device-wide synchronisation an allocation or free implies.  This entry
 * point does the same work with the scratch held in an array that is part of
 * the library image: MMS_STATIC_SCRATCH_BYTES of device memory on every GPU
 * that loads the library, held until the process exits.  It calls no
 * cudaMalloc, cudaFree or other allocating routine.
 *
 *  - Inputs and outputs are passed as for mms_sim_mixed; only `ws` is gone.
 *  - A shape whose scratch need (mms_sim_workspace_bytes) exceeds
 *    MMS_STATIC_SCRATCH_BYTES is rejected with MMS_ERR_UNSUPPORTED and a
 *    message in mms_last_error(); nothing is launched.
 *  - The first call on a device looks up the array's device address (once
 *    per device, with that device current; host threads that make it together
 *    are serialised).  Make that first call outside any stream capture.
 *  - Argument and shape errors are reported with the codes mms_sim_mixed
 *    returns for them.
 *  - Every call on a device uses the same array, and the array keeps what the
 *    previous call left in it.  The call clears what it needs cleared, so
 *    back-to-back calls on one stream are fine; two calls whose kernels
 *    overlap on the GPU (different streams, no ordering) race on the array
 *    and give wrong results.
 */
#define MMS_STATIC_SCRATCH_BYTES (32u << 20)
int mms_sim_mixed_static(const mms_trace *trace, const mms_placements *cands,
                         const mms_sum_plan *plan, const int32_t *model_hist,
                         const mms_sim_options *opts, const mms_results *out,
                         uint32_t flags, void *stream);

/* The search's selection step over the candidates one call scored
 * (np.argmax over get_scores, alpa_serve/placement_policy/model_parallelism.py:
 * 349-351, with the score of base_policy.py:225-226 formed from the reductions:
 * good_total / N - latency_sum / N / 10000 + num_replicas / 1000000, the same
 * fp64 operations in the same order).  best: f64[2] = {score, global index}; the
 * global index of candidate b is index_base + (index_map ? index_map[b] : b) and
 * the FIRST maximum wins, as in np.argmax.  With accumulate != 0 the pair
 * already in `best` competes too (a list scored in several calls).  With several
 * GPUs every rank all-gathers its pair and picks the first maximum again.
 * num_replicas (sum of len(group_models), i64[B]) and index_map may be NULL. */
int mms_argmax_scores(const int64_t *good_total, const double *latency_sum,
                      const int64_t *num_replicas, int64_t num_requests, int32_t num_candidates,
                      const int64_t *index_map, int64_t index_base, int32_t accumulate,
                      double *best, void *stream);

/* ---- batching simulator -------------------------------------------------
 * simulate_requests_mixed_batching (controller.py:630-798) for every
 * candidate.  `cands->latency` is f32[M][C][S][NB] here (NB batch sizes, the
 * table of controller.py:451-461); the extra tables below give each group's
 * models (g_id2m_id, controller.py:424-430).  Per-request outputs are always
 * written (requests finish out of arrival order).
 *
 *  group_off u16[B][G+1]  CSR offsets into group_mod
 *  group_mod u16[B][P]    models of each group in ascending model id
 *  group_cfg u32[B][G]    bits 0-7 first clock slot, 8-15 stages, 16-31 column
 *  batch_sizes            alpa_serve.util.batchsize_config (util.py:13): powers
 *                         of two starting at 1; column log2(bs) of the table
 *                         is read for batch size bs, as the reference does
 *  heap_capacity          pending (time, group) events per candidate; 0 picks
 *                         G + 16.  Overflow sets MMS_STATUS_HEAP_OVERFLOW in the
 *                         candidate's status; run it again with a larger heap.
 */
typedef struct {
    const uint16_t *group_off;
    const uint16_t *group_mod;
    const uint32_t *group_cfg;
    int32_t num_batch_sizes;       /* NB, 1..8 */
    int32_t heap_capacity;
    int32_t batch_sizes[8];
} mms_batching;

/* next_same[i] = index of the next request with request i's model, or -1:
 * the per-model FIFO queues of controller.py:648 are runs of this list.
 * next_same: i32[N], filled once per trace. */
int mms_trace_next_same_model(const mms_trace *trace, int32_t num_models, int32_t *next_same,
                              void *stream);

/* Scratch of mms_sim_batching (depends on the heap capacity in `batching`). */
size_t mms_sim_batching_workspace_bytes(int64_t num_requests, const mms_placements *cands,
                                        const mms_batching *batching);

/* The trace is cut in time like in mms_sim_mixed (speculative chunks, then an
 * exact chain pass), so results do not depend on the cut; out->resimulated,
 * when not NULL, gets the number of chunks the chain pass re-simulated. */

int mms_sim_batching(const mms_trace *trace, const mms_placements *cands,
                     const mms_batching *batching, const int32_t *next_same,
                     const mms_sum_plan *plan, const mms_workspace *ws, const mms_results *out,
                     void *stream);

/* ---- Workload.compute_stats ----------------------------------------------
 * alpa_serve/simulator/workload.py:308-354 on the device: per-model and
 * overall statistics of the per-request outputs (mms_results.finish / .good,
 * or any arrays of that layout) over the requests [first, first + window) —
 * the caller cuts `warmup` seconds off both ends as workload.py:312-318 does
 * and passes what is left.  model_ids here are indices into the WORKLOAD's
 * model names (compute_stats groups by request.model_name, whether or not the
 * model is registered); ids outside [0, num_models) are counted in no model.
 * One trace for all candidates.
 *
 *  num_requests  i32[M]     requests of the model in the window (may be NULL)
 *  num_good      i32[B][M]  ... of which good
 *  first_start,
 *  last_start    f64[B][M]  arrival of the model's first / last good request
 *                           (throughput = num_good / (last - first), :338)
 *  latency_mean  f64[B][M]  np.mean(finish - start) over the good requests,
 *  latency_std              np.std of the same, bit for bit (numpy's pairwise
 *                           sums); 0 where no request is good (:340-341)
 *  latency_p90,
 *  latency_p99   f64[B][M]  sorted[int(0.90 * n)], sorted[int(0.99 * n)]
 *  good_total    i64[B]     good requests in the window (np.mean(good) * n)
 *  latency_sum   f64[B]     numpy-ordered sum of finish - start over the
 *                           window (np.mean(finish - start) * n, :352)
 */
typedef struct {
    int32_t *num_requests;
    int32_t *num_good;
    double *first_start, *last_start;
    double *latency_mean, *latency_std, *latency_p90, *latency_p99;
    int64_t *good_total;
    double *latency_sum;
} mms_stats_out;

size_t mms_compute_stats_workspace_bytes(int64_t window, int32_t num_models,
                                         int32_t num_candidates);

/* finish f64 / good u8: row b starts at element b * row_stride. */
int mms_compute_stats(const double *arrivals, const int32_t *model_ids, int32_t num_models,
                      const double *finish, const uint8_t *good, int64_t row_stride,
                      int32_t num_candidates, int64_t first, int64_t window,
                      const mms_workspace *ws, const mms_stats_out *out, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* MMS_SIM_H_ */
