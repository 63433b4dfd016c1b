/*
 * CPU restatement of AlpaServe's placement-evaluation simulator.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker that the parity tests,
 * the smoke test and the benchmark's CPU baseline use.  Nothing in the
 * shipped package may link, load or call it.
 *
 * Every function states which part of the reference it restates, by path
 * inside the alpa-projects/mms project.  The arithmetic is plain IEEE fp64
 * in the reference's operation order: the fp32 latency and SLO tables are
 * widened to fp64 before use, each pipeline stage is "max then add", and the
 * 0.011 s fixed overhead is added last.  Build with -ffp-contract=off and
 * without -ffast-math so that the compiler keeps that order.
 *
 * Parity is pinned by differential runs against the live reference (its own
 * tests hold no per-request golden vectors): tests/golden/ holds outputs of
 * the reference's numba and pure-Python simulators on seeded inputs, made by
 * tests/golden/make_golden.py, and tests/test_oracle.py checks this file
 * against them.
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_INF 1e100          /* alpa_serve/util.py:23 */
#define ORC_OVERHEAD 0.011     /* alpa_serve/simulator/controller.py:575 */

#define ORC_OK 0
#define ORC_ERR_ARG (-1)
#define ORC_ERR_NOMEM (-2)
#define ORC_ERR_QUEUE_NOT_EMPTY (-3)

static inline double dmax(double a, double b) { return a > b ? a : b; }

/* ------------------------------------------------------------------------
 * simulate_requests_mixed, alpa_serve/simulator/controller.py:561-628.
 *
 * m2g            int32 [M][R]      groups that hold model m, -1 ends the row
 *                                  (the reference passes R == G)
 * num_stages     int32 [G]
 * stage_latency  float [M][G][S]   seconds per pipeline stage
 * Outputs finish[N], good[N] and the four int32 counter arrays (zeroed here).
 * ---------------------------------------------------------------------- */
int orc_simulate_requests_mixed(
    double *finish, uint8_t *good,
    const double *tstamps, const int32_t *model_ids, const float *slos,
    const int32_t *m2g, int R,
    const int32_t *num_stages, const float *stage_latency,
    int64_t N, int M, int G, int S,
    int32_t *model_num_requests, int32_t *model_num_good,
    int32_t *group_num_requests, int32_t *group_num_good)
{
    if (N < 0 || M < 0 || G < 0 || S < 0 || R < 0) return ORC_ERR_ARG;
    double *clocks = (double *)calloc((size_t)G * (size_t)S + 1, sizeof(double));
    double *tmp = (double *)calloc((size_t)S + 1, sizeof(double));
    if (!clocks || !tmp) { free(clocks); free(tmp); return ORC_ERR_NOMEM; }
    memset(model_num_requests, 0, sizeof(int32_t) * (size_t)M);
    memset(model_num_good, 0, sizeof(int32_t) * (size_t)M);
    memset(group_num_requests, 0, sizeof(int32_t) * (size_t)G);
    memset(group_num_good, 0, sizeof(int32_t) * (size_t)G);

    for (int64_t i = 0; i < N; ++i) {
        const double ts = tstamps[i];
        const int32_t m = model_ids[i];
        const double slo = (double)slos[i];

        if (m < 0) {                      /* :582-585 unknown model */
            finish[i] = ts; good[i] = 0;
            continue;
        }
        model_num_requests[m] += 1;       /* :587 */

        /* :589-598 replica whose last-stage clock is strictly smallest */
        int32_t g = -1;
        double best = ORC_INF;
        for (int r = 0; r < R; ++r) {
            const int32_t j = m2g[(size_t)m * R + r];
            if (j < 0) break;
            const double c = clocks[(size_t)j * S + (num_stages[j] - 1)];
            if (c < best) { best = c; g = j; }
        }
        if (g < 0) {                      /* :600-603 */
            finish[i] = ts; good[i] = 0;
            continue;
        }

        /* :605-610 walk the pipeline */
        const int ns = num_stages[g];
        const float *lat = stage_latency + ((size_t)m * G + g) * S;
        double t = ts;
        for (int k = 0; k < ns; ++k) {
            t = dmax(t, clocks[(size_t)g * S + k]) + (double)lat[k];
            tmp[k] = t;
        }
        const double fin = t + ORC_OVERHEAD;
        group_num_requests[g] += 1;       /* :611 */

        if (fin - ts <= slo) {            /* :613-619 */
            finish[i] = fin; good[i] = 1;
            for (int k = 0; k < ns; ++k) clocks[(size_t)g * S + k] = tmp[k];
            group_num_good[g] += 1;
            model_num_good[m] += 1;
        } else {                          /* :620-622 */
            finish[i] = ts; good[i] = 0;
        }
    }
    free(clocks); free(tmp);
    return ORC_OK;
}

/* ------------------------------------------------------------------------
 * simulate_requests, alpa_serve/simulator/controller.py:506-558 (one clock
 * per group; reached only with mixed=False).
 * group_max_latency / group_sum_latency: float [M][G].
 * ---------------------------------------------------------------------- */
int orc_simulate_requests(
    double *finish, uint8_t *good,
    const double *tstamps, const int32_t *model_ids, const float *slos,
    const int32_t *m2g, int R,
    const float *group_max_latency, const float *group_sum_latency,
    int64_t N, int M, int G,
    int32_t *model_num_requests, int32_t *model_num_good,
    int32_t *group_num_requests, int32_t *group_num_good)
{
    if (N < 0 || M < 0 || G < 0 || R < 0) return ORC_ERR_ARG;
    double *clocks = (double *)calloc((size_t)G + 1, sizeof(double));
    if (!clocks) return ORC_ERR_NOMEM;
    memset(model_num_requests, 0, sizeof(int32_t) * (size_t)M);
    memset(model_num_good, 0, sizeof(int32_t) * (size_t)M);
    memset(group_num_requests, 0, sizeof(int32_t) * (size_t)G);
    memset(group_num_good, 0, sizeof(int32_t) * (size_t)G);

    for (int64_t i = 0; i < N; ++i) {
        const double ts = tstamps[i];
        const int32_t m = model_ids[i];
        const double slo = (double)slos[i];
        if (m < 0) { finish[i] = ts; good[i] = 0; continue; }       /* :522-525 */
        model_num_requests[m] += 1;

        int32_t g = -1;
        double best = ORC_INF;
        for (int r = 0; r < R; ++r) {                               /* :528-536 */
            const int32_t j = m2g[(size_t)m * R + r];
            if (j < 0) break;
            if (clocks[j] < best) { best = clocks[j]; g = j; }
        }
        if (g < 0) { finish[i] = ts; good[i] = 0; continue; }       /* :538-541 */

        const double start = dmax(clocks[g], ts);                   /* :543 */
        const double fin = start + (double)group_sum_latency[(size_t)m * G + g]
                         + ORC_OVERHEAD;                            /* :544 */
        group_num_requests[g] += 1;
        if (fin - ts <= slo) {                                      /* :547-552 */
            finish[i] = fin; good[i] = 1;
            clocks[g] = start + (double)group_max_latency[(size_t)m * G + g];
            group_num_good[g] += 1;
            model_num_good[m] += 1;
        } else {
            finish[i] = ts; good[i] = 0;
        }
    }
    free(clocks);
    return ORC_OK;
}

/* ------------------------------------------------------------------------
 * simulate_requests_mixed_batching, controller.py:630-798 (pure Python in
 * the reference: closures, list queues and heapq).
 *
 * g2m            int32 [G][Q]        models of group g, -1 ends the row
 * stage_latency  float [M][G][S][NB] NB = len(batchsize_config)
 * batch_sizes    int32 [NB]          batchsize_config (alpa_serve/util.py:13),
 *                                    powers of two; column log2(bs) is read
 *                                    like the reference does (:699,:717)
 * ---------------------------------------------------------------------- */
typedef struct { double t; int32_t g; } orc_event;

typedef struct {
    /* inputs */
    double *finish; uint8_t *good;
    const double *tstamps; const float *slos;
    const int32_t *g2m; int Q;
    const int32_t *num_stages; const float *lat;
    int M, G, S, NB;
    const int32_t *batch_sizes;
    /* state */
    double *clocks, *tmp, *group_idle;
    int64_t *q_head, *q_len, *q_next, *q_tail;  /* per-model FIFO as linked list */
    orc_event *heap; int64_t heap_n, heap_cap;
    int32_t *model_num_good, *group_num_requests, *group_num_good;
    int err;
} orc_bsim;

static int ev_less(const orc_event *a, const orc_event *b)
{   /* Python tuple order on (time, group) — :728,:739-740 */
    if (a->t < b->t) return 1;
    if (a->t > b->t) return 0;
    return a->g < b->g;
}

static void heap_push(orc_bsim *s, double t, int32_t g)
{
    if (s->heap_n == s->heap_cap) {
        int64_t nc = s->heap_cap * 2;
        orc_event *nh = (orc_event *)realloc(s->heap, sizeof(orc_event) * (size_t)nc);
        if (!nh) { s->err = ORC_ERR_NOMEM; return; }
        s->heap = nh; s->heap_cap = nc;
    }
    int64_t i = s->heap_n++;
    orc_event e = { t, g };
    while (i > 0) {
        int64_t p = (i - 1) / 2;
        if (!ev_less(&e, &s->heap[p])) break;
        s->heap[i] = s->heap[p];
        i = p;
    }
    s->heap[i] = e;
}

static orc_event heap_pop(orc_bsim *s)
{
    orc_event top = s->heap[0];
    orc_event e = s->heap[--s->heap_n];
    int64_t i = 0;
    for (;;) {
        int64_t c = 2 * i + 1;
        if (c >= s->heap_n) break;
        if (c + 1 < s->heap_n && ev_less(&s->heap[c + 1], &s->heap[c])) c += 1;
        if (!ev_less(&s->heap[c], &e)) break;
        s->heap[i] = s->heap[c];
        i = c;
    }
    if (s->heap_n > 0) s->heap[i] = e;
    return top;
}

static int64_t queue_pop(orc_bsim *s, int32_t m)
{
    int64_t r = s->q_head[m];
    s->q_head[m] = s->q_next[r];
    s->q_len[m] -= 1;
    return r;
}

/* select_model, :654-664: model of the group whose queue head arrived first */
static int32_t pick_model(const orc_bsim *s, int32_t g)
{
    double first = ORC_INF;
    int32_t pick = -1;
    for (int q = 0; q < s->Q; ++q) {
        const int32_t m = s->g2m[(size_t)g * s->Q + q];
        if (m < 0) break;
        if (s->q_len[m] > 0 && s->tstamps[s->q_head[m]] < first) {
            first = s->tstamps[s->q_head[m]];
            pick = m;
        }
    }
    return pick;
}

/* check_slo, :666-672 */
static int meets_deadline(const orc_bsim *s, double ts, int32_t m, int32_t g,
                          int col, double deadline)
{
    const float *lat = s->lat + (((size_t)m * s->G + g) * s->S) * s->NB;
    double t = ts;
    for (int k = 0; k < s->num_stages[g]; ++k)
        t = dmax(s->clocks[(size_t)g * s->S + k], t) + (double)lat[(size_t)k * s->NB + col];
    return t + ORC_OVERHEAD <= deadline;
}

static int ilog2(int32_t v) { int r = 0; while (v > 1) { v >>= 1; ++r; } return r; }

/* handle_batched_requests + get_max_batch_under_slo, :674-732.  The
 * reference recurses when a model's whole queue is dropped; the loop below
 * is the same tail call. */
static void serve_group(orc_bsim *s, double ts, int32_t m, int32_t g)
{
    while (m >= 0) {
        /* :677-686 drop heads that cannot make it even alone */
        int64_t head = -1;
        while (s->q_len[m] > 0) {
            int64_t r = queue_pop(s, m);
            if (meets_deadline(s, ts, m, g, 0, s->tstamps[r] + (double)s->slos[r])) {
                head = r;
                break;
            }
            s->group_num_requests[g] += 1;
            s->finish[r] = s->tstamps[r];
            s->good[r] = 0;
        }
        if (head < 0) {                   /* :709-713 */
            m = pick_model(s, g);
            continue;
        }
        /* :693-702 grow the batch while the head's deadline still holds */
        int32_t bs = 1;
        const double deadline = s->tstamps[head] + (double)s->slos[head];
        for (int b = 1; b < s->NB; ++b) {
            const int32_t cand = s->batch_sizes[b];
            if (cand - 1 > s->q_len[m]) break;
            if (meets_deadline(s, ts, m, g, ilog2(cand), deadline)) bs = cand;
            else break;
        }
        /* :715-719 */
        const int col = ilog2(bs);
        const float *lat = s->lat + (((size_t)m * s->G + g) * s->S) * s->NB;
        const int ns = s->num_stages[g];
        double t = ts + ORC_OVERHEAD;
        for (int k = 0; k < ns; ++k) {
            t = dmax(t, s->clocks[(size_t)g * s->S + k]) + (double)lat[(size_t)k * s->NB + col];
            s->tmp[k] = t;
        }
        /* :721-725 */
        s->finish[head] = t; s->good[head] = 1;
        for (int32_t b = 1; b < bs; ++b) {
            int64_t r = queue_pop(s, m);
            s->finish[r] = t; s->good[r] = 1;
        }
        for (int k = 0; k < ns; ++k) s->clocks[(size_t)g * s->S + k] = s->tmp[k];
        /* :727-732 */
        s->group_idle[g] = s->tmp[0];
        heap_push(s, s->tmp[0], g);
        s->group_num_requests[g] += bs;
        s->group_num_good[g] += bs;
        s->model_num_good[m] += bs;
        return;
    }
}

int orc_simulate_requests_mixed_batching(
    double *finish, uint8_t *good,
    const double *tstamps, const int32_t *model_ids, const float *slos,
    const int32_t *m2g, int R, const int32_t *g2m, int Q,
    const int32_t *num_stages, const float *stage_latency,
    const int32_t *batch_sizes, int NB,
    int64_t N, int M, int G, int S,
    int32_t *model_num_requests, int32_t *model_num_good,
    int32_t *group_num_requests, int32_t *group_num_good)
{
    if (N < 0 || M < 0 || G < 0 || S < 0 || R < 0 || Q < 0 || NB < 1) return ORC_ERR_ARG;
    orc_bsim s;
    memset(&s, 0, sizeof(s));
    s.finish = finish; s.good = good; s.tstamps = tstamps; s.slos = slos;
    s.g2m = g2m; s.Q = Q; s.num_stages = num_stages; s.lat = stage_latency;
    s.M = M; s.G = G; s.S = S; s.NB = NB; s.batch_sizes = batch_sizes;
    s.model_num_good = model_num_good;
    s.group_num_requests = group_num_requests; s.group_num_good = group_num_good;
    s.clocks = (double *)calloc((size_t)G * S + 1, sizeof(double));
    s.tmp = (double *)calloc((size_t)S + 1, sizeof(double));
    s.group_idle = (double *)calloc((size_t)G + 1, sizeof(double));
    s.q_head = (int64_t *)calloc((size_t)M + 1, sizeof(int64_t));
    s.q_tail = (int64_t *)calloc((size_t)M + 1, sizeof(int64_t));
    s.q_len = (int64_t *)calloc((size_t)M + 1, sizeof(int64_t));
    s.q_next = (int64_t *)calloc((size_t)N + 1, sizeof(int64_t));
    s.heap_cap = 64;
    s.heap = (orc_event *)malloc(sizeof(orc_event) * (size_t)s.heap_cap);
    int rc = ORC_OK;
    if (!s.clocks || !s.tmp || !s.group_idle || !s.q_head || !s.q_tail ||
        !s.q_len || !s.q_next || !s.heap) { rc = ORC_ERR_NOMEM; goto done; }
    memset(model_num_requests, 0, sizeof(int32_t) * (size_t)M);
    memset(model_num_good, 0, sizeof(int32_t) * (size_t)M);
    memset(group_num_requests, 0, sizeof(int32_t) * (size_t)G);
    memset(group_num_good, 0, sizeof(int32_t) * (size_t)G);

    for (int64_t i = 0; i < N; ++i) {
        const double ts = tstamps[i];

        /* :739-744 groups whose first stage became free before this arrival */
        while (s.heap_n > 0 && s.heap[0].t <= ts) {
            orc_event e = heap_pop(&s);
            int32_t pm = pick_model(&s, e.g);
            if (pm == -1) break;          /* the reference breaks, not continues */
            serve_group(&s, e.t, pm, e.g);
        }

        const int32_t m = model_ids[i];
        if (m < 0 || m2g[(size_t)m * R] < 0) {   /* :748-757 */
            finish[i] = ts; good[i] = 0;
            continue;
        }
        int32_t g = -1;                   /* :759-770 */
        double best = ORC_INF;
        for (int r = 0; r < R; ++r) {
            const int32_t j = m2g[(size_t)m * R + r];
            if (j < 0) break;
            const double c = s.clocks[(size_t)j * S + (num_stages[j] - 1)];
            if (c < best) { best = c; g = j; }
        }
        /* :772-773 enqueue on the MODEL's queue */
        if (s.q_len[m] == 0) s.q_head[m] = i; else s.q_next[s.q_tail[m]] = i;
        s.q_tail[m] = i;
        s.q_len[m] += 1;
        model_num_requests[m] += 1;

        if (g >= 0 && ts >= s.group_idle[g])     /* :776-778 */
            serve_group(&s, ts, m, g);
        if (s.err) { rc = s.err; goto done; }
    }
    /* :781-787 drain */
    while (s.heap_n > 0) {
        orc_event e = heap_pop(&s);
        int32_t pm = pick_model(&s, e.g);
        if (pm == -1) continue;
        serve_group(&s, e.t, pm, e.g);
        if (s.err) { rc = s.err; goto done; }
    }
    for (int m = 0; m < M; ++m)           /* :789-790 */
        if (s.q_len[m] != 0) { rc = ORC_ERR_QUEUE_NOT_EMPTY; break; }
done:
    free(s.clocks); free(s.tmp); free(s.group_idle);
    free(s.q_head); free(s.q_tail); free(s.q_len); free(s.q_next); free(s.heap);
    return rc;
}

/* ------------------------------------------------------------------------
 * The summation order of numpy's float64 add-reduce over a contiguous 1-D
 * array (numpy/_core/src/umath/loops_utils.h.src, pairwise sum, block 128,
 * eight interleaved partial sums), which the reference reaches through
 * np.mean(finish - start) at controller.py:402.  Third-party arithmetic:
 * numpy is not vendored by the reference and not pinned (setup.py); the test
 * suite compares this function with the numpy that is installed.
 * ---------------------------------------------------------------------- */
double orc_pairwise_sum(const double *a, int64_t n)
{
    if (n < 8) {
        double r = 0.0;
        for (int64_t i = 0; i < n; ++i) r += a[i];
        return r;
    }
    if (n <= 128) {
        double p[8];
        for (int j = 0; j < 8; ++j) p[j] = a[j];
        int64_t i;
        for (i = 8; i < n - (n % 8); i += 8)
            for (int j = 0; j < 8; ++j) p[j] += a[i + j];
        double r = ((p[0] + p[1]) + (p[2] + p[3])) + ((p[4] + p[5]) + (p[6] + p[7]));
        for (; i < n; ++i) r += a[i];
        return r;
    }
    int64_t h = n / 2;
    h -= h % 8;
    return orc_pairwise_sum(a, h) + orc_pairwise_sum(a + h, n - h);
}

/* np.mean(finish - start), controller.py:402: elementwise fp64 difference,
 * numpy's add-reduce, then one division by N. */
double orc_latency_mean(const double *finish, const double *start, int64_t n)
{
    if (n <= 0) return NAN;
    double *d = (double *)malloc(sizeof(double) * (size_t)n);
    if (!d) return NAN;
    for (int64_t i = 0; i < n; ++i) d[i] = finish[i] - start[i];
    double s = orc_pairwise_sum(d, n);
    free(d);
    return s / (double)n;
}

/* ------------------------------------------------------------------------
 * Batch driver for timing: what PlacementEvaluator.get_scores
 * (alpa_serve/placement_policy/base_policy.py:175-226) computes for a list
 * of candidate placements against one trace, minus the Python around it.
 * Candidate b is described by the dense tables the reference builds in
 * approximate_one_case_one_placement (controller.py:418-476); threads take
 * candidates round-robin.  Per candidate it returns the good-request total
 * and the numpy-ordered latency sum, from which the caller forms the score.
 * ---------------------------------------------------------------------- */
typedef struct {
    const double *tstamps; const int32_t *model_ids; const float *slos;
    int64_t N; int M, G, S, R;
    const int32_t *m2g;        /* [B][M][R] */
    const int32_t *num_stages; /* [B][G] */
    const float *lat;          /* [B][M][G][S] */
    int64_t B; int tid, nthreads;
    int64_t *good_total; double *latency_sum;
    int32_t *model_good;       /* [B][M] */
    int32_t *group_req;        /* [B][G] */
    int rc;
} orc_job;

static void *score_worker(void *arg)
{
    orc_job *j = (orc_job *)arg;
    double *finish = (double *)malloc(sizeof(double) * (size_t)(j->N + 1));
    double *diff = (double *)malloc(sizeof(double) * (size_t)(j->N + 1));
    uint8_t *good = (uint8_t *)malloc((size_t)j->N + 1);
    int32_t *mreq = (int32_t *)malloc(sizeof(int32_t) * (size_t)(j->M + 1));
    int32_t *ggood = (int32_t *)malloc(sizeof(int32_t) * (size_t)(j->G + 1));
    if (!finish || !diff || !good || !mreq || !ggood) { j->rc = ORC_ERR_NOMEM; goto out; }
    for (int64_t b = j->tid; b < j->B; b += j->nthreads) {
        int rc = orc_simulate_requests_mixed(
            finish, good, j->tstamps, j->model_ids, j->slos,
            j->m2g + (size_t)b * j->M * j->R, j->R,
            j->num_stages + (size_t)b * j->G,
            j->lat + (size_t)b * j->M * j->G * j->S,
            j->N, j->M, j->G, j->S,
            mreq, j->model_good + (size_t)b * j->M,
            j->group_req + (size_t)b * j->G, ggood);
        if (rc) { j->rc = rc; break; }
        int64_t ng = 0;
        for (int64_t i = 0; i < j->N; ++i) {
            ng += good[i];
            diff[i] = finish[i] - j->tstamps[i];
        }
        j->good_total[b] = ng;
        j->latency_sum[b] = orc_pairwise_sum(diff, j->N);
    }
out:
    free(finish); free(diff); free(good); free(mreq); free(ggood);
    return NULL;
}

int orc_score_batch(
    const double *tstamps, const int32_t *model_ids, const float *slos, int64_t N,
    int M, int G, int S, int R,
    const int32_t *m2g, const int32_t *num_stages, const float *lat, int64_t B,
    int nthreads,
    int64_t *good_total, double *latency_sum, int32_t *model_good, int32_t *group_req)
{
    if (nthreads < 1) nthreads = 1;
    if (nthreads > 256) nthreads = 256;
    pthread_t th[256];
    orc_job jobs[256];
    for (int t = 0; t < nthreads; ++t) {
        orc_job *j = &jobs[t];
        j->tstamps = tstamps; j->model_ids = model_ids; j->slos = slos;
        j->N = N; j->M = M; j->G = G; j->S = S; j->R = R;
        j->m2g = m2g; j->num_stages = num_stages; j->lat = lat;
        j->B = B; j->tid = t; j->nthreads = nthreads;
        j->good_total = good_total; j->latency_sum = latency_sum;
        j->model_good = model_good; j->group_req = group_req;
        j->rc = ORC_OK;
        if (pthread_create(&th[t], NULL, score_worker, j) != 0) {
            for (int u = 0; u < t; ++u) pthread_join(th[u], NULL);
            return ORC_ERR_NOMEM;
        }
    }
    int rc = ORC_OK;
    for (int t = 0; t < nthreads; ++t) {
        pthread_join(th[t], NULL);
        if (jobs[t].rc) rc = jobs[t].rc;
    }
    return rc;
}
