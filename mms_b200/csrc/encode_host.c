/* encode_host.c — flattens and encodes a list of placements.
 *
 * Host-side helper of mms_b200/engine.py::encode_placements, loaded with
 * ctypes.PyDLL (the GIL stays held; no module object, no numpy C API: the
 * caller passes pointers to arrays it allocated).  It replaces the
 * per-object passes over 10^5 Python objects (group configs, model lists)
 * and the dozen numpy passes behind them (sort by model, prefix sums,
 * hashing of model sets) that dominated the encoding time: one walk over the
 * objects, one walk over the flat arrays.  A placement is any object with `group_configs` (a
 * sequence of (dp, op, pp) tuples, e.g. ParallelConfig namedtuples) and
 * `group_models` (a sequence of sequences of ints) —
 * alpa_serve/placement_policy/base_policy.py:18-27.
 *
 * The functions that take Python objects return 0, or -1 with a Python
 * exception set.
 */
#define PY_SSIZE_T_CLEAN
#include <Python.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

static PyObject *g_str_configs, *g_str_models;

static int intern_names(void)
{
    if (!g_str_configs) g_str_configs = PyUnicode_InternFromString("group_configs");
    if (!g_str_models) g_str_models = PyUnicode_InternFromString("group_models");
    return (g_str_configs && g_str_models) ? 0 : -1;
}

/* Pass 1: per placement the number of groups and of (group, model) pairs. */
int mms_host_scan(PyObject *placements, int64_t *n_groups, int64_t *n_pairs)
{
    if (intern_names()) return -1;
    PyObject *seq = PySequence_Fast(placements, "placements must be a sequence");
    if (!seq) return -1;
    const Py_ssize_t B = PySequence_Fast_GET_SIZE(seq);
    int rc = 0;
    for (Py_ssize_t b = 0; b < B && rc == 0; ++b) {
        PyObject *p = PySequence_Fast_GET_ITEM(seq, b);
        PyObject *cfgs = PyObject_GetAttr(p, g_str_configs);
        PyObject *mods = cfgs ? PyObject_GetAttr(p, g_str_models) : NULL;
        PyObject *mseq = mods ? PySequence_Fast(mods, "group_models must be a sequence") : NULL;
        if (!mseq) {
            rc = -1;
        } else {
            const Py_ssize_t G = PySequence_Fast_GET_SIZE(mseq);
            const Py_ssize_t GC = PyObject_Length(cfgs);
            if (GC < 0) {
                rc = -1;
            } else if (GC != G) {
                PyErr_SetString(PyExc_ValueError, "group_configs and group_models differ in length");
                rc = -1;
            }
            int64_t pairs = 0;
            for (Py_ssize_t g = 0; g < G && rc == 0; ++g) {
                const Py_ssize_t n = PyObject_Length(PySequence_Fast_GET_ITEM(mseq, g));
                if (n < 0) rc = -1; else pairs += n;
            }
            n_groups[b] = (int64_t)G;
            n_pairs[b] = pairs;
        }
        Py_XDECREF(mseq);
        Py_XDECREF(mods);
        Py_XDECREF(cfgs);
    }
    Py_DECREF(seq);
    return rc;
}

static inline int as_int64(PyObject *o, int64_t *out)
{
#if PY_VERSION_HEX >= 0x030C0000
    /* ints of one digit (every model id and parallel degree): read in place */
    if (PyLong_CheckExact(o) && PyUnstable_Long_IsCompact((const PyLongObject *)o)) {
        *out = (int64_t)PyUnstable_Long_CompactValue((const PyLongObject *)o);
        return 0;
    }
#endif
    const long long v = PyLong_AsLongLong(o);      /* goes through __index__ for numpy ints */
    if (v == -1 && PyErr_Occurred()) return -1;
    *out = (int64_t)v;
    return 0;
}

/* Pass 2: cfg i64[total groups][3] = (dp, op, pp), n_in_group i64[total
 * groups], placed_model i64[total pairs], all in placement order.  The
 * arrays hold cap_groups / cap_pairs entries (the totals of pass 1); a list
 * that grew in between is an error, not an overrun. */
int mms_host_flatten(PyObject *placements, int64_t *cfg, int64_t *n_in_group, int64_t *placed_model,
                     int64_t cap_groups, int64_t cap_pairs)
{
    if (intern_names()) return -1;
    PyObject *seq = PySequence_Fast(placements, "placements must be a sequence");
    if (!seq) return -1;
    const Py_ssize_t B = PySequence_Fast_GET_SIZE(seq);
    int rc = 0;
    int64_t gi = 0, pi = 0;
    for (Py_ssize_t b = 0; b < B && rc == 0; ++b) {
        PyObject *p = PySequence_Fast_GET_ITEM(seq, b);
        PyObject *cfgs = PyObject_GetAttr(p, g_str_configs);
        PyObject *mods = cfgs ? PyObject_GetAttr(p, g_str_models) : NULL;
        PyObject *cseq = mods ? PySequence_Fast(cfgs, "group_configs must be a sequence") : NULL;
        PyObject *mseq = cseq ? PySequence_Fast(mods, "group_models must be a sequence") : NULL;
        if (!mseq) {
            rc = -1;
        } else {
            const Py_ssize_t G = PySequence_Fast_GET_SIZE(mseq);
            if (PySequence_Fast_GET_SIZE(cseq) != G) {
                PyErr_SetString(PyExc_ValueError, "group_configs and group_models differ in length");
                rc = -1;
            }
            for (Py_ssize_t g = 0; g < G && rc == 0; ++g) {
                PyObject *c = PySequence_Fast_GET_ITEM(cseq, g);
                if (gi >= cap_groups) {
                    PyErr_SetString(PyExc_RuntimeError, "placements changed while being encoded");
                    rc = -1;
                    break;
                }
                if (!PyTuple_Check(c) || PyTuple_GET_SIZE(c) < 3) {
                    PyErr_SetString(PyExc_TypeError, "a group config must be a (dp, op, pp) tuple");
                    rc = -1;
                    break;
                }
                for (int k = 0; k < 3 && rc == 0; ++k)
                    rc = as_int64(PyTuple_GET_ITEM(c, k), &cfg[3 * gi + k]);
                if (rc) break;
                PyObject *ms = PySequence_Fast(PySequence_Fast_GET_ITEM(mseq, g),
                                               "a group's models must be a sequence");
                if (!ms) { rc = -1; break; }
                const Py_ssize_t n = PySequence_Fast_GET_SIZE(ms);
                if (gi >= cap_groups || pi + n > cap_pairs) {
                    PyErr_SetString(PyExc_RuntimeError, "placements changed while being encoded");
                    Py_DECREF(ms);
                    rc = -1;
                    break;
                }
                for (Py_ssize_t k = 0; k < n && rc == 0; ++k)
                    rc = as_int64(PySequence_Fast_GET_ITEM(ms, k), &placed_model[pi++]);
                Py_DECREF(ms);
                n_in_group[gi++] = (int64_t)n;
            }
        }
        Py_XDECREF(mseq);
        Py_XDECREF(cseq);
        Py_XDECREF(mods);
        Py_XDECREF(cfgs);
    }
    Py_DECREF(seq);
    return rc;
}

/* One pass instead of scan + flatten, for callers that come with room to
 * spare: fills n_groups[B], n_pairs[B] and the three flat arrays, totals[0] =
 * groups, totals[1] = pairs.  Returns -2 (no exception set) when the arrays
 * are too small; the caller then falls back to the two passes above. */
int mms_host_flatten_once(PyObject *placements, int64_t *n_groups, int64_t *n_pairs, int64_t *cfg,
                          int64_t *n_in_group, int64_t *placed_model, int64_t cap_groups,
                          int64_t cap_pairs, int64_t *totals)
{
    if (intern_names()) return -1;
    PyObject *seq = PySequence_Fast(placements, "placements must be a sequence");
    if (!seq) return -1;
    const Py_ssize_t B = PySequence_Fast_GET_SIZE(seq);
    int rc = 0;
    int64_t gi = 0, pi = 0;
    for (Py_ssize_t b = 0; b < B && rc == 0; ++b) {
        PyObject *p = PySequence_Fast_GET_ITEM(seq, b);
        PyObject *cfgs = PyObject_GetAttr(p, g_str_configs);
        PyObject *mods = cfgs ? PyObject_GetAttr(p, g_str_models) : NULL;
        PyObject *cseq = mods ? PySequence_Fast(cfgs, "group_configs must be a sequence") : NULL;
        PyObject *mseq = cseq ? PySequence_Fast(mods, "group_models must be a sequence") : NULL;
        if (!mseq) {
            rc = -1;
        } else {
            const Py_ssize_t G = PySequence_Fast_GET_SIZE(mseq);
            const int64_t p_first = pi;
            if (PySequence_Fast_GET_SIZE(cseq) != G) {
                PyErr_SetString(PyExc_ValueError, "group_configs and group_models differ in length");
                rc = -1;
            } else if (gi + G > cap_groups) {
                rc = -2;
            }
            for (Py_ssize_t g = 0; g < G && rc == 0; ++g) {
                PyObject *c = PySequence_Fast_GET_ITEM(cseq, g);
                if (!PyTuple_Check(c) || PyTuple_GET_SIZE(c) < 3) {
                    PyErr_SetString(PyExc_TypeError, "a group config must be a (dp, op, pp) tuple");
                    rc = -1;
                    break;
                }
                for (int k = 0; k < 3 && rc == 0; ++k)
                    rc = as_int64(PyTuple_GET_ITEM(c, k), &cfg[3 * gi + k]);
                if (rc) break;
                PyObject *ms = PySequence_Fast(PySequence_Fast_GET_ITEM(mseq, g),
                                               "a group's models must be a sequence");
                if (!ms) { rc = -1; break; }
                const Py_ssize_t n = PySequence_Fast_GET_SIZE(ms);
                if (pi + n > cap_pairs) rc = -2;
                for (Py_ssize_t k = 0; k < n && rc == 0; ++k)
                    rc = as_int64(PySequence_Fast_GET_ITEM(ms, k), &placed_model[pi++]);
                Py_DECREF(ms);
                n_in_group[gi++] = (int64_t)n;
            }
            n_groups[b] = (int64_t)G;
            n_pairs[b] = pi - p_first;
        }
        Py_XDECREF(mseq);
        Py_XDECREF(cseq);
        Py_XDECREF(mods);
        Py_XDECREF(cfgs);
    }
    Py_DECREF(seq);
    totals[0] = gi;
    totals[1] = pi;
    return rc;
}

/* ---- plain C from here on: no Python objects ---- */

/* Threads mms_host_encode may use (0: four).  One suffices for short lists. */
int mms_host_threads = 0;

/* Distinct (dp, op, pp) rows in order of first appearance: uniq[count][3],
 * inverse[n] = index into uniq.  Returns the count, or -1 when there are more
 * than cap. */
int64_t mms_host_configs(const int64_t *cfg, int64_t n, int64_t *uniq, int64_t cap, int32_t *inverse)
{
    int64_t count = 0;
    int32_t slot_of[64];                  /* a small direct-mapped cache in front of the search */
    for (int k = 0; k < 64; ++k) slot_of[k] = -1;
    for (int64_t i = 0; i < n; ++i) {
        const int64_t *c = cfg + 3 * i;
        const unsigned h = (unsigned)(c[0] * 31 + c[1] * 7 + c[2]) & 63u;
        int64_t hit = slot_of[h];
        if (hit < 0 || uniq[3 * hit] != c[0] || uniq[3 * hit + 1] != c[1] || uniq[3 * hit + 2] != c[2]) {
            hit = -1;
            for (int64_t u = 0; u < count; ++u)
                if (uniq[3 * u] == c[0] && uniq[3 * u + 1] == c[1] && uniq[3 * u + 2] == c[2]) { hit = u; break; }
            if (hit < 0) {
                if (count >= cap) return -1;
                uniq[3 * count] = c[0]; uniq[3 * count + 1] = c[1]; uniq[3 * count + 2] = c[2];
                hit = count++;
            }
            slot_of[h] = (int32_t)hit;
        }
        inverse[i] = (int32_t)hit;
    }
    return count;
}

static uint64_t mix64(uint64_t x)
{
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

/* The tables of mms_placements (include/mms_sim.h) from the flat arrays.
 * Per placement b with groups g = 0 .. n_groups[b]-1 in the given order:
 *   group_info[b][g] = first clock slot | stages << 8 | contested << 16
 *   model_off[b][m] .. model_off[b][m+1]: the replicas of model m in model_rep,
 *   ascending group id (dispatch ties go to the lowest group id,
 *   alpa_serve/simulator/controller.py:590-598)
 *   model_rep[b][k] = group | first clock slot << 8 | stages << 16 | column << 24
 * slots[b] = clock slots used; twin_items[n][3] = (placement, class number
 * inside the placement, group id) for every group that has the same column
 * and the same set of models as another group of its placement, classes and
 * groups ascending; *n_twin_items = n.  A placement whose classes can be
 * permuted in more than max_perms ways (the product of the factorials of
 * their sizes) is left out: it gets no mirror candidates anyway, and early in
 * a search nearly every placement is one.  counts is scratch of M + 1 entries,
 * mark of M.  Unused cells of the tables must come zeroed.
 * Returns 0, or 1 when a model id is outside [0, M). */
struct encode_ctx {
    int64_t M, G, P;
    const int64_t *n_groups, *cfg, *column_of, *n_in_group, *placed_model;
    const int32_t *cfg_index;
    uint16_t *model_off;
    uint32_t *model_rep, *group_info;
    int64_t *slots;
    int32_t *twin_items;
    int64_t max_perms;
};

/* Placements [b0, b1), whose groups start at flat group gi and whose pairs start at flat
 * pair pi.  Twin items go to twin_items rows [gi, ..) — a group appears in at most one
 * item, so the rows of a range never reach the next range's; *n_out = rows written. */
static int encode_range(const struct encode_ctx *c, int64_t b0, int64_t b1, int64_t gi, int64_t pi,
                        int64_t *counts, int64_t *mark, int64_t *n_out)
{
    const int64_t M = c->M;
    const int64_t *cfg = c->cfg, *column_of = c->column_of, *placed_model = c->placed_model;
    const int32_t *cfg_index = c->cfg_index;
    int32_t *twin_items = c->twin_items + 3 * gi;
    const int64_t max_perms = c->max_perms;
    int64_t n_items = 0;
    for (int64_t m = 0; m < M; ++m) mark[m] = -1;
    for (int64_t b = b0; b < b1; ++b) {
        const int64_t ng = c->n_groups[b];
        const int64_t *nin = c->n_in_group + gi;
        uint16_t *off = c->model_off + b * (M + 1);
        uint32_t *rep = c->model_rep + b * c->P;
        uint32_t *info = c->group_info + b * c->G;
        /* replicas per model */
        for (int64_t m = 0; m <= M; ++m) counts[m] = 0;
        int64_t q = pi;
        for (int64_t g = 0; g < ng; ++g)
            for (int64_t k = 0; k < nin[g]; ++k) {
                const int64_t m = placed_model[q++];
                if (m < 0 || m >= M) return 1;
                counts[m + 1]++;
            }
        int64_t run = 0;
        off[0] = 0;
        for (int64_t m = 0; m < M; ++m) {
            const int64_t cnt = counts[m + 1];
            counts[m + 1] = run;                      /* next free position of model m */
            run += cnt;
            off[m + 1] = (uint16_t)run;
        }
        /* groups in ascending id: positions inside a model's list come out ascending too */
        int64_t slot = 0;
        q = pi;
        uint64_t key[256];
        for (int64_t g = 0; g < ng; ++g) {
            const int64_t pp = cfg[3 * (gi + g) + 2];
            const int64_t col = column_of[cfg_index[gi + g]];
            uint32_t contested = 0;
            uint64_t h = 0;
            for (int64_t k = 0; k < nin[g]; ++k) {
                const int64_t m = placed_model[q++];
                rep[counts[m + 1]++] = (uint32_t)(g | (slot << 8) | (pp << 16) | (col << 24));
                if (off[m + 1] - off[m] > 1) contested = 1;
                h += mix64((uint64_t)m);
            }
            info[g] = (uint32_t)(slot | (pp << 8) | ((int64_t)contested << 16));
            if (g < 256) key[g] = h * 0x9E3779B97F4A7C15ull + (uint64_t)col * 0xC2B2AE3D27D4EB4Full + (uint64_t)nin[g];
            slot += pp;
        }
        c->slots[b] = slot;
        /* interchangeable groups: same column, same set of models (non-empty) */
        if (ng <= 256) {
            int64_t first_of[256];                     /* start of each group's models */
            int64_t at = pi;
            for (int64_t g = 0; g < ng; ++g) { first_of[g] = at; at += nin[g]; }
            uint8_t done[256];
            for (int64_t g = 0; g < ng; ++g) done[g] = 0;
            int32_t cls = 0;
            const int64_t first_item = n_items;
            int64_t perms = 1;
            for (int64_t g = 0; g < ng; ++g) {
                if (done[g] || nin[g] == 0) continue;
                int marked = 0, found = 0;
                for (int64_t h2 = g + 1; h2 < ng; ++h2) {
                    if (done[h2] || key[h2] != key[g] || nin[h2] != nin[g]) continue;
                    if (column_of[cfg_index[gi + h2]] != column_of[cfg_index[gi + g]]) continue;
                    if (!marked) {
                        for (int64_t k = 0; k < nin[g]; ++k) mark[placed_model[first_of[g] + k]] = gi + g;
                        marked = 1;
                    }
                    int same = 1;
                    for (int64_t k = 0; k < nin[h2] && same; ++k)
                        same = mark[placed_model[first_of[h2] + k]] == gi + g;
                    if (!same) continue;
                    if (!found) {
                        twin_items[3 * n_items] = (int32_t)b; twin_items[3 * n_items + 1] = cls;
                        twin_items[3 * n_items + 2] = (int32_t)g; ++n_items;
                        found = 1;
                    }
                    twin_items[3 * n_items] = (int32_t)b; twin_items[3 * n_items + 1] = cls;
                    twin_items[3 * n_items + 2] = (int32_t)h2; ++n_items;
                    done[h2] = 1;
                }
                if (found) {
                    int64_t size = 0;
                    for (int64_t k = n_items - 1; k >= first_item && twin_items[3 * k + 1] == cls; --k)
                        ++size;
                    for (int64_t k = 2; k <= size && perms <= max_perms; ++k) perms *= k;
                    ++cls;
                }
                if (perms > max_perms) break;
            }
            if (perms > max_perms) n_items = first_item;
        }
        pi = q;
        gi += ng;
    }
    *n_out = n_items;
    return 0;
}

struct encode_job {
    const struct encode_ctx *ctx;
    int64_t b0, b1, gi, pi, n_items;
    int64_t *scratch;          /* counts (M + 1) then mark (M) */
    int rc;
};

static void *encode_thread(void *arg)
{
    struct encode_job *j = (struct encode_job *)arg;
    j->rc = encode_range(j->ctx, j->b0, j->b1, j->gi, j->pi, j->scratch, j->scratch + j->ctx->M + 1,
                         &j->n_items);
    return NULL;
}

#define MMS_ENCODE_MAX_THREADS 8

int mms_host_encode(int64_t B, int64_t M, int64_t G, int64_t P,
                    const int64_t *n_groups, const int64_t *cfg, const int32_t *cfg_index,
                    const int64_t *column_of, const int64_t *n_in_group, const int64_t *placed_model,
                    uint16_t *model_off, uint32_t *model_rep, uint32_t *group_info,
                    int64_t *slots, int32_t *twin_items, int64_t *n_twin_items,
                    int64_t *counts, int64_t *mark, int64_t max_perms)
{
    struct encode_ctx ctx = {M, G, P, n_groups, cfg, column_of, n_in_group, placed_model, cfg_index,
                             model_off, model_rep, group_info, slots, twin_items, max_perms};
    /* placements are independent: a long list is cut into ranges, one thread each (the
     * caller holds the GIL; these threads touch no Python object) */
    int threads = mms_host_threads > 0 ? mms_host_threads : 4;
    if (threads > MMS_ENCODE_MAX_THREADS) threads = MMS_ENCODE_MAX_THREADS;
    if (B < 512 * threads) threads = (int)(B / 512);
    if (threads <= 1) return encode_range(&ctx, 0, B, 0, 0, counts, mark, n_twin_items);

    struct encode_job jobs[MMS_ENCODE_MAX_THREADS];
    pthread_t tid[MMS_ENCODE_MAX_THREADS];
    int64_t *scratch = (int64_t *)malloc(sizeof(int64_t) * (size_t)threads * (size_t)(2 * M + 1));
    if (!scratch) return encode_range(&ctx, 0, B, 0, 0, counts, mark, n_twin_items);
    int64_t gi = 0, pi = 0, b = 0;
    for (int t = 0; t < threads; ++t) {
        const int64_t b1 = (t + 1 == threads) ? B : B * (t + 1) / threads;
        jobs[t].ctx = &ctx; jobs[t].b0 = b; jobs[t].b1 = b1; jobs[t].gi = gi; jobs[t].pi = pi;
        jobs[t].n_items = 0; jobs[t].rc = 0;
        jobs[t].scratch = scratch + (size_t)t * (size_t)(2 * M + 1);
        for (; b < b1; ++b)
            for (int64_t g = 0; g < n_groups[b]; ++g) pi += n_in_group[gi++];
    }
    int started = 0;
    for (int t = 1; t < threads; ++t) {
        if (pthread_create(&tid[t], NULL, encode_thread, &jobs[t]) != 0) break;
        started = t;
    }
    encode_thread(&jobs[0]);
    for (int t = started + 1; t < threads; ++t) encode_thread(&jobs[t]);   /* threads that did not start */
    for (int t = 1; t <= started; ++t) pthread_join(tid[t], NULL);
    free(scratch);
    /* the ranges' twin items, one after the other */
    int64_t n_items = 0;
    int rc = 0;
    for (int t = 0; t < threads; ++t) {
        if (jobs[t].rc) rc = jobs[t].rc;
        if (jobs[t].n_items && 3 * jobs[t].gi != 3 * n_items)
            memmove(twin_items + 3 * n_items, twin_items + 3 * jobs[t].gi,
                    sizeof(int32_t) * 3 * (size_t)jobs[t].n_items);
        n_items += jobs[t].n_items;
    }
    *n_twin_items = n_items;
    return rc;
}
