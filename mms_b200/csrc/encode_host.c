/* encode_host.c — flattens a list of placements for the numpy encoder.
 *
 * Host-side helper of mms_b200/engine.py::encode_placements, loaded with
 * ctypes.PyDLL (the GIL stays held; no module object, no numpy C API: the
 * caller passes pointers to arrays it allocated).  It replaces the
 * per-object passes over 10^5 Python objects (group configs, model lists)
 * that dominated the encoding time; everything after the flattening stays
 * vectorised numpy.  A placement is any object with `group_configs` (a
 * sequence of (dp, op, pp) tuples, e.g. ParallelConfig namedtuples) and
 * `group_models` (a sequence of sequences of ints) —
 * alpa_serve/placement_policy/base_policy.py:18-27.
 *
 * Every function returns 0, or -1 with a Python exception set.
 */
#define PY_SSIZE_T_CLEAN
#include <Python.h>
#include <stdint.h>

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

static int as_int64(PyObject *o, int64_t *out)
{
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
