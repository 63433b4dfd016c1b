"""Host side of the GPU simulator: trace upload, placement encoding, launch.

The three steps mirror what the reference does per candidate in
alpa_serve/simulator/controller.py:410-503 (approximate_one_case_one_placement
builds m_id2g_id / num_stages / stage_latency, then calls the numba kernel),
but for a whole list of candidates at once and in the compact form that
include/mms_sim.h describes.  PyTorch is used for device memory and streams
only; all compute goes through the C ABI in libmms_sim.so.
"""
import ctypes
import operator
from itertools import chain, permutations, product
from math import factorial
from typing import List, Sequence

import numpy as np
import torch

from . import _native as nat
from .profiling import ParallelConfig

inf = 1e100      # alpa_serve/util.py:23
_PP = operator.itemgetter(2)     # pipeline degree of a ParallelConfig(dp, op, pp)


def _require_cuda():
    if not torch.cuda.is_available():
        raise RuntimeError("mms_b200 needs a CUDA device: the simulator has no CPU path")


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None and t.numel() > 0 else ctypes.c_void_p(0)


def _stream_ptr():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _to_device(arr: np.ndarray, device, pinned=False):
    t = torch.from_numpy(np.ascontiguousarray(arr))
    if pinned:
        t = t.pin_memory()
    return t.to(device, non_blocking=pinned)


_UPLOAD_STAGE = {}       # device -> page-locked staging buffer of _to_device_many
_UPLOAD_STAGE_MAX = 128 << 20


def _to_device_many(arrays, device):
    """Several host arrays to the device as ONE transfer from a page-locked staging
    buffer (kept per device): a launch uploads half a dozen small tables, and each
    transfer from pageable memory costs tens of microseconds whatever its size.
    Returns device tensors that are views of one buffer, each 16-byte aligned."""
    device = torch.device(device)
    arrays = [np.ascontiguousarray(a) for a in arrays]
    offsets, total = [], 0
    for a in arrays:
        offsets.append(total)
        total += (a.nbytes + 15) & ~15
    total = max(total, 16)
    if total > _UPLOAD_STAGE_MAX:         # not worth holding that much page-locked memory
        return [_to_device(a, device) for a in arrays]
    stage = _UPLOAD_STAGE.get(device)
    if stage is None or stage.numel() < total:
        stage = torch.empty(min(max(2 * total, 1 << 20), _UPLOAD_STAGE_MAX),
                            dtype=torch.uint8).pin_memory()
        _UPLOAD_STAGE[device] = stage
    host = stage.numpy()
    for a, o in zip(arrays, offsets):
        if a.nbytes:
            host[o:o + a.nbytes] = a.reshape(-1).view(np.uint8)
    buf = torch.empty(total, dtype=torch.uint8, device=device)
    buf.copy_(stage[:total])              # returns when the copy is done: the stage is free again
    out = []
    for a, o in zip(arrays, offsets):
        dtype = torch.from_numpy(np.empty(0, a.dtype)).dtype
        out.append(buf[o:o + a.nbytes].view(dtype).reshape(a.shape))
    return out


class DeviceTrace:
    """A request trace resident on one GPU: arrivals f64[N], model ids i32[N]
    (-1 = unknown model), SLOs f32[N] — the arrays controller.py:335-336
    caches per workload — plus what depends on the trace alone: the per-model
    request counts (controller.py:587) and numpy's summation plan for N."""

    def __init__(self, arrivals, model_ids, slos, num_models: int, device=None):
        _require_cuda()
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None \
            else torch.device(device)
        arrivals = np.ascontiguousarray(arrivals, dtype=np.float64)
        model_ids = np.ascontiguousarray(model_ids, dtype=np.int32)
        slos = np.ascontiguousarray(slos, dtype=np.float32)
        if not (len(arrivals) == len(model_ids) == len(slos)):
            raise ValueError("arrivals, model_ids and slos must have one entry per request")
        self.num_requests = int(len(arrivals))
        self.num_models = int(num_models)
        self.host_arrivals = arrivals
        self.h2d_bytes = arrivals.nbytes + model_ids.nbytes + slos.nbytes
        L = nat.lib()
        with torch.cuda.device(self.device):
            n_leaves = L.mms_sum_plan_leaves(self.num_requests)
            if n_leaves < 0:
                nat.check(n_leaves, "mms_sum_plan_leaves")
            leaf_start = np.zeros(n_leaves + 1, np.int32)
            leaf_merges = np.zeros(max(n_leaves, 1), np.uint8)
            nat.check(L.mms_sum_plan_fill(self.num_requests, leaf_start.ctypes.data,
                                          leaf_merges.ctypes.data), "mms_sum_plan_fill")
            self.num_leaves = n_leaves
            (self.arrivals, self.model_ids, self.slos, self.leaf_start,
             self.leaf_merges) = _to_device_many(
                (arrivals, model_ids, slos, leaf_start, leaf_merges), self.device)
            self.model_hist = torch.zeros(self.num_models + 1, dtype=torch.int32,
                                          device=self.device)
            tr = self.c_trace()
            nat.check(L.mms_trace_model_histogram(ctypes.byref(tr), self.num_models,
                                                  _ptr(self.model_hist), _stream_ptr()),
                      "mms_trace_model_histogram")

    def next_same_model(self):
        """i32[N] on the device: index of the next request with the same model
        (the per-model FIFO queues of the batching simulator run along it)."""
        if getattr(self, "_next_same", None) is None:
            with torch.cuda.device(self.device):
                buf = torch.empty(max(self.num_requests, 1), dtype=torch.int32,
                                  device=self.device)
                tr = self.c_trace()
                nat.check(nat.lib().mms_trace_next_same_model(
                    ctypes.byref(tr), self.num_models, _ptr(buf), _stream_ptr()),
                    "mms_trace_next_same_model")
            self._next_same = buf
        return self._next_same

    def c_trace(self):
        return nat.Trace(self.num_requests, _ptr(self.arrivals), _ptr(self.model_ids),
                         _ptr(self.slos))

    def c_plan(self):
        return nat.SumPlan(self.num_leaves, 0, _ptr(self.leaf_start), _ptr(self.leaf_merges))


class LazyArray:
    """A host array that is produced piece by piece, straight into an upload
    buffer: fill(out, lo, hi) writes elements [lo, hi) into `out` (a numpy view
    of hi - lo elements of `dtype`).  Saves the pass that would materialise it."""

    def __init__(self, size, dtype, fill):
        self.size, self.dtype, self.fill = int(size), np.dtype(dtype), fill

    def __len__(self):
        return self.size

    def materialize(self):
        out = np.empty(self.size, self.dtype)
        self.fill(out, 0, self.size)
        return out


class PinnedStager:
    """Uploads many host arrays through pinned staging buffers: a few threads
    copy pieces of the arrays into page-locked buffers (numpy copies run
    outside the interpreter lock) and enqueue the transfers from there, each on
    a stream of its own.  Pageable memory goes to the device at about a third
    of the rate of page-locked memory, whatever the number of threads that
    ask; staging by hand is what lets the threads help.  One instance per
    device is kept (page-locked allocations are slow)."""

    _instances = {}

    @classmethod
    def get(cls, dev, threads=8, piece_bytes=16 << 20):
        key = (torch.device(dev), threads, piece_bytes)
        if key not in cls._instances:
            cls._instances[key] = cls(*key)
        return cls._instances[key]

    def __init__(self, dev, threads, piece_bytes):
        from concurrent.futures import ThreadPoolExecutor
        self.device, self.threads, self.piece = torch.device(dev), int(threads), int(piece_bytes)
        self.pool = ThreadPoolExecutor(self.threads)
        self.streams = [torch.cuda.Stream(device=self.device) for _ in range(self.threads)]
        self.buffers = [[torch.empty(self.piece, dtype=torch.uint8).pin_memory() for _ in range(2)]
                        for _ in range(self.threads)]

    def upload(self, tasks):
        """tasks: [(device tensor, numpy array or LazyArray)] of equal byte sizes
        pairwise, contiguous.  Returns when every transfer has been enqueued;
        the current stream waits for them."""
        pieces = [[] for _ in range(self.threads)]
        load = [0] * self.threads
        for dst, src in tasks:
            d8 = dst.reshape(-1).view(torch.uint8)
            lazy = isinstance(src, LazyArray)
            if lazy:
                item, count = src.dtype.itemsize, src.size
            else:
                src = np.ascontiguousarray(src).reshape(-1)
                item, count = src.dtype.itemsize, src.size
            if d8.numel() != item * count:
                raise ValueError("upload: sizes differ")
            step = max(self.piece // item, 1)
            for lo in range(0, count, step):
                k = load.index(min(load))
                hi = min(lo + step, count)
                pieces[k].append((d8[lo * item:hi * item], src, lo, hi))
                load[k] += (hi - lo) * item
        main = torch.cuda.current_stream(self.device)

        def work(k):
            stream, bufs = self.streams[k], self.buffers[k]
            events = [None, None]
            stream.wait_stream(main)            # the destinations were allocated there
            with torch.cuda.device(self.device), torch.cuda.stream(stream):
                for j, (d8, src, lo, hi) in enumerate(pieces[k]):
                    if events[j & 1] is not None:
                        events[j & 1].synchronize()      # the buffer's last transfer is done
                    buf = bufs[j & 1][:d8.numel()]
                    view = buf.numpy().view(src.dtype)
                    if isinstance(src, LazyArray):
                        src.fill(view, lo, hi)
                    else:
                        np.copyto(view, src[lo:hi])
                    d8.copy_(buf, non_blocking=True)
                    ev = torch.cuda.Event()
                    ev.record(stream)
                    events[j & 1] = ev
            for ev in events:                   # the buffers are free for the next upload
                if ev is not None:
                    ev.synchronize()

        list(self.pool.map(work, [k for k in range(self.threads) if pieces[k]]))
        for k in range(self.threads):
            if pieces[k]:
                main.wait_stream(self.streams[k])


class DeviceTraceBatch:
    """T request traces resident on one GPU for runs in which every candidate
    has a trace of its own (one placement scored on many traces).  The traces
    are stored request-major ([N][T]: the 32 candidates of a warp read
    consecutive addresses) and padded to the longest one with requests of
    model -1 at the last arrival time, which change no clock and no counter.
    The host uploads every trace as it is, one after the other; the
    request-major batch is made on the device (mms_trace_pack).
    Duck-type compatible with DeviceTrace where launches are concerned."""

    def __init__(self, arrivals: Sequence, model_ids: Sequence, slos: Sequence, num_models: int,
                 device=None, staged=False):
        """staged: upload through PinnedStager (worth it from about a gigabyte)."""
        _require_cuda()
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None \
            else torch.device(device)
        T = len(arrivals)
        if T == 0 or not (len(model_ids) == len(slos) == T):
            raise ValueError("need one (arrivals, model_ids, slos) triple per trace")
        self.lengths = np.fromiter((len(a) for a in arrivals), np.int64, T)
        for t in range(T):
            if not (len(model_ids[t]) == len(slos[t]) == int(self.lengths[t])):
                raise ValueError(f"trace {t}: arrays differ in length")
        N = int(self.lengths.max())
        total = int(self.lengths.sum())
        self.num_traces, self.num_requests, self.num_models = T, N, int(num_models)
        offsets = np.concatenate(([0], np.cumsum(self.lengths))).astype(np.int64)
        self.h2d_bytes = total * 16 + offsets.nbytes
        L = nat.lib()
        dev = self.device
        with torch.cuda.device(dev):
            cat_arr = torch.empty(max(total, 1), dtype=torch.float64, device=dev)
            cat_mid = torch.empty(max(total, 1), dtype=torch.int32, device=dev)
            cat_slo = torch.empty(max(total, 1), dtype=torch.float32, device=dev)
            tasks = []
            for t in range(T):
                lo, hi = int(offsets[t]), int(offsets[t + 1])
                if hi > lo:
                    for dst, src, dtype in ((cat_arr, arrivals[t], np.float64),
                                            (cat_mid, model_ids[t], np.int32),
                                            (cat_slo, slos[t], np.float32)):
                        if isinstance(src, LazyArray):
                            if src.dtype != dtype:
                                raise ValueError("lazy trace array of the wrong type")
                            src = src if staged else src.materialize()
                        else:
                            src = np.ascontiguousarray(src, dtype)
                        tasks.append((dst[lo:hi], src))
            if staged:
                PinnedStager.get(dev).upload(tasks)
            else:
                for dst, src in tasks:
                    dst.copy_(torch.from_numpy(src), non_blocking=True)
            d_off = _to_device(offsets, dev)
            self.arrivals = torch.empty((max(N, 1), T), dtype=torch.float64, device=dev)
            self.model_ids = torch.empty((max(N, 1), T), dtype=torch.int32, device=dev)
            self.slos = torch.empty((max(N, 1), T), dtype=torch.float32, device=dev)
            nat.check(L.mms_trace_pack(_ptr(cat_arr), _ptr(cat_mid), _ptr(cat_slo), _ptr(d_off),
                                       T, N, _ptr(self.arrivals), _ptr(self.model_ids),
                                       _ptr(self.slos), _stream_ptr()), "mms_trace_pack")
            n_leaves = L.mms_sum_plan_leaves(N)
            if n_leaves < 0:
                nat.check(n_leaves, "mms_sum_plan_leaves")
            leaf_start = np.zeros(n_leaves + 1, np.int32)
            leaf_merges = np.zeros(max(n_leaves, 1), np.uint8)
            nat.check(L.mms_sum_plan_fill(N, leaf_start.ctypes.data, leaf_merges.ctypes.data),
                      "mms_sum_plan_fill")
            self.num_leaves = n_leaves
            self.leaf_start = _to_device(leaf_start, dev)
            self.leaf_merges = _to_device(leaf_merges, dev)
            # [T][M + 1] counts, then the total of unsorted positions (T == 1: plain [M + 1])
            cells = T * (self.num_models + 1) + (1 if T > 1 else 0)
            self.model_hist = torch.zeros(cells, dtype=torch.int32, device=dev)
            tr = self.c_trace()
            nat.check(L.mms_trace_model_histogram(ctypes.byref(tr), self.num_models,
                                                  _ptr(self.model_hist), _stream_ptr()),
                      "mms_trace_model_histogram")

    def c_trace(self):
        return nat.Trace(self.num_requests, _ptr(self.arrivals), _ptr(self.model_ids),
                         _ptr(self.slos), self.num_traces)

    def c_plan(self):
        return nat.SumPlan(self.num_leaves, 0, _ptr(self.leaf_start), _ptr(self.leaf_merges))


class LatencyTable:
    """stage latency per (model, parallel config, stage) in f32, with the
    0.9 %-per-stage penalty of controller.py:467-476 folded in.  Column c is
    the parallel config `configs[c]`; a config a model has no profile for is
    +inf (the f32 cast of 1e100), so such a replica never meets an SLO."""

    def __init__(self, prof_ress: Sequence, batch_sizes=None):
        """batch_sizes None: one latency per stage (batch size 1, table
        [M][C][S]); else the table gets a last axis over those batch sizes
        ([M][C][S][NB], controller.py:451-461)."""
        self.prof_ress = list(prof_ress)
        self.batch_sizes = None if batch_sizes is None else [int(b) for b in batch_sizes]
        self.configs: List = []
        self.column = {}
        self.max_stages = 1
        tail = () if batch_sizes is None else (len(self.batch_sizes),)
        self._host = np.zeros((len(self.prof_ress), 0, 1) + tail, np.float32)
        self._device = None

    def columns_for(self, configs) -> None:
        new = [c for c in dict.fromkeys(configs) if c not in self.column]
        if not new:
            return
        for c in new:
            self.column[c] = len(self.configs)
            self.configs.append(c)
        S = max([self.max_stages] + [int(c.pp) for c in new])
        M, C = len(self.prof_ress), len(self.configs)
        old = self._host
        tab = np.zeros((M, C, S) + old.shape[3:], np.float32)
        tab[:, :old.shape[1], :old.shape[2]] = old
        with np.errstate(over="ignore"):
            for m, prof in enumerate(self.prof_ress):
                for c in new:
                    col = self.column[c]
                    value = prof.para_dict.get(c, None)
                    if value:
                        penalty = 0.009 * len(value.latency[1])
                        for k in range(int(c.pp)):
                            if self.batch_sizes is None:
                                tab[m, col, k] = value.latency[1][k] * (1 + penalty)
                            else:
                                for j, bs in enumerate(self.batch_sizes):
                                    tab[m, col, k, j] = value.latency[bs][k] * (1 + penalty)
                    else:
                        tab[m, col] = np.float32(inf)
        self._host = tab
        self.max_stages = S
        self._device = None

    @property
    def host(self):
        return self._host

    def device(self, dev):
        """The table on `dev`; uploaded on the current stream when it changed,
        and any stream that asks for it waits for that upload."""
        if self._device is None or self._device.device != dev:
            self._device = _to_device(self._host, dev)
            self._ready = torch.cuda.Event()
            self._ready.record(torch.cuda.current_stream(dev))
        torch.cuda.current_stream(dev).wait_event(self._ready)
        return self._device


class EncodedBatch:
    """Host arrays of a placement batch in the layout of mms_placements."""

    def __init__(self, B, M, G, P, T, S, C, model_off, model_rep, group_info, num_groups,
                 num_replicas, twins=None):
        self.B, self.M, self.G, self.P, self.T, self.S, self.C = B, M, G, P, T, S, C
        self.model_off = model_off        # u16[B][M+1]
        self.model_rep = model_rep        # u32[B][P]
        self.group_info = group_info      # u32[B][G]
        self.num_groups = num_groups      # i64[B]
        self.num_replicas = num_replicas  # i64[B]: sum of len(group_models)
        # (candidate index, [[group ids of one class of interchangeable groups], ...])
        # for every placement that has such groups, see twin_groups()
        self.twins = twins
        self._mirror_table = None         # see mirror_table()

    def mirror_table(self):
        """(counts i64[len(twins)], words u64[sum(counts)]): the exchange lists of
        every placement's mirrors (mirror_swaps), placement after placement in the
        order of `twins`; made once, for all placements of one class pattern together."""
        if self._mirror_table is None:
            self._mirror_table = mirror_swaps_batch([classes for _, classes in (self.twins or [])])
        return self._mirror_table

    def take(self, index):
        """The sub-batch of the placements `index` (ascending)."""
        index = np.asarray(index, np.int64)
        new_id = np.full(self.B, -1, np.int64)
        new_id[index] = np.arange(len(index))
        keep = [k for k, (b, _) in enumerate(self.twins or []) if new_id[b] >= 0]
        twins = [(int(new_id[self.twins[k][0]]), self.twins[k][1]) for k in keep]
        sub = EncodedBatch(len(index), self.M, self.G, self.P, self.T, self.S, self.C,
                           self.model_off[index], self.model_rep[index], self.group_info[index],
                           self.num_groups[index], self.num_replicas[index], twins)
        if self._mirror_table is not None:
            counts, words = self._mirror_table
            keep = np.asarray(keep, np.int64)
            start = np.concatenate(([0], np.cumsum(counts)))[:-1]
            sub_counts = counts[keep]
            # the kept placements' stretches of `words`, one after the other
            pos = np.repeat(start[keep] - (np.cumsum(sub_counts) - sub_counts), sub_counts) \
                + np.arange(int(sub_counts.sum()))
            sub._mirror_table = (sub_counts, words[pos])
        return sub

    def repeat(self, count: int):
        """This batch `count` times over (placement 0 .. B-1, then again ...):
        the tables of one placement for `count` traces."""
        B = self.B
        twins = [(b + k * B, classes) for k in range(count) for b, classes in (self.twins or [])]
        return EncodedBatch(B * count, self.M, self.G, self.P, self.T, self.S, self.C,
                            np.tile(self.model_off, (count, 1)), np.tile(self.model_rep, (count, 1)),
                            np.tile(self.group_info, (count, 1)), np.tile(self.num_groups, count),
                            np.tile(self.num_replicas, count), twins)

    def with_mirrors(self):
        """The tables with mirror candidates appended for every placement
        that has interchangeable groups (see "Mirrors" in include/mms_sim.h),
        one per way of permuting them: (model_off, model_rep, group_info,
        partner i32[B'], mirror_swap u32[B'][2]) or None when no placement
        has any."""
        if not self.twins:
            return None
        counts, words = self.mirror_table()
        total = int(counts.sum())
        if total == 0:
            return None
        twin_b = np.fromiter((b for b, _ in self.twins), np.int64, len(self.twins))
        has = counts > 0
        first = self.B + np.cumsum(counts) - counts
        owners = np.repeat(twin_b, counts)
        at = self.B + total
        partner = np.full(at, -1, np.int32)
        partner[twin_b[has]] = first[has]
        partner[self.B:] = owners
        swap = np.full((at, 2), NO_SWAP, np.uint32)
        swap[self.B:] = words.view(np.uint32).reshape(-1, 2)
        return (np.concatenate((self.model_off, self.model_off[owners])),
                np.concatenate((self.model_rep, self.model_rep[owners])),
                np.concatenate((self.group_info, self.group_info[owners])), partner, swap)

    @property
    def nbytes(self):
        return self.model_off.nbytes + self.model_rep.nbytes + self.group_info.nbytes


NO_SWAP = np.uint32(0xFFFFFFFF)
_MODEL_KEYS = {}


MAX_MIRRORS = 15          # per placement
_PERM_CACHE = {}


def _perm_swaps(sizes):
    """Every non-identity way of permuting classes of the given sizes among
    themselves, each as a list of exchanges (i, j) of positions in the
    concatenated classes, at most four per permutation."""
    if sizes not in _PERM_CACHE:
        offsets = np.concatenate(([0], np.cumsum(sizes)))[:-1]
        per_class = []
        for off, n in zip(offsets, sizes):
            options = []
            for perm in permutations(range(n)):
                # exchanges that turn the identity arrangement into `perm`
                cur, ex = list(range(n)), []
                for i in range(n):
                    if cur[i] != perm[i]:
                        k = cur.index(perm[i])
                        cur[i], cur[k] = cur[k], cur[i]
                        ex.append((int(off) + i, int(off) + k))
                options.append(ex)
            per_class.append(options)
        out = []
        for combo in product(*per_class):
            ex = [e for part in combo for e in part]
            if ex and len(ex) <= 4:
                out.append(ex)
        _PERM_CACHE[sizes] = out
    return _PERM_CACHE[sizes]


def mirror_swaps(classes):
    """64-bit exchange lists (see mirror_swap in include/mms_sim.h) of the
    mirrors for one placement whose interchangeable groups are `classes`: one
    per permutation, or none at all when there are more than MAX_MIRRORS
    (covering only some would cost throughput without removing the serial
    repairs of the rest)."""
    sizes = tuple(len(c) for c in classes)
    count = 1
    for n in sizes:
        count *= factorial(n) if n < 5 else MAX_MIRRORS + 2
    if count - 1 > MAX_MIRRORS:
        return []
    groups = [g for c in classes for g in c]
    words = []
    for ex in _perm_swaps(sizes):
        w = 0xFFFFFFFFFFFFFFFF
        for k, (i, j) in enumerate(ex):
            w &= ~(0xFFFF << (16 * k))
            w |= (groups[i] | (groups[j] << 8)) << (16 * k)
        words.append(w)
    return words


def mirror_swaps_batch(class_lists):
    """mirror_swaps for many placements at once: (counts i64[n], words u64[sum])
    with the words of placement k at [sum(counts[:k]), sum(counts[:k + 1])), in
    the order mirror_swaps gives them.  Placements with the same class sizes
    share their permutations, so their words are formed together."""
    n = len(class_lists)
    counts = np.zeros(n, np.int64)
    by_sizes = {}
    for k, classes in enumerate(class_lists):
        by_sizes.setdefault(tuple(map(len, classes)), []).append(k)
    made = {}
    for sizes, members in by_sizes.items():
        ways = 1
        for size in sizes:
            ways *= factorial(size) if size < 5 else MAX_MIRRORS + 2
        if ways - 1 > MAX_MIRRORS:
            continue
        perms = _perm_swaps(sizes)
        if not perms:
            continue
        groups = np.array([[g for c in class_lists[k] for g in c] for k in members], np.uint64)
        words = np.empty((len(members), len(perms)), np.uint64)
        for q, ex in enumerate(perms):
            w = np.full(len(members), 0xFFFFFFFFFFFFFFFF, np.uint64)
            for t, (i, j) in enumerate(ex):
                w &= np.uint64(~(0xFFFF << (16 * t)) & 0xFFFFFFFFFFFFFFFF)
                w |= (groups[:, i] | (groups[:, j] << np.uint64(8))) << np.uint64(16 * t)
            words[:, q] = w
        counts[members] = len(perms)
        made[sizes] = (np.asarray(members, np.int64), words)
    out = np.empty(int(counts.sum()), np.uint64)
    start = np.cumsum(counts) - counts
    for members, words in made.values():
        pos = start[members][:, None] + np.arange(words.shape[1])[None, :]
        out[pos] = words
    return counts, out


def _arrangements(classes) -> int:
    count = 1
    for cls in classes:
        count *= factorial(len(cls)) if len(cls) < 5 else MAX_MIRRORS + 2
    return count


def twin_groups(B, M, grp_b, grp_g, cfg_col, n_in_group, placed_model):
    """Classes of groups of one placement with the same parallel config and
    the same set of models (flat arrays as in encode_placements).  Such groups
    are interchangeable: which of them is ahead after a stretch of the trace
    depends on history long past, and a speculative chunk may come out with
    their roles permuted.  Returns [(placement index, [[group ids], ...])] for
    the placements that have any and at most MAX_MIRRORS + 1 ways of arranging
    them.  The sets are compared through a 64-bit sum
    of random per-model keys; a collision could only cost speed, never
    exactness."""
    tot_groups = len(grp_b)
    if tot_groups < 2 or len(placed_model) == 0:
        return []
    if M not in _MODEL_KEYS:
        _MODEL_KEYS[M] = np.random.RandomState(20240229).randint(
            1, 2 ** 62, size=max(M, 1), dtype=np.int64).astype(np.uint64)
    with np.errstate(over="ignore"):
        csum = np.concatenate((np.zeros(1, np.uint64),
                               np.cumsum(_MODEL_KEYS[M][placed_model], dtype=np.uint64)))
        ends = np.cumsum(n_in_group)
        key = (csum[ends] - csum[ends - n_in_group]) * np.uint64(0x9E3779B97F4A7C15) \
            + cfg_col.astype(np.uint64) * np.uint64(0xC2B2AE3D27D4EB4F) + n_in_group.astype(np.uint64)
    # keys as a [B][G] matrix (unused cells and empty groups get keys of their own: top bit
    # set, which no hash has), each row sorted on its own: equal neighbours are a class
    G = int(grp_g.max()) + 1
    mat = (np.arange(B * G, dtype=np.uint64) | np.uint64(1 << 63)).reshape(B, G)
    live = n_in_group > 0
    mat[grp_b[live], grp_g[live]] = key[live] & np.uint64((1 << 63) - 1)
    order = np.argsort(mat, axis=1)
    srt = np.take_along_axis(mat, order, axis=1)
    same = srt[:, 1:] == srt[:, :-1]
    rows, cols = np.nonzero(same)                     # sorted by row, then column
    lo_ids = order[rows, cols].tolist()
    hi_ids = order[rows, cols + 1].tolist()
    out = []
    prev_b, prev_c = -1, -2
    for b, c, g_lo, g_hi in zip(rows.tolist(), cols.tolist(), lo_ids, hi_ids):
        if b != prev_b:
            out.append((b, []))
        if b == prev_b and c == prev_c + 1:
            out[-1][1][-1].append(g_hi)                # the run of equal keys goes on
        else:
            out[-1][1].append([g_lo, g_hi])
        prev_b, prev_c = b, c
    for _, classes in out:
        for cls in classes:
            cls.sort()
    # placements with more arrangements than get mirrors are of no use to anyone
    return [(b, classes) for b, classes in out if _arrangements(classes) <= MAX_MIRRORS + 1]


def _flatten(placements):
    """(groups per placement i64[B], configs i64[groups][3] = (dp, op, pp),
    models per group i64[groups], the models of all groups i64[pairs]) in
    placement order: by the C helper when it is built, else by passes over the
    Python objects."""
    B = len(placements)
    H = nat.host_lib()
    if H is not None and isinstance(placements, (list, tuple)):
        n_groups = np.zeros(B, np.int64)
        n_pairs = np.zeros(B, np.int64)
        # one pass with room for 96 groups and 256 (group, model) pairs per placement
        # (untouched room costs nothing) ...
        cap_g, cap_p = 96 * B + 64, 256 * B + 256
        cfg = np.empty((cap_g, 3), np.int64)
        n_in_group = np.empty(cap_g, np.int64)
        placed_model = np.empty(cap_p, np.int64)
        totals = np.zeros(2, np.int64)
        rc = H.mms_host_flatten_once(placements, n_groups.ctypes.data, n_pairs.ctypes.data,
                                     cfg.ctypes.data, n_in_group.ctypes.data,
                                     placed_model.ctypes.data, cap_g, cap_p, totals.ctypes.data)
        if rc == 0:
            tg, tp = int(totals[0]), int(totals[1])
            return n_groups, cfg[:tg], n_in_group[:tg], placed_model[:tp]
        if rc != -2:
            raise RuntimeError("mms_host_flatten_once failed")   # a Python exception is normally set
        # ... else count first, then fill
        if H.mms_host_scan(placements, n_groups.ctypes.data, n_pairs.ctypes.data) != 0:
            raise RuntimeError("mms_host_scan failed")
        tot_groups, tot_placed = int(n_groups.sum()), int(n_pairs.sum())
        cfg = np.zeros((tot_groups, 3), np.int64)
        n_in_group = np.zeros(tot_groups, np.int64)
        placed_model = np.zeros(tot_placed, np.int64)
        if H.mms_host_flatten(placements, cfg.ctypes.data, n_in_group.ctypes.data,
                              placed_model.ctypes.data, tot_groups, tot_placed) != 0:
            raise RuntimeError("mms_host_flatten failed")
        return n_groups, cfg, n_in_group, placed_model
    all_cfgs = list(chain.from_iterable(p.group_configs for p in placements))
    all_groups = list(chain.from_iterable(p.group_models for p in placements))
    n_groups = np.fromiter(map(len, (p.group_configs for p in placements)), np.int64, B)
    tot_groups = len(all_cfgs)
    if len(all_groups) != tot_groups:
        raise ValueError("group_configs and group_models differ in length")
    cfg = np.fromiter(chain.from_iterable(c[:3] for c in all_cfgs), np.int64,
                      3 * tot_groups).reshape(tot_groups, 3)
    n_in_group = np.fromiter(map(len, all_groups), np.int64, tot_groups)
    placed_model = np.fromiter(chain.from_iterable(all_groups), np.int64, int(n_in_group.sum()))
    return n_groups, cfg, n_in_group, placed_model


def _too_large(G, T, S, C):
    if G > nat.MAX_GROUPS or T > nat.MAX_SLOTS or S > nat.MAX_STAGES or C > nat.MAX_COLUMNS:
        raise NotImplementedError(
            f"placement too large for the kernels: {G} groups (max {nat.MAX_GROUPS}), "
            f"{T} pipeline stages in total (max {nat.MAX_SLOTS}), {C} parallel configs "
            f"(max {nat.MAX_COLUMNS})")


def _encode_native(H, B, M, table, n_groups, cfg, n_in_group, placed_model) -> EncodedBatch:
    """encode_placements behind the flattening, by csrc/encode_host.c."""
    tot_groups = len(n_in_group)
    cfg = np.ascontiguousarray(cfg)
    uniq = np.zeros((nat.MAX_COLUMNS + 1, 3), np.int64)
    cfg_index = np.zeros(max(tot_groups, 1), np.int32)
    n_uniq = H.mms_host_configs(cfg.ctypes.data, tot_groups, uniq.ctypes.data, len(uniq),
                                cfg_index.ctypes.data)
    if n_uniq < 0:
        raise NotImplementedError(f"more than {nat.MAX_COLUMNS} parallel configs in one batch")
    # new columns are handed out in ascending (dp, op, pp)
    found = [ParallelConfig(*map(int, row)) for row in uniq[:n_uniq]]
    table.columns_for(sorted(found))
    column_of = np.fromiter(map(table.column.__getitem__, found), np.int64, n_uniq)
    G = int(n_groups.max()) if B else 0
    S, C = int(table.max_stages), len(table.configs)
    _too_large(G, 0, S, C)
    # pairs per placement: the sums of n_in_group over each placement's groups
    ends = np.cumsum(n_groups)
    csum = np.concatenate(([0], np.cumsum(n_in_group)))
    placed_per_b = csum[ends] - csum[ends - n_groups] if B else np.zeros(0, np.int64)
    P = int(placed_per_b.max()) if B else 0
    if P > nat.MAX_PLACED:
        raise NotImplementedError(f"{P} (group, model) pairs in one placement (max {nat.MAX_PLACED})")
    Gc, Pc = max(G, 1), max(P, 1)
    model_off = np.zeros((B, M + 1), np.uint16)
    model_rep = np.zeros((B, Pc), np.uint32)
    group_info = np.zeros((B, Gc), np.uint32)
    slots = np.zeros(max(B, 1), np.int64)
    items = np.empty((max(tot_groups, 1), 3), np.int32)
    n_items = np.zeros(1, np.int64)
    counts = np.zeros(M + 1, np.int64)
    mark = np.zeros(max(M, 1), np.int64)
    n_groups = np.ascontiguousarray(n_groups, np.int64)
    rc = H.mms_host_encode(B, M, Gc, Pc, n_groups.ctypes.data, cfg.ctypes.data,
                           cfg_index.ctypes.data, column_of.ctypes.data, n_in_group.ctypes.data,
                           placed_model.ctypes.data, model_off.ctypes.data, model_rep.ctypes.data,
                           group_info.ctypes.data, slots.ctypes.data, items.ctypes.data,
                           n_items.ctypes.data, counts.ctypes.data, mark.ctypes.data,
                           MAX_MIRRORS + 1)
    if rc == 1:
        raise IndexError("model id in group_models is out of range")
    T = int(slots[:B].max()) if B else 0
    _too_large(G, T, S, C)
    twins = []
    prev_b, prev_c = -1, -1
    for b, c, g in items[:int(n_items[0])].tolist():
        if b != prev_b:
            twins.append((b, []))
            prev_c = -1
        if c != prev_c:
            twins[-1][1].append([])
        twins[-1][1][-1].append(g)
        prev_b, prev_c = b, c
    return EncodedBatch(B, M, Gc, Pc, max(T, 1), S, C, model_off, model_rep, group_info,
                        n_groups, placed_per_b.astype(np.int64), twins)


def encode_placements(placements: Sequence, table: LatencyTable, num_models: int,
                      native: bool = True) -> EncodedBatch:
    """List of ModelPlacement -> compact tables.  Each placement is taken as
    given: group order decides dispatch ties (controller.py:596 is a strict
    '<' over groups in ascending id), so nothing is re-sorted.  With the host
    helper built (and `native`), one C pass makes the tables; else numpy does."""
    B = len(placements)
    M = int(num_models)
    n_groups, cfg, n_in_group, placed_model = _flatten(placements)
    tot_groups, tot_placed = len(n_in_group), len(placed_model)
    H = nat.host_lib() if native else None
    if H is not None:
        return _encode_native(H, B, M, table, n_groups, cfg, n_in_group, placed_model)
    # distinct (dp, op, pp) rows -> columns of the latency table
    cfg_key = (cfg[:, 0] << 40) | (cfg[:, 1] << 20) | cfg[:, 2]
    uniq, inverse = np.unique(cfg_key, return_inverse=True)
    uniq_cfgs = [ParallelConfig(int(k >> 40), int((k >> 20) & 0xFFFFF), int(k & 0xFFFFF))
                 for k in uniq]
    table.columns_for(uniq_cfgs)
    cfg_col = np.fromiter(map(table.column.__getitem__, uniq_cfgs), np.int64,
                          len(uniq_cfgs))[inverse] if tot_groups else np.zeros(0, np.int64)
    cfg_pp = cfg[:, 2].copy()
    if tot_placed and (placed_model.min() < 0 or placed_model.max() >= M):
        raise IndexError("model id in group_models is out of range")

    G = int(n_groups.max()) if B else 0
    grp_first = np.concatenate(([0], np.cumsum(n_groups)))[:-1]     # first flat group of b
    grp_b = np.repeat(np.arange(B), n_groups)                       # candidate of flat group
    grp_g = np.arange(tot_groups) - grp_first[grp_b]                # group id inside b
    # clock slots: exclusive prefix sum of stages inside each candidate
    csum = np.cumsum(cfg_pp)
    base = np.concatenate(([0], csum))[grp_first]
    slot_first = (csum - cfg_pp) - base[grp_b]
    slots_per_b = np.bincount(grp_b, weights=cfg_pp, minlength=B).astype(np.int64)
    T = int(slots_per_b.max()) if B else 0
    S = int(table.max_stages)
    C = len(table.configs)
    _too_large(G, T, S, C)

    # (candidate, model, group) triples, ordered by model then group inside b
    pl_grp = np.repeat(np.arange(tot_groups), n_in_group)           # flat group of each pair
    pl_b = grp_b[pl_grp]
    pl_g = grp_g[pl_grp]
    # one composite key: by candidate, then model, then group id
    order = np.argsort((pl_b * max(M, 1) + placed_model) * (G + 1) + pl_g)      # keys are unique
    pl_b, pl_g, pl_m, pl_grp = pl_b[order], pl_g[order], placed_model[order], pl_grp[order]
    placed_per_b = np.bincount(pl_b, minlength=B) if tot_placed else np.zeros(B, np.int64)
    P = int(placed_per_b.max()) if B else 0
    if P > nat.MAX_PLACED:
        raise NotImplementedError(f"{P} (group, model) pairs in one placement (max {nat.MAX_PLACED})")
    pair_first = np.concatenate(([0], np.cumsum(placed_per_b)))[:-1]
    pos = np.arange(tot_placed) - pair_first[pl_b]
    model_rep = np.zeros((B, max(P, 1)), np.uint32)
    model_rep[pl_b, pos] = (pl_g | (slot_first[pl_grp] << 8) | (cfg_pp[pl_grp] << 16)
                            | (cfg_col[pl_grp] << 24)).astype(np.uint32)
    counts = np.bincount(pl_b * (M + 1) + pl_m + 1, minlength=B * (M + 1)).reshape(B, M + 1)
    model_off = np.cumsum(counts, axis=1).astype(np.uint16)
    # a group is contested when one of its models has more than one replica
    replicas = counts[pl_b, pl_m + 1]
    contested = (np.bincount(pl_grp, weights=(replicas > 1), minlength=tot_groups) > 0
                 ).astype(np.int64)
    group_info = np.zeros((B, max(G, 1)), np.uint32)
    group_info[grp_b, grp_g] = (slot_first | (cfg_pp << 8) | (contested << 16)).astype(np.uint32)

    twins = twin_groups(B, M, grp_b, grp_g, cfg_col, n_in_group, placed_model)
    return EncodedBatch(B, M, max(G, 1), max(P, 1), max(T, 1), S, C, model_off, model_rep,
                        group_info, n_groups, placed_per_b.astype(np.int64), twins)


class BatchResult:
    """Outputs of one launch, as numpy arrays on the host."""
    __slots__ = ("model_num_requests", "model_num_good", "group_num_requests",
                 "group_num_good", "good_total", "latency_sum", "status", "finish", "good",
                 "resimulated", "finish_device", "good_device")

    def __init__(self):
        # per-request outputs left on the GPU (f64[B][N], u8[B][N]) when a caller asked for that
        self.finish_device = self.good_device = None

    @staticmethod
    def concatenate(parts):
        """Results of consecutive sub-batches as one (per-request outputs are
        not carried); group columns are padded to the widest part."""
        res = BatchResult()
        G = max(p.group_num_requests.shape[1] for p in parts)

        def wide(a):
            return np.pad(a, ((0, 0), (0, G - a.shape[1])))
        res.model_num_requests = np.concatenate([p.model_num_requests for p in parts])
        res.model_num_good = np.concatenate([p.model_num_good for p in parts])
        res.group_num_requests = np.concatenate([wide(p.group_num_requests) for p in parts])
        res.group_num_good = (np.concatenate([wide(p.group_num_good) for p in parts])
                              if parts[0].group_num_good is not None else None)
        for name in ("good_total", "latency_sum", "status", "resimulated"):
            setattr(res, name, np.concatenate([getattr(p, name) for p in parts]))
        res.finish = res.good = None
        return res


class BatchSummary:
    """What callers read from an encoded batch after evaluation, for a batch
    that was encoded and launched in several parts."""

    def __init__(self, encs):
        self.parts = encs
        self.B = sum(e.B for e in encs)
        self.num_groups = np.concatenate([e.num_groups for e in encs])
        self.num_replicas = np.concatenate([e.num_replicas for e in encs])


def sim_options(chunk_requests=0, warmup_requests=0, repair_rounds=0, repair_segments=0):
    """How the trace is cut for time-parallel execution (mms_sim_options):
    0 lets the library choose, chunk_requests < 0 forces one chunk.  Results
    never depend on these numbers, only the run time does."""
    return nat.SimOptions(int(chunk_requests), int(warmup_requests), int(repair_rounds),
                          int(repair_segments))


class _Pending:
    """A submitted launch: device tensors and what collect() needs."""
    __slots__ = ("keep", "out", "B", "Bs", "M", "N", "full", "want_group_good", "h2d", "stream",
                 "scratch", "call", "trace")


# Scratch buffers of finished launches, per device, kept for the next ones: a
# search scores batch after batch of slowly changing size, and a fresh
# cudaMalloc for each would cost more than the kernels.  A buffer is handed to
# one launch at a time (taken in _submit, returned in _collect).
_SCRATCH_POOL = {}


def _take_scratch(dev, need):
    pool = _SCRATCH_POOL.setdefault(dev, [])
    fits = [k for k, t in enumerate(pool) if t.numel() >= need]
    if fits:
        return pool.pop(min(fits, key=lambda k: pool[k].numel()))
    if pool:                       # grow instead of hoarding: drop the largest idle one
        pool.pop(max(range(len(pool)), key=lambda k: pool[k].numel()))
    return torch.empty(max(int(need * 1.25), 1 << 20), dtype=torch.uint8, device=dev)


def _return_scratch(dev, t):
    pool = _SCRATCH_POOL.setdefault(dev, [])
    if len(pool) < 8:
        pool.append(t)


def _submit(trace: DeviceTrace, B, M, G, P, T, S, C, model_off, model_rep, group_info,
            latency, latency_stride, flags, want_group_good, pinned=False, options=None,
            num_scored=None, partner=None, mirror_swap=None) -> _Pending:
    """Uploads the tables and enqueues mms_sim_mixed on the current stream;
    nothing waits for the GPU.  With num_scored < B the candidates behind the
    first num_scored are mirrors (partner, mirror_swap as in mms_placements)
    and get no results."""
    job = _prepare(trace, B, M, G, P, T, S, C, model_off, model_rep, group_info, latency,
                   latency_stride, flags, want_group_good, pinned, options, num_scored, partner,
                   mirror_swap)
    _enqueue(job)
    return job


def _enqueue(job: _Pending):
    """The C call of a prepared launch, on the current stream (again and
    again, if the caller wishes: everything it reads stays on the device)."""
    trace = job.trace
    cands, opts, ws, out, flags = job.call
    with torch.cuda.device(trace.device):
        tr, plan = trace.c_trace(), trace.c_plan()
        rc = nat.lib().mms_sim_mixed(ctypes.byref(tr), ctypes.byref(cands), ctypes.byref(plan),
                                     _ptr(trace.model_hist), ctypes.byref(opts), ctypes.byref(ws),
                                     ctypes.byref(out), flags, _stream_ptr())
        nat.check(rc, "mms_sim_mixed")
        job.stream = torch.cuda.current_stream()


def _prepare(trace: DeviceTrace, B, M, G, P, T, S, C, model_off, model_rep, group_info,
             latency, latency_stride, flags, want_group_good, pinned=False, options=None,
             num_scored=None, partner=None, mirror_swap=None) -> _Pending:
    """Uploads the tables and allocates scratch and outputs of one launch."""
    _require_cuda()
    L = nat.lib()
    dev = trace.device
    N = trace.num_requests
    opts = options if options is not None else sim_options()
    if not want_group_good:
        flags |= nat.FLAG_NO_GROUP_GOOD
    job = _Pending()
    with torch.cuda.device(dev):
        h2d = model_off.nbytes + model_rep.nbytes + group_info.nbytes
        Bs = B if num_scored is None else int(num_scored)
        d_partner = d_swap = None
        if pinned:
            d_off = _to_device(model_off, dev, pinned)
            d_rep = _to_device(model_rep, dev, pinned)
            d_info = _to_device(group_info, dev, pinned)
            if Bs != B:
                d_partner = _to_device(partner, dev, pinned)
                d_swap = _to_device(mirror_swap, dev, pinned)
        elif Bs != B:
            d_off, d_rep, d_info, d_partner, d_swap = _to_device_many(
                (model_off, model_rep, group_info, partner, mirror_swap), dev)
        else:
            d_off, d_rep, d_info = _to_device_many((model_off, model_rep, group_info), dev)
        if Bs != B:
            h2d += partner.nbytes + mirror_swap.nbytes
        d_lat = latency if isinstance(latency, torch.Tensor) else _to_device(latency, dev, pinned)
        cands = nat.Placements(B, M, G, P, T, S, C, Bs if Bs != B else 0, _ptr(d_off), _ptr(d_rep),
                               _ptr(d_info), _ptr(d_lat), int(latency_stride), _ptr(d_partner),
                               _ptr(d_swap))
        need = L.mms_sim_workspace_bytes(N, ctypes.byref(cands), ctypes.byref(opts), flags)
        if need == 0 and B > 0:
            raise NotImplementedError("placement batch outside the kernel limits "
                                      "(see MMS_MAX_* in include/mms_sim.h)")
        ws_t = _take_scratch(dev, max(need, 256))
        ws = nat.Workspace(_ptr(ws_t), need)
        i32 = dict(dtype=torch.int32, device=dev)
        rows = max(Bs, 1)
        o_mreq = torch.empty((rows, max(M, 1)), **i32)
        o_mgood = torch.empty((rows, max(M, 1)), **i32)
        o_greq = torch.empty((rows, G), **i32)
        o_ggood = torch.empty((rows, G), **i32) if want_group_good else None
        o_total = torch.empty(rows, dtype=torch.int64, device=dev)
        o_lsum = torch.empty(rows, dtype=torch.float64, device=dev)
        o_status = torch.zeros(rows, dtype=torch.int32, device=dev)
        o_redo = torch.zeros(rows, dtype=torch.int32, device=dev)
        full = bool(flags & nat.FLAG_PER_REQUEST)
        o_fin = torch.empty((rows, max(N, 1)), dtype=torch.float64, device=dev) if full else None
        o_good = torch.empty((rows, max(N, 1)), dtype=torch.uint8, device=dev) if full else None
        out = nat.Results(_ptr(o_mreq), _ptr(o_mgood), _ptr(o_greq), _ptr(o_ggood),
                          _ptr(o_total), _ptr(o_lsum), _ptr(o_status), _ptr(o_fin), _ptr(o_good),
                          _ptr(o_redo))
        job.stream = torch.cuda.current_stream()
    job.call = (cands, opts, ws, out, flags)
    job.trace = trace
    job.keep = (d_off, d_rep, d_info, d_lat, d_partner, d_swap)
    job.scratch = ws_t
    job.out = (o_mreq, o_mgood, o_greq, o_ggood, o_total, o_lsum, o_status, o_redo, o_fin, o_good)
    job.B, job.Bs, job.M, job.N, job.full = B, Bs, M, N, full
    job.want_group_good, job.h2d = want_group_good, h2d
    return job


def _download(job: _Pending, rows_on_device=False):
    """Waits for the launch and copies its results to the host.  Returns
    (BatchResult, d2h_bytes).  rows_on_device: the per-request outputs are not
    downloaded; the result carries the device tensors instead."""
    (o_mreq, o_mgood, o_greq, o_ggood, o_total, o_lsum, o_status, o_redo, o_fin, o_good) = job.out
    Bs, M, N, full = job.Bs, job.M, job.N, job.full
    res = BatchResult()
    with torch.cuda.stream(job.stream):
        res.model_num_requests = o_mreq[:Bs].cpu().numpy()[:, :M]
        res.model_num_good = o_mgood[:Bs].cpu().numpy()[:, :M]
        res.group_num_requests = o_greq[:Bs].cpu().numpy()
        res.group_num_good = o_ggood[:Bs].cpu().numpy() if job.want_group_good else None
        res.good_total = o_total[:Bs].cpu().numpy()
        res.latency_sum = o_lsum[:Bs].cpu().numpy()
        res.status = o_status[:Bs].cpu().numpy().astype(np.uint32)
        res.resimulated = o_redo[:Bs].cpu().numpy()
        host_rows = full and not rows_on_device
        res.finish = o_fin[:Bs].cpu().numpy()[:, :N] if host_rows else None
        res.good = o_good[:Bs].cpu().numpy()[:, :N].astype(bool) if host_rows else None
        if full and rows_on_device:
            res.finish_device, res.good_device = o_fin[:Bs, :N], o_good[:Bs, :N]
    d2h = sum(x.nbytes for x in (res.model_num_requests, res.model_num_good,
                                 res.group_num_requests, res.good_total, res.latency_sum,
                                 res.status))
    if host_rows:
        d2h += res.finish.nbytes + res.good.nbytes
    return res, d2h


def _release(job: _Pending):
    """Hands the scratch buffer back; every kernel that used it has finished."""
    job.keep = job.out = job.call = None
    if job.scratch is not None:
        _return_scratch(job.scratch.device, job.scratch)
        job.scratch = None


def _check_status(res):
    if np.any(res.status):
        bad = int(np.flatnonzero(res.status)[0])
        raise RuntimeError(f"simulator kernel reported status {int(res.status[bad])} "
                           f"for candidate {bad} (bad table index or capacity overflow)")


def _collect(job, rows_on_device=False):
    """Waits for a submitted launch and downloads its results.  Returns
    (BatchResult, h2d_bytes, d2h_bytes)."""
    if isinstance(job, ResidentBatch):
        res, d2h = job.results()
        h2d = job.h2d_bytes
        job.release()
        _check_status(res)
        return res, h2d, d2h
    res, d2h = _download(job, rows_on_device)
    h2d = job.h2d
    _release(job)
    _check_status(res)
    return res, h2d, d2h


def _launch(*args, rows_on_device=False, **kwargs):
    """_submit + _collect: uploads the tables, runs mms_sim_mixed on the current
    stream, downloads the results.  Returns (BatchResult, h2d_bytes, d2h_bytes)."""
    return _collect(_submit(*args, **kwargs), rows_on_device)


SPLIT_MIN_EASY = 512      # placements without mirrors a batch must have to be split
SPLIT_MIN_HARD = 32       # ... and placements with mirrors
# Run-in of the launch that holds the placements with mirrors, when a batch is split (the
# library's default is 2048): the few chunks of these placements that no stored run continues
# are re-simulated one after the other by single lanes, and the longest such chain decides when
# the launch ends.  A longer run-in makes its speculative pass longer (which delays the other
# launch's) and those chains shorter.  Measured over four candidate lists, slowest / mean step:
# 24.7 / 22.6 ms with 2048, 22.6 / 22.0 ms with 2560, 22.9 / 22.3 ms with 3072.
HARD_RUN_IN = 2560
_SIDE_STREAMS = {}


def _side_streams(main):
    """Two side streams per calling stream, so that batches launched from
    different streams do not queue up behind each other."""
    key = (main.device, main.cuda_stream)
    if key not in _SIDE_STREAMS:
        _SIDE_STREAMS[key] = (torch.cuda.Stream(device=main.device),
                              torch.cuda.Stream(device=main.device))
    return _SIDE_STREAMS[key]


class ResidentBatch:
    """An encoded batch with its tables, scratch and outputs on the GPU, ready
    to be launched (any number of times).

    A batch whose placements partly have mirrors is launched as TWO calls of
    mms_sim_mixed on two side streams: the placements with mirrors first, cut
    into many short chunks, and the rest beside them.  The first finish their
    speculative pass early, and their repair rounds — a few long, serial
    re-simulations that leave the GPU almost idle — run while the rest are
    still in theirs.  Results are the same as from one call."""

    def __init__(self, trace, enc: EncodedBatch, table: LatencyTable, group_good=False,
                 pinned=False, options=None, mirrors=True, split=True, crowded=False,
                 hard_options=None, launch_now=False):
        """crowded: other launches will be filling the GPU while this batch
        repairs its chunks (a pipelined part that is not the last).
        hard_options: sim_options for the launch that holds the placements with
        mirrors, when the batch is split (default: `options`).
        launch_now: every call is enqueued as soon as its tables are uploaded
        (as launch() would afterwards), so that the GPU starts on the first
        while the host prepares the second."""
        self.trace, self.enc = trace, enc
        dev = trace.device
        ext_owner = []
        if mirrors and enc.twins:
            counts, _ = enc.mirror_table()
            ext_owner = [b for (b, _), c in zip(enc.twins, counts.tolist()) if c]
        parts = [(None, enc)]
        if (split and len(ext_owner) >= SPLIT_MIN_HARD
                and enc.B - len(ext_owner) >= SPLIT_MIN_EASY):
            hard = np.asarray(ext_owner, np.int64)
            rest = np.ones(enc.B, bool)
            rest[hard] = False
            easy = np.flatnonzero(rest)
            parts = [(hard, enc.take(hard)), (easy, enc.take(easy))]
        self.index = [p[0] for p in parts]
        self.jobs = []
        self.h2d_bytes = 0
        self.launched = False
        lat = table.device(dev)
        main = sides = None
        if launch_now and len(parts) > 1:
            main = torch.cuda.current_stream(dev)
            sides = _side_streams(main)
        for k, (_, e) in enumerate(parts):
            # the first of two calls repairs while the second one fills the GPU
            flags = nat.FLAG_CROWDED if (crowded or k + 1 < len(parts)) else 0
            # (the second of two parts holds the placements without mirrors)
            ext = e.with_mirrors() if mirrors and not (len(parts) > 1 and k == 1) else None
            opts_k = options
            if len(parts) > 1 and k == 0:
                if hard_options is not None:
                    opts_k = hard_options
                elif options is None or options.warmup_requests == 0:
                    o = options if options is not None else sim_options()
                    opts_k = sim_options(o.chunk_requests, HARD_RUN_IN, o.repair_rounds,
                                         o.repair_segments)
            if ext is not None:
                off, rep, info, partner, swap = ext
                job = _prepare(trace, len(partner), e.M, e.G, e.P, e.T, e.S, e.C, off, rep, info,
                               lat, 0, flags, group_good, pinned, opts_k, e.B, partner, swap)
            else:
                job = _prepare(trace, e.B, e.M, e.G, e.P, e.T, e.S, e.C, e.model_off, e.model_rep,
                               e.group_info, lat, 0, flags, group_good, pinned, opts_k)
            self.jobs.append(job)
            self.h2d_bytes += job.h2d
            if launch_now:              # the GPU starts on this call while the next is prepared
                if sides is None:
                    _enqueue(job)
                else:
                    sides[k].wait_stream(main)
                    with torch.cuda.stream(sides[k]):
                        _enqueue(job)
        if launch_now:
            if sides is not None:
                for side in sides:
                    main.wait_stream(side)
                for job in self.jobs:   # results are read in order behind the join
                    job.stream = main
            self.launched = True

    def launch(self):
        """Enqueues the call(s); stream-ordered with respect to the current
        stream on both sides, nothing waits for the GPU."""
        if len(self.jobs) == 1:
            _enqueue(self.jobs[0])
            return self
        main = torch.cuda.current_stream(self.trace.device)
        sides = _side_streams(main)
        for job, side in zip(self.jobs, sides):
            side.wait_stream(main)
            with torch.cuda.stream(side):
                _enqueue(job)
        for side in sides:
            main.wait_stream(side)
        for job in self.jobs:           # results are read in order behind the join
            job.stream = main
        return self

    def device_outputs(self):
        """[(candidate indices or None, good_total i64[.], latency_sum f64[.])] per call, on the
        device."""
        return [(idx, job.out[4][:job.Bs], job.out[5][:job.Bs])
                for idx, job in zip(self.index, self.jobs)]

    def results(self):
        """Waits and downloads: (BatchResult in the order of the batch, d2h bytes)."""
        done = [_download(job) for job in self.jobs]
        d2h = sum(d[1] for d in done)
        if len(done) == 1:
            return done[0][0], d2h
        res = BatchResult()
        B = self.enc.B
        for name in BatchResult.__slots__:
            first = getattr(done[0][0], name)
            if first is None:
                setattr(res, name, None)
                continue
            whole = np.zeros((B,) + first.shape[1:], first.dtype)
            for idx, (part, _) in zip(self.index, done):
                whole[idx] = getattr(part, name)
            setattr(res, name, whole)
        return res, d2h

    def release(self):
        for job in self.jobs:
            _release(job)


def submit_batch(trace: DeviceTrace, enc: EncodedBatch, table: LatencyTable, group_good=False,
                 pinned=False, options=None, mirrors=True, split=True,
                 crowded=False) -> ResidentBatch:
    """run_batch without waiting: returns a handle for collect_batch."""
    return ResidentBatch(trace, enc, table, group_good, pinned, options, mirrors, split,
                         crowded, launch_now=True)


collect_batch = _collect


def run_batch(trace: DeviceTrace, enc: EncodedBatch, table: LatencyTable,
              per_request=False, group_good=False, pinned=False, options=None, mirrors=True,
              split=True, crowded=False, rows_on_device=False):
    """Simulates every placement of `enc` against `trace`
    (simulate_requests_mixed, controller.py:561-628).  `mirrors`: placements
    with interchangeable groups get a mirror candidate (a speed-up of the
    time-parallel execution; results are the same with and without).
    `crowded`: the MMS_FLAG_CROWDED hint (results are the same).
    `rows_on_device` (with per_request): finish and good stay on the GPU, as
    BatchResult.finish_device / .good_device."""
    if not per_request:
        return _collect(submit_batch(trace, enc, table, group_good, pinned, options, mirrors,
                                     split, crowded))
    return _launch(trace, enc.B, enc.M, enc.G, enc.P, enc.T, enc.S, enc.C,
                   enc.model_off, enc.model_rep, enc.group_info,
                   table.device(trace.device), 0,
                   nat.FLAG_PER_REQUEST | (nat.FLAG_CROWDED if crowded else 0), group_good,
                   pinned, options, rows_on_device=rows_on_device)


def encode_dense(m_id2g_id, num_stages, num_models):
    """One candidate given as the reference's dense tables (m_id2g_id [M][*]
    with -1 ending a row, num_stages [G]) -> (model_off, model_rep,
    group_info, T) with latency column = group id."""
    m2g = np.asarray(m_id2g_id, dtype=np.int64).reshape(num_models, -1)
    ns = np.asarray(num_stages, dtype=np.int64)
    G = len(ns)
    if G > nat.MAX_COLUMNS or (G and ns.max() > nat.MAX_STAGES) or ns.sum() > nat.MAX_SLOTS:
        raise NotImplementedError("placement too large for the kernels")
    slot_first = np.cumsum(ns) - ns
    rows, offs = [], [0]
    contested = np.zeros(G, np.int64)
    for m in range(num_models):
        row = m2g[m]
        stop = np.flatnonzero(row < 0)
        row = row[:stop[0]] if len(stop) else row
        if len(row) and (row.max() >= G):
            raise IndexError("group id in m_id2g_id is out of range")
        if len(row) > 1:
            contested[row] = 1
        rows.append(row | (slot_first[row] << 8) | (ns[row] << 16) | (row << 24))
        offs.append(offs[-1] + len(row))
    if offs[-1] > nat.MAX_PLACED:
        raise NotImplementedError("too many (group, model) pairs")
    rep = np.concatenate(rows).astype(np.uint32) if rows and offs[-1] else np.zeros(0, np.uint32)
    rep = rep.reshape(1, -1) if len(rep) else np.zeros((1, 1), np.uint32)
    off = np.asarray(offs, dtype=np.uint16).reshape(1, -1)
    info = (slot_first | (ns << 8) | (contested << 16)).astype(np.uint32).reshape(1, -1)
    if info.shape[1] == 0:
        info = np.zeros((1, 1), np.uint32)
    return off, rep, info, max(int(ns.sum()), 1)


def group_lists(model_off, model_rep, group_info, G):
    """g_id2m_id of controller.py:424-430 as CSR per candidate, from the
    compact tables: (group_off u16[B][G+1], group_mod u16[B][P], group_cfg
    u32[B][G] = first slot | stages << 8 | column << 16)."""
    B, P = model_rep.shape
    M = model_off.shape[1] - 1
    group_off = np.zeros((B, G + 1), np.int64)
    group_mod = np.zeros((B, P), np.uint16)
    group_cfg = np.zeros((B, G), np.uint32)
    for b in range(B):
        n = int(model_off[b, M])
        ents = model_rep[b, :n].astype(np.int64)
        g = ents & 0xFF
        m = np.repeat(np.arange(M), np.diff(model_off[b].astype(np.int64)))
        order = np.lexsort((m, g))                  # by group, models ascending
        group_mod[b, :n] = m[order]
        group_off[b, 1:] = np.cumsum(np.bincount(g, minlength=G))
        info = group_info[b].astype(np.int64)
        cfg = info & 0xFFFF                         # first slot | stages << 8
        col = np.zeros(G, np.int64)
        col[g] = ents >> 24
        group_cfg[b] = (cfg | (col << 16)).astype(np.uint32)
    return group_off.astype(np.uint16), group_mod, group_cfg


class ResidentBatching:
    """A placement batch for the batching simulator with its tables, scratch
    and outputs on the GPU, ready to be launched (any number of times) on the
    current stream."""

    def __init__(self, trace: DeviceTrace, B, M, G, P, T, S, C, model_off, model_rep, group_info,
                 latency, latency_stride, batch_sizes, heap_capacity=0):
        _require_cuda()
        L = nat.lib()
        dev = trace.device
        N = trace.num_requests
        self.trace, self.B, self.M, self.G, self.N = trace, B, M, G, N
        goff, gmod, gcfg = group_lists(model_off, model_rep, group_info, G)
        self.h2d_bytes = sum(x.nbytes for x in (model_off, model_rep, goff, gmod, gcfg))
        with torch.cuda.device(dev):
            d_off, d_rep = _to_device(model_off, dev), _to_device(model_rep, dev)
            d_goff, d_gmod, d_gcfg = (_to_device(x, dev) for x in (goff, gmod, gcfg))
            d_lat = latency if isinstance(latency, torch.Tensor) else _to_device(latency, dev)
            self.cands = nat.Placements(B, M, G, P, T, S, C, 0, _ptr(d_off), _ptr(d_rep), None,
                                        _ptr(d_lat), int(latency_stride))
            self.bat = nat.Batching(_ptr(d_goff), _ptr(d_gmod), _ptr(d_gcfg), len(batch_sizes),
                                    int(heap_capacity), (ctypes.c_int32 * 8)(*list(batch_sizes)))
            need = L.mms_sim_batching_workspace_bytes(N, ctypes.byref(self.cands),
                                                      ctypes.byref(self.bat))
            ws_t = torch.empty(max(need, 256), dtype=torch.uint8, device=dev)
            self.ws = nat.Workspace(_ptr(ws_t), need)
            i32 = dict(dtype=torch.int32, device=dev)
            o_mreq, o_mgood = torch.zeros((B, max(M, 1)), **i32), torch.zeros((B, max(M, 1)), **i32)
            o_greq, o_ggood = torch.zeros((B, G), **i32), torch.zeros((B, G), **i32)
            o_total = torch.zeros(B, dtype=torch.int64, device=dev)
            o_lsum = torch.zeros(B, dtype=torch.float64, device=dev)
            o_status = torch.zeros(B, **i32)
            o_fin = torch.empty((B, max(N, 1)), dtype=torch.float64, device=dev)
            o_good = torch.empty((B, max(N, 1)), dtype=torch.uint8, device=dev)
            o_redo = torch.zeros(B, **i32)
            self.res = nat.Results(_ptr(o_mreq), _ptr(o_mgood), _ptr(o_greq), _ptr(o_ggood),
                                   _ptr(o_total), _ptr(o_lsum), _ptr(o_status), _ptr(o_fin),
                                   _ptr(o_good), _ptr(o_redo))
            self.next_same = trace.next_same_model()
        self.keep = (d_off, d_rep, d_goff, d_gmod, d_gcfg, d_lat, ws_t)
        self.out = (o_mreq, o_mgood, o_greq, o_ggood, o_total, o_lsum, o_status, o_fin, o_good,
                    o_redo)

    def launch(self):
        trace = self.trace
        with torch.cuda.device(trace.device):
            tr, plan = trace.c_trace(), trace.c_plan()
            rc = nat.lib().mms_sim_batching(ctypes.byref(tr), ctypes.byref(self.cands),
                                            ctypes.byref(self.bat), _ptr(self.next_same),
                                            ctypes.byref(plan), ctypes.byref(self.ws),
                                            ctypes.byref(self.res), _stream_ptr())
            nat.check(rc, "mms_sim_batching")
        return self

    def results(self, per_request=True, rows_on_device=False):
        """Waits and downloads: (BatchResult, d2h bytes).  rows_on_device: the
        result carries the per-request outputs as device tensors."""
        (o_mreq, o_mgood, o_greq, o_ggood, o_total, o_lsum, o_status, o_fin, o_good,
         o_redo) = self.out
        M, N = self.M, self.N
        res = BatchResult()
        res.model_num_requests = o_mreq.cpu().numpy()[:, :M]
        res.model_num_good = o_mgood.cpu().numpy()[:, :M]
        res.group_num_requests = o_greq.cpu().numpy()
        res.group_num_good = o_ggood.cpu().numpy()
        res.good_total = o_total.cpu().numpy()
        res.latency_sum = o_lsum.cpu().numpy()
        res.status = o_status.cpu().numpy().astype(np.uint32)
        res.resimulated = o_redo.cpu().numpy()
        res.finish = o_fin.cpu().numpy()[:, :N] if per_request else None
        res.good = o_good.cpu().numpy()[:, :N].astype(bool) if per_request else None
        if rows_on_device:
            res.finish_device, res.good_device = o_fin[:, :N], o_good[:, :N]
        d2h = sum(x.nbytes for x in (res.model_num_requests, res.model_num_good,
                                     res.group_num_requests, res.group_num_good, res.good_total,
                                     res.latency_sum, res.status))
        if per_request:
            d2h += res.finish.nbytes + res.good.nbytes
        return res, d2h


def launch_batching(trace: DeviceTrace, B, M, G, P, T, S, C, model_off, model_rep, group_info,
                    latency, latency_stride, batch_sizes, heap_capacity=0, per_request=True,
                    rows_on_device=False):
    """simulate_requests_mixed_batching (controller.py:630-798) for every
    candidate.  The kernel always writes per-request outputs (the latency sums
    are formed from them); per_request=False does not download them."""
    job = ResidentBatching(trace, B, M, G, P, T, S, C, model_off, model_rep, group_info, latency,
                           latency_stride, batch_sizes, heap_capacity).launch()
    res, _ = job.results(per_request, rows_on_device)
    if heap_capacity == 0 and np.any(res.status & nat.STATUS_HEAP_OVERFLOW):
        # the default capacity (G + 16 pending events) is what the simulation was seen to
        # need; nothing bounds it, so a run that overflowed is repeated with room to spare
        job = ResidentBatching(trace, B, M, G, P, T, S, C, model_off, model_rep, group_info,
                               latency, latency_stride, batch_sizes, 8 * G + 64).launch()
        res, _ = job.results(per_request, rows_on_device)
    if np.any(res.status):
        bad = int(np.flatnonzero(res.status)[0])
        what = {nat.STATUS_HEAP_OVERFLOW: "event heap overflow (raise heap_capacity)",
                nat.STATUS_QUEUE_LEFT: "a request was left queued",
                nat.STATUS_BAD_INDEX: "bad table index"}
        raise RuntimeError(f"batching simulator reported status {int(res.status[bad])} for "
                           f"candidate {bad}: " + ", ".join(v for k, v in what.items()
                                                            if res.status[bad] & k))
    return res


def resident_batching(trace: DeviceTrace, enc: EncodedBatch, table: LatencyTable,
                      heap_capacity=0) -> ResidentBatching:
    """ResidentBatching for an encoded batch and a table built with batch sizes."""
    if table.batch_sizes is None:
        raise ValueError("the latency table has no batch-size axis")
    return ResidentBatching(trace, enc.B, enc.M, enc.G, enc.P, enc.T, enc.S, enc.C,
                            enc.model_off, enc.model_rep, enc.group_info,
                            table.device(trace.device), 0, table.batch_sizes, heap_capacity)


def run_batch_batching(trace: DeviceTrace, enc: EncodedBatch, table: LatencyTable,
                       heap_capacity=0, per_request=True, rows_on_device=False):
    """Batching simulation of every placement of `enc`; `table` must have been
    built with batch sizes.  per_request=False leaves the per-request outputs
    (9 bytes per candidate and request) on the device."""
    if table.batch_sizes is None:
        raise ValueError("the latency table has no batch-size axis")
    return launch_batching(trace, enc.B, enc.M, enc.G, enc.P, enc.T, enc.S, enc.C, enc.model_off,
                           enc.model_rep, enc.group_info, table.device(trace.device), 0,
                           table.batch_sizes, heap_capacity, per_request, rows_on_device)


STATS_FIELDS = ("num_good", "first_start", "last_start", "latency_mean", "latency_std",
                "latency_p90", "latency_p99")


def device_compute_stats(arrivals, model_ids, num_models: int, finish, good, first: int,
                         window: int):
    """Workload.compute_stats (alpa_serve/simulator/workload.py:308-354) on the
    GPU, through mms_compute_stats: statistics of the requests [first, first +
    window) of per-request outputs that are already on the device.  arrivals
    f64[N], model_ids i32[N] (index into the WORKLOAD's names), finish f64[B][N],
    good u8[B][N]: torch tensors on one GPU.  Returns a dict of numpy arrays:
    num_requests i32[M]; num_good, first_start, last_start, latency_mean,
    latency_std, latency_p90, latency_p99 [B][M]; good_total i64[B],
    latency_sum f64[B]; and "d2h_bytes"."""
    _require_cuda()
    L = nat.lib()
    dev = finish.device
    if finish.dim() != 2 or good.shape != finish.shape or finish.stride(1) != 1 \
            or good.stride(1) != 1 or finish.stride(0) != good.stride(0):
        raise ValueError("finish and good must be [B][N] rows of one pitch")
    if finish.dtype != torch.float64 or good.dtype != torch.uint8:
        raise ValueError("finish must be float64 and good uint8")
    B, N = finish.shape
    M = int(num_models)
    first, window = int(first), int(window)
    if first < 0 or window < 0 or first + window > N or arrivals.numel() < N \
            or model_ids.numel() < N:
        raise ValueError("window outside the trace")
    with torch.cuda.device(dev):
        need = L.mms_compute_stats_workspace_bytes(window, M, B)
        if need == 0:
            raise NotImplementedError("statistics outside the kernel limits")
        ws_t = _take_scratch(dev, max(need, 256))
        ws = nat.Workspace(_ptr(ws_t), need)
        f64 = dict(dtype=torch.float64, device=dev)
        o = {"num_requests": torch.zeros(max(M, 1), dtype=torch.int32, device=dev),
             "num_good": torch.zeros((B, max(M, 1)), dtype=torch.int32, device=dev),
             "good_total": torch.zeros(B, dtype=torch.int64, device=dev),
             "latency_sum": torch.zeros(B, **f64)}
        for name in STATS_FIELDS[1:]:
            o[name] = torch.zeros((B, max(M, 1)), **f64)
        out = nat.StatsOut(*[_ptr(o[k]) for k in ("num_requests",) + STATS_FIELDS
                             + ("good_total", "latency_sum")])
        rc = L.mms_compute_stats(_ptr(arrivals), _ptr(model_ids), M, _ptr(finish), _ptr(good),
                                 finish.stride(0), B, first, window, ctypes.byref(ws),
                                 ctypes.byref(out), _stream_ptr())
        nat.check(rc, "mms_compute_stats")
        res = {k: v.cpu().numpy() for k, v in o.items()}      # waits for the kernels
        _return_scratch(dev, ws_t)
    res["d2h_bytes"] = sum(v.nbytes for v in res.values())
    res["num_requests"] = res["num_requests"][:M]
    for name in STATS_FIELDS:
        res[name] = res[name][:, :M]
    return res
