"""Request traces: arrival processes, the Workload container and stats types.

Host-side mirror of alpa_serve/simulator/workload.py.  A Workload here keeps
the trace as arrays (arrival time, model index, SLO per request) from the
start instead of one Python object per request; `requests` builds the
reference's list of Request objects only when someone asks for it.  The
arrival times are produced with the same numpy calls in the same order as
the reference, so a trace generated here equals the reference's bit for bit
under the same numpy.
"""
from collections import namedtuple
import dataclasses
from typing import Any, Dict, List, Optional, Sequence

import numpy as np

DEFAULT_WARMUP = 10      # workload.py:14
eps = 1e-6               # alpa_serve/util.py:22


@dataclasses.dataclass
class Request:
    """workload.py:17-25."""
    model_name: str
    data: Any
    slo: Optional[float]
    idx: int
    time_stamp: Dict
    submit_time: float = None


# workload.py:28-43
PerModelStatsResult = namedtuple(
    "PerModelStatsResult",
    ("name", "num_requests", "goodput", "throughput", "latency_mean", "latency_std",
     "latency_p90", "latency_p99", "latency", "request_starts", "request_finishes"))


@dataclasses.dataclass
class StatsResult:
    per_model_stats: List[PerModelStatsResult]
    group_num_requests: Sequence[int]
    goodput: float
    latency_mean: float
    num_requests: int
    request_rate: float


class GammaProcess:
    """Gamma renewal arrivals (workload.py:114-162): gaps ~ Gamma(1/cv^2,
    cv^2/rate), drawn from numpy's global legacy generator after
    np.random.seed(seed), in batches of int(rate*duration*1.2)."""

    def __init__(self, arrival_rate: float, cv: float):
        self.rate_ = arrival_rate
        self.cv_ = cv
        self.shape = 1 / (cv * cv)
        self.scale = cv * cv / arrival_rate

    def rate(self):
        return self.rate_

    def cv(self):
        return self.cv_

    def generate_arrivals(self, start: float, duration: float, seed: int = 0) -> np.ndarray:
        """Same values as workload.py:135-155, which adds one gap at a time in
        a Python loop.  A running fp64 sum taken left to right is what
        np.cumsum computes, so each batch of gaps is accumulated with cumsum
        seeded by the last tick."""
        np.random.seed(seed)
        batch = max(int(self.rate_ * duration * 1.2), 1)
        end = start + duration
        pieces = []
        cur = float(start)
        while True:
            gaps = np.random.gamma(self.shape, self.scale, size=batch)
            ticks = np.cumsum(np.concatenate(([cur], gaps)))[1:]
            stop = int(np.searchsorted(ticks >= end, True))  # first tick at or past the end
            if stop < batch:
                pieces.append(ticks[:stop])
                break
            pieces.append(ticks)
            cur = float(ticks[-1])
        return np.concatenate(pieces) if pieces else np.empty(0)

    def generate_workload(self, model_name: str, start: float, duration: float,
                          slo: Optional[float] = None, seed: int = 0) -> "Workload":
        ticks = self.generate_arrivals(start, duration, seed)
        return Workload.from_arrays(ticks, np.zeros(len(ticks), np.int32),
                                    np.full(len(ticks), np.nan if slo is None else slo),
                                    [model_name])


class PoissonProcess(GammaProcess):
    """workload.py:165-176."""

    def __init__(self, arrival_rate: float):
        super().__init__(arrival_rate, 1)


class Workload:
    """A time-sorted request trace (workload.py:266-421)."""

    def __init__(self, arrivals, requests: List[Request]):
        assert len(arrivals) == len(requests)
        names, index = [], {}
        which = np.empty(len(requests), np.int32)
        slo = np.empty(len(requests), np.float64)
        for i, r in enumerate(requests):
            k = index.get(r.model_name)
            if k is None:
                k = index[r.model_name] = len(names)
                names.append(r.model_name)
            which[i] = k
            slo[i] = np.nan if r.slo is None else r.slo
        self._init(np.array(arrivals, dtype=np.float64), which, slo, names)
        self._requests = requests

    @classmethod
    def from_arrays(cls, arrivals, name_index, slo, names) -> "Workload":
        w = cls.__new__(cls)
        w._init(np.asarray(arrivals, dtype=np.float64), np.asarray(name_index, dtype=np.int32),
                np.asarray(slo, dtype=np.float64), list(names))
        w._requests = None
        return w

    def _init(self, arrivals, name_index, slo, names):
        self.arrivals = arrivals
        self.name_index = name_index      # position of the request's model in `names`
        self.request_slo = slo            # NaN where the request carries no SLO
        self.names = names
        self.enable_simulator_cache = False
        self.cached_data = None
        if len(arrivals) > 1:             # workload.py:278-284
            gaps = arrivals[1:] - arrivals[:-1]
            self.rate = 1 / (np.mean(gaps) + eps)
            self.cv = np.std(gaps) * self.rate
        else:
            self.rate = 0
            self.cv = 0

    @property
    def requests(self) -> List[Request]:
        if self._requests is None:
            self._requests = [
                Request(self.names[k], None, None if np.isnan(s) else float(s), i, {})
                for i, (k, s) in enumerate(zip(self.name_index.tolist(),
                                               self.request_slo.tolist()))]
        return self._requests

    @classmethod
    def empty(cls):
        return cls.from_arrays(np.empty(0), np.empty(0, np.int32), np.empty(0), [])

    @classmethod
    def merge(cls, *args: "Workload") -> "Workload":
        """workload.py:382-401: concatenate, then order by np.argsort of the
        arrival times (numpy's default sort, as the reference calls it)."""
        if len(args) == 1:
            return args[0]
        names, index = [], {}
        parts = []
        for w in args:
            remap = np.empty(max(len(w.names), 1), np.int32)
            for k, n in enumerate(w.names):
                if n not in index:
                    index[n] = len(names)
                    names.append(n)
                remap[k] = index[n]
            parts.append(remap[w.name_index] if len(w.name_index) else w.name_index)
        arrivals = np.concatenate([w.arrivals for w in args])
        which = np.concatenate(parts)
        slo = np.concatenate([w.request_slo for w in args])
        order = np.argsort(arrivals)
        return cls.from_arrays(arrivals[order], which[order], slo[order], names)

    def __getitem__(self, key):
        if not isinstance(key, slice):
            raise NotImplementedError()
        return Workload.from_arrays(self.arrivals[key], self.name_index[key],
                                    self.request_slo[key], self.names)

    def __add__(self, other):
        return Workload.merge(self, other)

    def __len__(self):
        return len(self.arrivals)

    def __str__(self):
        return f"Workload(len={len(self)}, rate={self.rate:.2f}, CV={self.cv:.2f})"

    def compute_stats(self, start, finish, good, warmup: float) -> StatsResult:
        """Per-model latency statistics with `warmup` seconds trimmed at both
        ends (workload.py:308-354)."""
        start = np.asarray(start); finish = np.asarray(finish); good = np.asarray(good)
        which = self.name_index
        if len(self.arrivals) > 1:
            skip = int(warmup / (self.arrivals[-1] - self.arrivals[0]) * len(self.arrivals))
            if skip > 0:
                start, finish, good = start[skip:-skip], finish[skip:-skip], good[skip:-skip]
                which = which[skip:-skip]
        # models in order of first appearance, then by request count (stable sort)
        _, first = np.unique(which, return_index=True)
        seen = which[np.sort(first)]
        counts = {int(k): int(np.sum(which == k)) for k in seen}
        ordered = sorted((int(k) for k in seen), key=lambda k: counts[k])
        stats = []
        for k in ordered:
            idx = np.nonzero(which == k)[0].astype(np.int32)
            g = np.asarray(good[idx], dtype=bool)
            s, f = start[idx][g], finish[idx][g]
            goodput = np.mean(g)
            if goodput > 0:
                throughput = len(s) / (s[-1] - s[0])
                latency = f - s
            else:
                throughput = 0
                latency = [0]
            srt = np.sort(latency)
            stats.append(PerModelStatsResult(
                self.names[k], len(idx), goodput, throughput, np.mean(latency), np.std(latency),
                srt[int(0.90 * len(srt))], srt[int(0.99 * len(srt))], latency, s, f))
        return StatsResult(stats, None, np.mean(good), np.mean(finish - start), len(start),
                           len(start) / (start[-1] - start[0]))
