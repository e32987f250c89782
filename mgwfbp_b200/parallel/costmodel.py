# -*- coding: utf-8 -*-
"""All-reduce cost models ``t(bytes)`` used by the merge scheduler.

The reference models one all-reduce as ``alpha + beta * bytes`` with constants that were
measured on its authors' clusters and hard-coded per worker count
(``distributed_optimizer.py:166-177``, ``utils.py:83-88``).  Those tables are kept here
verbatim as *data* so that the scheduler can be checked against the reference, but the
production path fits the constants from an event-timed sweep of this package's own
all-reduce kernels (one fit per algorithm: one-shot, two-shot, NVLS) and the scheduler
consumes the lower envelope of those fits (:class:`PiecewiseAlphaBeta`).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np

# (alpha seconds, beta seconds/byte) per world size -- reference distributed_optimizer.py:166-171
TABLE_56GBIB: Dict[int, Tuple[float, float]] = {
    16: (0.00023583677659915685, 4.0594787739537565e-10),
    8: (9.75367204301171e-05, 3.0568230536676206e-10),
    4: (4.204298980348825e-05, 2.0589360830118177e-10),
    2: (2.554691138304671e-06, 9.837548167872609e-11),
}
# reference distributed_optimizer.py:172-177
TABLE_10GBE: Dict[int, Tuple[float, float]] = {
    16: (0.0009080981007148093, 7.395651186836712e-10),
    8: (0.0005230272768511732, 8.570746975492128e-10),
    4: (4.204298980348825e-05, 2.0589360830118177e-10),
    2: (2.554691138304671e-06, 9.837548167872609e-11),
}
# The fused peer-to-peer kernels of this package on one NVSwitch box of B200s, used until a fit measured on the
# running box is supplied (``engine.fit_comm_model``, ``DistributedOptimizer.benchmark_communication`` or
# ``MGWFBP_ALPHA_BETA``).  Least-squares fits of the two-shot kernel (write-back mode, 128 CTAs at most) over 1 KB ..
# 128 MB, device-timed from CUDA-graph replays (``python -m mgwfbp_b200.parallel.comm.bench``) at 2, 4 and 8 GPUs; the
# 16-rank row is extrapolated.  The one-shot kernel that serves messages up to 512 KB starts in 9-12 us.
TABLE_NVLINK5: Dict[int, Tuple[float, float]] = {
    2: (1.87e-05, 2.07e-12),
    4: (1.99e-05, 3.12e-12),
    8: (2.03e-05, 3.65e-12),
    16: (2.2e-05, 3.9e-12),
}

_TABLES = {'10GbE': TABLE_10GBE, '56GbIB': TABLE_56GBIB, 'NVLink5': TABLE_NVLINK5}


@dataclass(frozen=True)
class AlphaBeta:
    """``t = alpha + beta * nbytes`` (0 for an empty message, as reference utils.py:151-154)."""
    alpha: float
    beta: float
    name: str = 'allreduce'

    def __call__(self, nbytes: float) -> float:
        if nbytes == 0:
            return 0.0
        return self.alpha + self.beta * nbytes

    def startup(self, nbytes: float = 0) -> float:
        """Latency that a merge saves: one start-up per message avoided."""
        return self.alpha


@dataclass(frozen=True)
class PiecewiseAlphaBeta:
    """Lower envelope of several per-algorithm fits, each valid on ``[lo, hi)`` bytes.

    The fused all-reduce picks its algorithm by message size; each algorithm has its own
    (alpha, beta).  ``__call__`` returns the cheapest admissible algorithm's time and
    ``startup`` the alpha of that algorithm, which is what merging two messages saves.
    """
    pieces: Tuple[Tuple[float, float, AlphaBeta], ...]

    def _best(self, nbytes: float) -> AlphaBeta:
        best, best_t = None, float('inf')
        for lo, hi, ab in self.pieces:
            if lo <= nbytes < hi:
                t = ab(nbytes)
                if t < best_t:
                    best, best_t = ab, t
        if best is None:  # outside every declared range: use the last piece
            best = self.pieces[-1][2]
        return best

    def __call__(self, nbytes: float) -> float:
        if nbytes == 0:
            return 0.0
        return self._best(nbytes)(nbytes)

    def startup(self, nbytes: float = 0) -> float:
        return self._best(max(nbytes, 1)).alpha

    def choose(self, nbytes: float) -> str:
        return self._best(nbytes).name


def table_lookup(connection: str, world_size: int) -> AlphaBeta:
    """Constants for ``world_size`` workers on ``connection``.

    The reference raises ``KeyError`` for any world size outside {2, 4, 8, 16}
    (``distributed_optimizer.py:180-184``).  Here intermediate sizes are interpolated in
    log2(P) and sizes beyond the table are extrapolated from its last two entries.
    """
    table = _TABLES.get(connection, TABLE_56GBIB)
    if world_size in table:
        a, b = table[world_size]
        return AlphaBeta(a, b, connection)
    if world_size <= 1:
        return AlphaBeta(0.0, 0.0, connection)
    ps = sorted(table)
    xs = np.log2(ps)
    x = np.log2(world_size)
    alphas = [table[p][0] for p in ps]
    betas = [table[p][1] for p in ps]
    if world_size > ps[-1] or world_size < ps[0]:
        i = len(ps) - 2 if world_size > ps[-1] else 0
        sa = (alphas[i + 1] - alphas[i]) / (xs[i + 1] - xs[i])
        sb = (betas[i + 1] - betas[i]) / (xs[i + 1] - xs[i])
        a = alphas[i] + sa * (x - xs[i])
        b = betas[i] + sb * (x - xs[i])
    else:
        a = float(np.interp(x, xs, alphas))
        b = float(np.interp(x, xs, betas))
    return AlphaBeta(max(float(a), 0.0), max(float(b), 0.0), connection)


def fit_alpha_beta(sizes_elems: Sequence[float], times_s: Sequence[float], bytes_per_elem: int = 4,
                   name: str = 'allreduce') -> AlphaBeta:
    """Ordinary least squares of time on bytes.

    Same estimator as the reference's ``_fit_linear_function`` (sklearn ``LinearRegression`` on
    ``sizes * 4`` bytes, ``distributed_optimizer.py:109-116``), in closed form.
    """
    x = np.asarray(sizes_elems, dtype=np.float64) * bytes_per_elem
    y = np.asarray(times_s, dtype=np.float64)
    if x.size < 2:
        raise ValueError('need at least two (size, time) samples to fit alpha and beta')
    xm, ym = x.mean(), y.mean()
    sxx = float(((x - xm) ** 2).sum())
    if sxx == 0.0:
        raise ValueError('all sample sizes are equal; cannot fit beta')
    beta = float(((x - xm) * (y - ym)).sum() / sxx)
    alpha = float(ym - beta * xm)
    return AlphaBeta(alpha, beta, name)


def fit_piecewise(samples: Dict[str, Tuple[Sequence[float], Sequence[float]]],
                  ranges: Optional[Dict[str, Tuple[float, float]]] = None,
                  bytes_per_elem: int = 4) -> PiecewiseAlphaBeta:
    """One fit per algorithm name; ``ranges`` bounds (in bytes) where each may be chosen."""
    pieces: List[Tuple[float, float, AlphaBeta]] = []
    for algo, (sizes, times) in samples.items():
        ab = fit_alpha_beta(sizes, times, bytes_per_elem, name=algo)
        # A noisy sweep can produce a slightly negative intercept; a start-up cost is never negative.
        ab = AlphaBeta(max(ab.alpha, 0.0), max(ab.beta, 0.0), algo)
        lo, hi = (ranges or {}).get(algo, (0.0, float('inf')))
        pieces.append((float(lo), float(hi), ab))
    return PiecewiseAlphaBeta(tuple(pieces))


def predict_allreduce_time_with_size(alpha: float, beta: float, size: float, P: int = 0) -> float:
    """Reference-compatible helper (``utils.py:151-154``): ``size`` is in bytes."""
    if size == 0:
        return 0.0
    return alpha + beta * size
