"""Surrogate models and acquisition for the two-objective (time, energy) search.

The reference trains XGBoost regressors (depth 6, eta 0.3, 100 rounds) for effective energy and
time, a 5-member bootstrap ensemble for uncertainty, derives real energy as ``E_eff + P_p2p·t`` and
scores candidates by the hypervolume gain of their predicted point (BoTorch ``Hypervolume``)
(``tests/bayesian/common/surrogates.py:14-208``).  Neither package is available offline, so the
regressor is scikit-learn's gradient boosting with the same hyper-parameters (falling back to a
small own implementation of boosted regression stumps) and the 2-D hypervolume is a sorted sweep.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import numpy as np


class _Stumps:
    """Minimal gradient-boosted regression trees (depth-limited, squared loss)."""

    def __init__(self, n_estimators=100, learning_rate=0.3, max_depth=3, rng=None):
        self.n, self.lr, self.depth = n_estimators, learning_rate, max_depth
        self.trees, self.base = [], 0.0

    def _fit_tree(self, X, r, depth):
        if depth == 0 or len(r) < 2 or np.allclose(r, r[0]):
            return ("leaf", float(r.mean()))
        best = None
        for j in range(X.shape[1]):
            vals = np.unique(X[:, j])
            for thr in (vals[:-1] + vals[1:]) / 2:
                m = X[:, j] <= thr
                if m.all() or not m.any():
                    continue
                sse = ((r[m] - r[m].mean()) ** 2).sum() + ((r[~m] - r[~m].mean()) ** 2).sum()
                if best is None or sse < best[0]:
                    best = (sse, j, thr, m)
        if best is None:
            return ("leaf", float(r.mean()))
        _, j, thr, m = best
        return ("node", j, thr, self._fit_tree(X[m], r[m], depth - 1), self._fit_tree(X[~m], r[~m], depth - 1))

    def _pred_tree(self, t, X):
        if t[0] == "leaf":
            return np.full(len(X), t[1])
        _, j, thr, l, r = t
        out = np.empty(len(X))
        m = X[:, j] <= thr
        out[m] = self._pred_tree(l, X[m])
        out[~m] = self._pred_tree(r, X[~m])
        return out

    def fit(self, X, y):
        self.base = float(y.mean())
        pred = np.full(len(y), self.base)
        self.trees = []
        for _ in range(self.n):
            t = self._fit_tree(X, y - pred, self.depth)
            self.trees.append(t)
            pred = pred + self.lr * self._pred_tree(t, X)
        return self

    def predict(self, X):
        out = np.full(len(X), self.base)
        for t in self.trees:
            out = out + self.lr * self._pred_tree(t, X)
        return out


def make_regressor(seed: int = 0):
    try:
        from sklearn.ensemble import GradientBoostingRegressor
        return GradientBoostingRegressor(n_estimators=100, learning_rate=0.3, max_depth=6, random_state=seed)
    except Exception:  # pragma: no cover
        return _Stumps(n_estimators=60, learning_rate=0.3, max_depth=3)


class Surrogates:
    """Models of effective energy and time (+ bootstrap ensemble)."""

    def __init__(self, p2p_power: float, ensemble: int = 5, seed: int = 0):
        self.p2p, self.k, self.seed = p2p_power, ensemble, seed
        self.m_e = self.m_t = None
        self.ens: List[Tuple[object, object]] = []

    def fit(self, X: np.ndarray, eff_energy: np.ndarray, time_s: np.ndarray) -> "Surrogates":
        self.m_e = make_regressor(self.seed).fit(X, eff_energy)
        self.m_t = make_regressor(self.seed + 1).fit(X, time_s)
        rng = np.random.default_rng(self.seed)
        self.ens = []
        for i in range(self.k):
            idx = rng.integers(0, len(X), len(X))
            self.ens.append((make_regressor(self.seed + 10 + i).fit(X[idx], eff_energy[idx]),
                             make_regressor(self.seed + 20 + i).fit(X[idx], time_s[idx])))
        return self

    def predict(self, X: np.ndarray):
        """``(effective energy, real energy, time)`` predictions."""
        t = self.m_t.predict(X)
        e = self.m_e.predict(X)
        return e, e + self.p2p * t, t

    def uncertainty(self, X: np.ndarray) -> np.ndarray:
        if not self.ens:
            return np.zeros(len(X))
        pe = np.stack([m[0].predict(X) for m in self.ens])
        pt = np.stack([m[1].predict(X) for m in self.ens])
        se = pe.std(0) / (np.abs(pe.mean(0)) + 1e-12)
        st = pt.std(0) / (np.abs(pt.mean(0)) + 1e-12)
        return se + st


def pareto_mask(Y: np.ndarray) -> np.ndarray:
    """Non-dominated rows of ``Y`` (both objectives minimised)."""
    n = len(Y)
    keep = np.ones(n, dtype=bool)
    order = np.lexsort((Y[:, 1], Y[:, 0]))
    best = np.inf
    for i in order:
        if Y[i, 1] < best:
            best = Y[i, 1]
        else:
            keep[i] = False
    return keep


def hypervolume_2d(Y: np.ndarray, ref: Sequence[float]) -> float:
    """Area dominated by the Pareto front of ``Y`` and bounded by ``ref`` (minimisation)."""
    P = Y[(Y[:, 0] < ref[0]) & (Y[:, 1] < ref[1])]
    if len(P) == 0:
        return 0.0
    P = P[pareto_mask(P)]
    P = P[np.argsort(P[:, 0])]
    hv, prev_y = 0.0, ref[1]
    for x, y in P:
        hv += (ref[0] - x) * (prev_y - y)
        prev_y = y
    return float(hv)


def hv_improvement(front: np.ndarray, cand: np.ndarray, ref: Sequence[float]) -> np.ndarray:
    """Hypervolume gained by adding each candidate point to ``front`` (the reference's "EHVI" is the
    gain of the predicted point, ``surrogates.py:137-208``)."""
    base = hypervolume_2d(front, ref) if len(front) else 0.0
    out = np.zeros(len(cand))
    for i, c in enumerate(cand):
        out[i] = hypervolume_2d(np.vstack([front, c[None]]) if len(front) else c[None], ref) - base
    return out
