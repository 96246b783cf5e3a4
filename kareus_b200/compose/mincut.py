"""Minimum cut with lower/upper edge bounds: native (C++) when the library is built, Python otherwise."""
from __future__ import annotations

import ctypes
from collections import deque
from typing import List, Optional, Sequence, Tuple

INF = 1e18
_NATIVE = None


def _native():
    global _NATIVE
    if _NATIVE is None:
        _NATIVE = False
        try:
            import torch  # noqa: F401  (loads the CUDA runtime the library links against)
            from ..kernels import cuda as KC
            L = ctypes.CDLL(str(KC.LIB_PATH))
            fn = L.kb_bounded_min_cut
            fn.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int),
                           ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_double), ctypes.c_int,
                           ctypes.c_int, ctypes.c_double, ctypes.POINTER(ctypes.c_int)]
            fn.restype = ctypes.c_int
            _NATIVE = fn
        except Exception:
            _NATIVE = False
    return _NATIVE


class _Dinic:
    def __init__(self, n):
        self.g = [[] for _ in range(n)]

    def add(self, u, v, c):
        self.g[u].append([v, c, len(self.g[v])])
        self.g[v].append([u, 0.0, len(self.g[u]) - 1])
        return len(self.g[u]) - 1

    def bfs(self, s, t):
        self.level = [-1] * len(self.g)
        self.level[s] = 0
        q = deque([s])
        while q:
            u = q.popleft()
            for v, c, _ in self.g[u]:
                if c > 1e-12 and self.level[v] < 0:
                    self.level[v] = self.level[u] + 1
                    q.append(v)
        return self.level[t] >= 0

    def dfs(self, u, t, f):
        if u == t:
            return f
        g = self.g[u]
        while self.it[u] < len(g):
            e = g[self.it[u]]
            if e[1] > 1e-12 and self.level[e[0]] == self.level[u] + 1:
                d = self.dfs(e[0], t, min(f, e[1]))
                if d > 1e-12:
                    e[1] -= d
                    self.g[e[0]][e[2]][1] += d
                    return d
            self.it[u] += 1
        return 0.0

    def run(self, s, t):
        flow = 0.0
        while self.bfs(s, t):
            self.it = [0] * len(self.g)
            while True:
                f = self.dfs(s, t, float("inf"))
                if f <= 1e-12:
                    break
                flow += f
        return flow


def _python_min_cut(n, edges, s, t):
    SS, TT = n, n + 1
    d = _Dinic(n + 2)
    excess = [0.0] * n
    for u, v, lb, ub in edges:
        cap = (INF if ub >= INF else ub) - lb
        d.add(u, v, max(cap, 0.0))
        excess[v] += lb
        excess[u] -= lb
    need = 0.0
    for v in range(n):
        if excess[v] > 1e-12:
            d.add(SS, v, excess[v])
            need += excess[v]
        elif excess[v] < -1e-12:
            d.add(v, TT, -excess[v])
    back = d.add(t, s, INF)
    got = d.run(SS, TT)
    if got + 1e-7 * (1.0 + need) < need:
        return None
    e = d.g[t][back]
    d.g[s][e[2]][1] = 0.0
    e[1] = 0.0
    for e in d.g[SS]:
        e[1] = 0.0
    for v in range(n):
        for e in d.g[v]:
            if e[0] in (SS, TT):
                e[1] = 0.0
    d.run(s, t)
    d.bfs(s, t)
    return [1 if d.level[v] >= 0 else 0 for v in range(n)]


def bounded_min_cut(n: int, edges: Sequence[Tuple[int, int, float, float]], s: int, t: int,
                    use_native: Optional[bool] = None) -> Optional[List[int]]:
    """``edges`` are ``(u, v, lower, upper)``.  Returns the source-side indicator of a minimum
    cut, or ``None`` when the lower bounds cannot be satisfied."""
    fn = _native() if use_native is not False else False
    if fn and use_native is not False:
        m = len(edges)
        eu = (ctypes.c_int * m)(*[e[0] for e in edges])
        ev = (ctypes.c_int * m)(*[e[1] for e in edges])
        lb = (ctypes.c_double * m)(*[float(e[2]) for e in edges])
        ub = (ctypes.c_double * m)(*[float(min(e[3], INF)) for e in edges])
        side = (ctypes.c_int * n)()
        rc = fn(n, m, eu, ev, lb, ub, s, t, INF, side)
        return None if rc != 0 else list(side)
    if use_native is True:
        raise RuntimeError("native min-cut requested but the library is not built")
    return _python_min_cut(n, list(edges), s, t)
