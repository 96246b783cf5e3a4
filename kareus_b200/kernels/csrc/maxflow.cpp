// Max-flow / min-cut with lower and upper edge bounds on a small DAG (Dinic's algorithm).
// The planner's hot loop: one bounded min-cut per millisecond of iteration time removed, thousands
// of times per plan (the reference delegates this to the `lowtime` package, which ships a native
// Edmonds-Karp for the same reason).
#include <algorithm>
#include <cmath>
#include <limits>
#include <queue>
#include <vector>

namespace {

struct Edge {
  int to;
  double cap;
  int rev;
};

struct Dinic {
  std::vector<std::vector<Edge>> g;
  std::vector<int> level, it;
  explicit Dinic(int n) : g(n), level(n), it(n) {}
  int add(int u, int v, double c) {
    g[u].push_back({v, c, (int)g[v].size()});
    g[v].push_back({u, 0.0, (int)g[u].size() - 1});
    return (int)g[u].size() - 1;
  }
  bool bfs(int s, int t) {
    std::fill(level.begin(), level.end(), -1);
    std::queue<int> q;
    level[s] = 0;
    q.push(s);
    while (!q.empty()) {
      int u = q.front();
      q.pop();
      for (const Edge& e : g[u])
        if (e.cap > 1e-12 && level[e.to] < 0) {
          level[e.to] = level[u] + 1;
          q.push(e.to);
        }
    }
    return level[t] >= 0;
  }
  double dfs(int u, int t, double f) {
    if (u == t) return f;
    for (int& i = it[u]; i < (int)g[u].size(); ++i) {
      Edge& e = g[u][i];
      if (e.cap > 1e-12 && level[e.to] == level[u] + 1) {
        double d = dfs(e.to, t, std::min(f, e.cap));
        if (d > 1e-12) {
          e.cap -= d;
          g[e.to][e.rev].cap += d;
          return d;
        }
      }
    }
    return 0.0;
  }
  double run(int s, int t) {
    double flow = 0.0;
    while (bfs(s, t)) {
      std::fill(it.begin(), it.end(), 0);
      while (true) {
        double f = dfs(s, t, std::numeric_limits<double>::infinity());
        if (f <= 1e-12) break;
        flow += f;
      }
    }
    return flow;
  }
};

}  // namespace

// Nodes 0..n-1; edge i goes eu[i] -> ev[i] with bounds [lb[i], ub[i]] (ub >= inf_value means
// unbounded).  Writes side[v] = 1 for nodes on the source side of a minimum cut.
// Returns 0 on success, 1 if the lower bounds admit no feasible flow.
extern "C" int kb_bounded_min_cut(int n, int m, const int* eu, const int* ev, const double* lb, const double* ub,
                                  int s, int t, double inf_value, int* side) {
  const int SS = n, TT = n + 1;
  Dinic d(n + 2);
  std::vector<double> excess(n, 0.0);
  double need = 0.0;
  for (int i = 0; i < m; ++i) {
    const double cap = (ub[i] >= inf_value ? inf_value : ub[i]) - lb[i];
    d.add(eu[i], ev[i], cap < 0 ? 0.0 : cap);
    excess[ev[i]] += lb[i];
    excess[eu[i]] -= lb[i];
  }
  for (int v = 0; v < n; ++v) {
    if (excess[v] > 1e-12) {
      d.add(SS, v, excess[v]);
      need += excess[v];
    } else if (excess[v] < -1e-12) {
      d.add(v, TT, -excess[v]);
    }
  }
  const int back_idx = d.add(t, s, inf_value);
  const double got = d.run(SS, TT);
  if (got + 1e-7 * (1.0 + need) < need) return 1;
  // drop the t->s edge, then push as much extra s->t flow as the residual network allows
  d.g[t][back_idx].cap = 0.0;
  d.g[s][d.g[t][back_idx].rev].cap = 0.0;
  for (Edge& e : d.g[SS]) e.cap = 0.0;
  for (int v = 0; v < n; ++v)
    for (Edge& e : d.g[v])
      if (e.to == SS || e.to == TT) e.cap = 0.0;
  d.run(s, t);
  d.bfs(s, t);
  for (int v = 0; v < n; ++v) side[v] = d.level[v] >= 0 ? 1 : 0;
  return 0;
}
