// Integer schedule selector.
//
// A candidate "split the layer into c chunks" is the graph EDMBuilder
// (EDM-IR/ir/builder.py:22-110) would hold for it:
//   id 0            phase.begin
//   ids 1..c        compute.gemm chunk i        (stream_order chain)
//   ids c+1..2c     comm.* chunk i              (stream_order chain)
//   id 2c+1         phase.end
//   data_dependency gemm_i -> comm_i (or comm_i -> gemm_i when the collective feeds the GEMM)
//   phase_boundary  begin -> body, body -> end  (bind_phase order: per body node, in id order)
// and its cost is what analyze_critical_path (EDM-IR/ir/analysis.py:36-65) returns for that
// graph: best[u] = dur(u) + max over predecessors, first maximum in edge-insertion order
// (analysis.py:51); end node = max by (best, end_us, id) (analysis.py:58); topological order is
// Kahn's with the zero-indegree ids seeded in sorted order and successors visited in
// edge-insertion order (EDM-IR/ir/graph.py:54-72).  Exposed communication is the summed duration
// of comm nodes on that path (analysis.py:93-95).  All arithmetic is int64, so the result is exact.
#include <algorithm>
#include <cstdint>
#include <deque>
#include <vector>

#include "../../include/edm_b200.h"

namespace {

struct Node {
  int64_t dur = 0, start = 0, end = 0;
  bool is_comm = false;
};

int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// share of `total` given to chunk i of c (remainder spread over the first chunks)
int64_t share(int64_t total, int32_t c, int32_t i) {
  return total / c + (i < total % c ? 1 : 0);
}

// Critical path of an arbitrary graph with the reference's tie rules (see the file comment).
// Nodes are ids 0..n-1; edges in insertion order.  Returns false on a cycle or a bad edge.
bool critical_path(const std::vector<Node>& node, const std::vector<std::pair<int, int>>& edges,
                   int64_t& makespan, int64_t& exposed, std::vector<int>* path) {
  const int n = static_cast<int>(node.size());
  if (n == 0) { makespan = exposed = 0; if (path) path->clear(); return true; }
  std::vector<std::vector<int>> succ(n), pred(n);
  std::vector<int> indeg(n, 0);
  for (auto& e : edges) {
    if (e.first < 0 || e.first >= n || e.second < 0 || e.second >= n) return false;
    succ[e.first].push_back(e.second);
    pred[e.second].push_back(e.first);
    ++indeg[e.second];
  }
  std::deque<int> ready;
  for (int u = 0; u < n; ++u)
    if (indeg[u] == 0) ready.push_back(u);
  std::vector<int> order;
  order.reserve(n);
  while (!ready.empty()) {
    const int u = ready.front();
    ready.pop_front();
    order.push_back(u);
    for (int v : succ[u])
      if (--indeg[v] == 0) ready.push_back(v);
  }
  if (static_cast<int>(order.size()) != n) return false;

  std::vector<int64_t> best(n, 0);
  std::vector<int> parent(n, -1);
  for (int u : order) {
    if (pred[u].empty()) { best[u] = node[u].dur; continue; }
    int arg = pred[u][0];
    for (int q : pred[u])
      if (best[q] > best[arg]) arg = q;  // strict: the first maximum wins
    best[u] = best[arg] + node[u].dur;
    parent[u] = arg;
  }
  int last = 0;
  for (int u = 1; u < n; ++u) {
    if (best[u] > best[last] ||
        (best[u] == best[last] && (node[u].end > node[last].end ||
                                   (node[u].end == node[last].end && u > last))))
      last = u;
  }
  exposed = 0;
  if (path) path->clear();
  for (int u = last; u >= 0; u = parent[u]) {
    if (node[u].is_comm) exposed += node[u].dur;
    if (path) path->push_back(u);
  }
  if (path) std::reverse(path->begin(), path->end());
  makespan = best[last];
  return true;
}

int evaluate(const edm_cost_params_t& p, int32_t c, edm_candidate_cost_t& out) {
  if (c < 1 || c > 4096) return EDM_ERR_BAD_ARG;
  if (p.gemm_total < 0 || p.comm_bytes < 0 || p.alpha < 0 || p.beta_num < 0 || p.beta_den <= 0 ||
      p.split_overhead < 0)
    return EDM_ERR_BAD_ARG;
  const int n = 2 * c + 2;
  std::vector<Node> node(n);
  const int begin = 0, end = 2 * c + 1;
  auto gemm = [&](int i) { return 1 + i; };
  auto comm = [&](int i) { return 1 + c + i; };

  int64_t total_comm = 0;
  for (int i = 0; i < c; ++i) {
    node[gemm(i)].dur = share(p.gemm_total, c, i) + (c > 1 ? p.split_overhead : 0);
    const int64_t bytes = share(p.comm_bytes, c, i);
    // a byte count up to 2^40 times a numerator up to 2^20 stays inside int64
    node[comm(i)].dur = p.alpha + ceil_div(bytes * p.beta_num, p.beta_den);
    node[comm(i)].is_comm = true;
    total_comm += node[comm(i)].dur;
  }
  // as-soon-as-possible timestamps (only end_us takes part in tie-breaking)
  {
    int64_t g_end = 0, m_end = 0;
    for (int i = 0; i < c; ++i) {
      if (!p.comm_first) {
        node[gemm(i)].start = g_end; g_end += node[gemm(i)].dur; node[gemm(i)].end = g_end;
        const int64_t s = g_end > m_end ? g_end : m_end;
        node[comm(i)].start = s; m_end = s + node[comm(i)].dur; node[comm(i)].end = m_end;
      } else {
        node[comm(i)].start = m_end; m_end += node[comm(i)].dur; node[comm(i)].end = m_end;
        const int64_t s = g_end > m_end ? g_end : m_end;
        node[gemm(i)].start = s; g_end = s + node[gemm(i)].dur; node[gemm(i)].end = g_end;
      }
    }
    const int64_t fin = g_end > m_end ? g_end : m_end;
    node[end].start = node[end].end = fin;
  }

  // edges in builder insertion order
  std::vector<std::pair<int, int>> edges;
  for (int i = 0; i + 1 < c; ++i) edges.push_back({gemm(i), gemm(i + 1)});
  for (int i = 0; i + 1 < c; ++i) edges.push_back({comm(i), comm(i + 1)});
  for (int i = 0; i < c; ++i) {
    if (!p.comm_first) edges.push_back({gemm(i), comm(i)});
    else edges.push_back({comm(i), gemm(i)});
  }
  for (int u = 1; u <= 2 * c; ++u) {
    edges.push_back({begin, u});
    edges.push_back({u, end});
  }

  int64_t makespan = 0, exposed = 0;
  if (!critical_path(node, edges, makespan, exposed, nullptr)) return EDM_ERR_BAD_ARG;

  out.makespan = makespan;
  out.exposed_comm = exposed;
  out.total_comm = total_comm;
  out.gemm_chunk = node[gemm(0)].dur;
  out.comm_chunk = node[comm(0)].dur;
  return EDM_OK;
}

}  // namespace

extern "C" {

int edm_schedule_cost(const edm_cost_params_t* p, int32_t chunks, edm_candidate_cost_t* out) {
  if (!p || !out) return EDM_ERR_BAD_ARG;
  return evaluate(*p, chunks, *out);
}

int edm_graph_cost(int32_t n_nodes, const int64_t* dur, const int64_t* end, const uint8_t* is_comm,
                   int32_t n_edges, const int32_t* src, const int32_t* dst, int64_t* makespan,
                   int64_t* exposed_comm, int32_t* path, int32_t* path_len) {
  if (n_nodes < 0 || n_edges < 0 || n_nodes > (1 << 20) || n_edges > (1 << 22) || !makespan || !exposed_comm)
    return EDM_ERR_BAD_ARG;
  if ((n_nodes > 0 && (!dur || !end || !is_comm)) || (n_edges > 0 && (!src || !dst))) return EDM_ERR_BAD_ARG;
  std::vector<Node> node(n_nodes);
  for (int i = 0; i < n_nodes; ++i) {
    if (dur[i] < 0) return EDM_ERR_BAD_ARG;
    node[i].dur = dur[i]; node[i].end = end[i]; node[i].start = end[i] - dur[i]; node[i].is_comm = is_comm[i] != 0;
  }
  std::vector<std::pair<int, int>> edges(n_edges);
  for (int i = 0; i < n_edges; ++i) edges[i] = {src[i], dst[i]};
  std::vector<int> p;
  if (!critical_path(node, edges, *makespan, *exposed_comm, &p)) return EDM_ERR_BAD_ARG;
  if (path_len) {
    if (path) {
      if (*path_len < static_cast<int32_t>(p.size())) return EDM_ERR_CAPACITY;
      for (size_t i = 0; i < p.size(); ++i) path[i] = p[i];
    }
    *path_len = static_cast<int32_t>(p.size());
  }
  return EDM_OK;
}

int edm_select_schedule(const edm_cost_params_t* p, const int32_t* candidates, int32_t n,
                        edm_candidate_cost_t* costs, int32_t* chosen) {
  if (!p || !candidates || !chosen || n < 1) return EDM_ERR_BAD_ARG;
  int32_t arg = 0;
  int64_t best = 0;
  for (int32_t i = 0; i < n; ++i) {
    edm_candidate_cost_t c;
    const int rc = evaluate(*p, candidates[i], c);
    if (rc) return rc;
    if (costs) costs[i] = c;
    if (i == 0 || c.makespan < best) { best = c.makespan; arg = i; }
  }
  *chosen = arg;
  return EDM_OK;
}

}  // extern "C"
