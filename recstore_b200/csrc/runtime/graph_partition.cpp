// Balanced k-way edge-cut partition of the entity graph of a knowledge graph.
//
// The reference cuts the training graph with METIS before it hands every trainer its triples
// (src/kg/kg/dgl-ke/python/dglke/dataloader/sampler.py:408-429, partition.py:35-160): nodes are
// spread over the parts so that few triples cross parts and the parts have equal size; a triple
// belongs to the part of its tail.  No METIS library is needed here: the partitioner below is a
// self-contained multilevel scheme of the same family:
//   1. coarsen  : heavy-edge matching (visit nodes in random order, merge each with the unmatched
//                 neighbour of the heaviest connecting edge, bounded node weight) until the graph
//                 is small or stops shrinking;
//   2. initial  : greedy graph growing on the coarsest graph: parts are grown one node at a time,
//                 the lightest part takes the frontier node with the largest connection to it;
//   3. uncoarsen: project the parts to the finer graph and refine with boundary moves of positive
//                 gain that keep every part under (1 + imbalance) * total / k (a balanced label
//                 propagation, a few sweeps per level).
// Weights: a node weighs the number of fine nodes merged into it, an edge the number of triples
// between its ends.  Everything is deterministic for a given seed.
#include <algorithm>
#include <cstdint>
#include <numeric>
#include <vector>

#include "common/rs_common.h"

namespace {

struct Graph {
  int64_t n = 0;
  std::vector<int64_t> off;      // CSR offsets [n + 1]
  std::vector<int64_t> adj;      // neighbour ids
  std::vector<int64_t> ew;       // edge weights
  std::vector<int64_t> nw;       // node weights
};

struct Rng {
  uint64_t s;
  explicit Rng(uint64_t seed) : s(seed * 0x9E3779B97F4A7C15ull + 0x632BE59BD9B4E019ull) {}
  uint64_t next() { s ^= s << 13; s ^= s >> 7; s ^= s << 17; return s; }
};

// Symmetric CSR with merged parallel edges and no self loops, from (u, v, w) triples.
Graph build_graph(int64_t n, std::vector<int64_t>& eu, std::vector<int64_t>& ev, std::vector<int64_t>& ewt,
                  std::vector<int64_t> nw) {
  const size_t m = eu.size();
  std::vector<int64_t> deg(n + 1, 0);
  for (size_t e = 0; e < m; ++e) {
    if (eu[e] == ev[e]) continue;
    ++deg[eu[e] + 1]; ++deg[ev[e] + 1];
  }
  for (int64_t i = 0; i < n; ++i) deg[i + 1] += deg[i];
  std::vector<int64_t> adj(deg[n]), w(deg[n]), pos(deg.begin(), deg.end() - 1);
  for (size_t e = 0; e < m; ++e) {
    if (eu[e] == ev[e]) continue;
    adj[pos[eu[e]]] = ev[e]; w[pos[eu[e]]++] = ewt[e];
    adj[pos[ev[e]]] = eu[e]; w[pos[ev[e]]++] = ewt[e];
  }
  Graph g;
  g.n = n; g.nw = std::move(nw); g.off.assign(n + 1, 0);
  std::vector<std::pair<int64_t, int64_t>> row;
  for (int64_t i = 0; i < n; ++i) {      // sort each row, merge duplicates
    row.clear();
    for (int64_t p = deg[i]; p < deg[i + 1]; ++p) row.emplace_back(adj[p], w[p]);
    std::sort(row.begin(), row.end());
    for (size_t p = 0; p < row.size(); ++p) {
      if (!g.adj.empty() && static_cast<int64_t>(g.adj.size()) > g.off[i] && g.adj.back() == row[p].first) {
        g.ew.back() += row[p].second;
      } else {
        g.adj.push_back(row[p].first); g.ew.push_back(row[p].second);
      }
    }
    g.off[i + 1] = static_cast<int64_t>(g.adj.size());
  }
  return g;
}

// Heavy-edge matching; returns the coarse graph and fills map[fine] = coarse.
Graph coarsen(const Graph& g, std::vector<int64_t>& map, int64_t max_nw, Rng& rng) {
  std::vector<int64_t> order(g.n);
  std::iota(order.begin(), order.end(), 0);
  for (int64_t i = g.n - 1; i > 0; --i) std::swap(order[i], order[rng.next() % static_cast<uint64_t>(i + 1)]);
  map.assign(g.n, -1);
  int64_t nc = 0;
  for (int64_t v : order) {
    if (map[v] >= 0) continue;
    int64_t best = -1, best_w = 0;
    for (int64_t p = g.off[v]; p < g.off[v + 1]; ++p) {
      const int64_t u = g.adj[p];
      if (map[u] < 0 && g.ew[p] > best_w && g.nw[v] + g.nw[u] <= max_nw) { best = u; best_w = g.ew[p]; }
    }
    map[v] = nc;
    if (best >= 0) map[best] = nc;
    ++nc;
  }
  std::vector<int64_t> nw(nc, 0), eu, ev, ewt;
  for (int64_t v = 0; v < g.n; ++v) nw[map[v]] += g.nw[v];
  eu.reserve(g.adj.size() / 2); ev.reserve(g.adj.size() / 2); ewt.reserve(g.adj.size() / 2);
  for (int64_t v = 0; v < g.n; ++v)
    for (int64_t p = g.off[v]; p < g.off[v + 1]; ++p)
      if (v < g.adj[p] && map[v] != map[g.adj[p]]) { eu.push_back(map[v]); ev.push_back(map[g.adj[p]]); ewt.push_back(g.ew[p]); }
  return build_graph(nc, eu, ev, ewt, std::move(nw));
}

// Greedy graph growing: the lightest part takes the unassigned node it is best connected to (a random one if it has
// no frontier).
void initial_partition(const Graph& g, int k, std::vector<int32_t>& part, Rng& rng) {
  part.assign(g.n, -1);
  std::vector<int64_t> load(k, 0);
  std::vector<std::vector<int64_t>> conn(k, std::vector<int64_t>(g.n, 0));   // coarsest graph only: k * n is small
  std::vector<int64_t> free_nodes(g.n);
  std::iota(free_nodes.begin(), free_nodes.end(), 0);
  for (int64_t i = g.n - 1; i > 0; --i) std::swap(free_nodes[i], free_nodes[rng.next() % static_cast<uint64_t>(i + 1)]);
  size_t cursor = 0;
  for (int64_t done = 0; done < g.n; ++done) {
    const int p = static_cast<int>(std::min_element(load.begin(), load.end()) - load.begin());
    int64_t best = -1, best_c = 0;
    for (int64_t v = 0; v < g.n; ++v)
      if (part[v] < 0 && conn[p][v] > best_c) { best = v; best_c = conn[p][v]; }
    if (best < 0) {
      while (part[free_nodes[cursor]] >= 0) ++cursor;
      best = free_nodes[cursor];
    }
    part[best] = p; load[p] += g.nw[best];
    for (int64_t q = g.off[best]; q < g.off[best + 1]; ++q) conn[p][g.adj[q]] += g.ew[q];
  }
}

// Boundary refinement: move a node to the neighbouring part with the largest positive gain that has room; a node of
// an overweight part may also move at zero or negative gain to the best part with room.
void refine(const Graph& g, int k, std::vector<int32_t>& part, int64_t cap, int sweeps, Rng& rng) {
  std::vector<int64_t> load(k, 0), conn(k, 0);
  for (int64_t v = 0; v < g.n; ++v) load[part[v]] += g.nw[v];
  std::vector<int64_t> order(g.n);
  std::iota(order.begin(), order.end(), 0);
  std::vector<int> touched;
  for (int s = 0; s < sweeps; ++s) {
    for (int64_t i = g.n - 1; i > 0; --i) std::swap(order[i], order[rng.next() % static_cast<uint64_t>(i + 1)]);
    int64_t moved = 0;
    for (int64_t v : order) {
      const int from = part[v];
      touched.clear();
      for (int64_t p = g.off[v]; p < g.off[v + 1]; ++p) {
        const int q = part[g.adj[p]];
        if (conn[q] == 0) touched.push_back(q);
        conn[q] += g.ew[p];
      }
      const bool over = load[from] > cap;
      int best = -1;
      int64_t best_gain = over ? INT64_MIN : 0;
      for (int q : touched) {
        if (q == from || load[q] + g.nw[v] > cap) continue;
        const int64_t gain = conn[q] - conn[from];
        if (gain > best_gain || (gain == best_gain && best >= 0 && load[q] < load[best])) { best = q; best_gain = gain; }
      }
      if (over && best < 0) {                      // no neighbouring part has room: take the lightest part
        const int q = static_cast<int>(std::min_element(load.begin(), load.end()) - load.begin());
        if (q != from && load[q] + g.nw[v] <= cap) best = q;
      }
      if (best >= 0) { part[v] = best; load[from] -= g.nw[v]; load[best] += g.nw[v]; ++moved; }
      for (int q : touched) conn[q] = 0;
    }
    if (moved == 0) break;
  }
}

}  // namespace

// Partitions the nodes [0, n_nodes) of the graph given by `n_edges` (src, dst) pairs into `k` parts.
// `node_weight` (optional, [n_nodes], positive) is what the parts balance; without it every node weighs 1.
// part_out[n_nodes] receives the part of every node; stats_out[0] = number of edges whose ends lie in different
// parts, stats_out[1] = weight of the heaviest part, stats_out[2] = number of levels used, stats_out[3] = total weight.
static int partition_impl(long long n_nodes, long long n_edges, const long long* src, const long long* dst,
                          const long long* node_weight, int k, double imbalance, unsigned long long seed,
                          int refine_sweeps, int* part_out, long long* stats_out) {
  RS_REQUIRE(n_nodes > 0 && n_edges >= 0 && k > 0 && part_out, "rs_graph_partition: bad sizes");
  RS_REQUIRE(n_edges == 0 || (src && dst), "rs_graph_partition: null edge list");
  RS_REQUIRE(imbalance >= 0.0 && refine_sweeps >= 0, "rs_graph_partition: bad imbalance / sweeps");
  for (long long e = 0; e < n_edges; ++e)
    RS_REQUIRE(src[e] >= 0 && src[e] < n_nodes && dst[e] >= 0 && dst[e] < n_nodes, "rs_graph_partition: node id out of range");
  if (k == 1) {
    std::fill(part_out, part_out + n_nodes, 0);
    if (stats_out) { stats_out[0] = 0; stats_out[1] = n_nodes; stats_out[2] = 0; stats_out[3] = n_nodes; }
    return RS_OK;
  }
  Rng rng(seed);
  std::vector<int64_t> eu(src, src + n_edges), ev(dst, dst + n_edges), ew(n_edges, 1);
  std::vector<int64_t> nw0(n_nodes, 1);
  if (node_weight)
    for (long long v = 0; v < n_nodes; ++v) {
      RS_REQUIRE(node_weight[v] > 0, "rs_graph_partition: node weights must be positive");
      nw0[v] = node_weight[v];
    }
  const int64_t total_w = std::accumulate(nw0.begin(), nw0.end(), static_cast<int64_t>(0));
  std::vector<Graph> levels;
  levels.push_back(build_graph(n_nodes, eu, ev, ew, nw0));
  std::vector<std::vector<int64_t>> maps;
  const int64_t coarse_target = std::max<int64_t>(64, 20ll * k);
  const int64_t max_nw = std::max<int64_t>(1, total_w / (4ll * k));     // no coarse node heavier than a quarter of a part
  while (levels.back().n > coarse_target && levels.size() < 40) {
    std::vector<int64_t> map;
    Graph c = coarsen(levels.back(), map, max_nw, rng);
    if (c.n > levels.back().n * 95 / 100) break;                         // matching no longer shrinks the graph
    maps.push_back(std::move(map));
    levels.push_back(std::move(c));
  }
  const int64_t cap = static_cast<int64_t>((1.0 + imbalance) * static_cast<double>(total_w) / k) + 1;
  std::vector<int32_t> part;
  if (levels.back().n <= 4096) {
    initial_partition(levels.back(), k, part, rng);
  } else {                                                                // coarsening stalled on a large graph: start from blocks
    part.resize(levels.back().n);
    for (int64_t v = 0; v < levels.back().n; ++v) part[v] = static_cast<int32_t>(v * k / levels.back().n);
  }
  refine(levels.back(), k, part, cap, refine_sweeps, rng);
  for (int64_t l = static_cast<int64_t>(levels.size()) - 2; l >= 0; --l) {
    std::vector<int32_t> fine(levels[l].n);
    for (int64_t v = 0; v < levels[l].n; ++v) fine[v] = part[maps[l][v]];
    part.swap(fine);
    refine(levels[l], k, part, cap, refine_sweeps, rng);
  }
  std::vector<int64_t> load(k, 0);
  for (long long v = 0; v < n_nodes; ++v) { part_out[v] = part[v]; load[part[v]] += nw0[v]; }
  if (stats_out) {
    long long cut = 0;
    for (long long e = 0; e < n_edges; ++e) cut += part[src[e]] != part[dst[e]];
    stats_out[0] = cut;
    stats_out[1] = *std::max_element(load.begin(), load.end());
    stats_out[2] = static_cast<long long>(levels.size());
    stats_out[3] = total_w;
  }
  return RS_OK;
}

RS_API int rs_graph_partition(long long n_nodes, long long n_edges, const long long* src, const long long* dst,
                              const long long* node_weight, int k, double imbalance, unsigned long long seed,
                              int refine_sweeps, int* part_out, long long* stats_out) {
  RS_NOEXCEPT_BODY(return partition_impl(n_nodes, n_edges, src, dst, node_weight, k, imbalance, seed, refine_sweeps, part_out, stats_out);)
}
