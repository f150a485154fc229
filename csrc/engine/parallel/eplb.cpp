#include "eplb.h"

#include <algorithm>
#include <numeric>
#include <stdexcept>

namespace b200 {

void eplb_balanced_packing(const std::vector<double>& weight, int rows, int n, int num_packs,
                           std::vector<int32_t>* pack_index, std::vector<int32_t>* rank_in_pack) {
  if (num_packs <= 0 || n % num_packs) throw std::invalid_argument("eplb: items do not divide into packs");
  const int per_pack = n / num_packs;
  pack_index->assign((size_t)rows * n, -1);
  rank_in_pack->assign((size_t)rows * n, -1);
  std::vector<int> order(n);
  std::vector<double> load(num_packs);
  std::vector<int> count(num_packs);
  for (int r = 0; r < rows; ++r) {
    const double* w = weight.data() + (size_t)r * n;
    if (per_pack == 1) {
      for (int i = 0; i < n; ++i) { (*pack_index)[(size_t)r * n + i] = i; (*rank_in_pack)[(size_t)r * n + i] = 0; }
      continue;
    }
    std::iota(order.begin(), order.end(), 0);
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return w[a] > w[b]; });
    std::fill(load.begin(), load.end(), 0.0);
    std::fill(count.begin(), count.end(), 0);
    for (int idx : order) {
      int best = -1;
      for (int p = 0; p < num_packs; ++p)
        if (count[p] < per_pack && (best < 0 || load[p] < load[best])) best = p;
      (*pack_index)[(size_t)r * n + idx] = best;
      (*rank_in_pack)[(size_t)r * n + idx] = count[best];
      load[best] += w[idx];
      count[best]++;
    }
  }
}

void eplb_replicate(const std::vector<double>& weight, int rows, int num_log, int num_phy,
                    std::vector<int32_t>* phy2log, std::vector<int32_t>* phy_rank, std::vector<int32_t>* logcnt) {
  if (num_phy < num_log) throw std::invalid_argument("eplb: fewer physical slots than experts");
  phy2log->assign((size_t)rows * num_phy, 0);
  phy_rank->assign((size_t)rows * num_phy, 0);
  logcnt->assign((size_t)rows * num_log, 1);
  for (int r = 0; r < rows; ++r) {
    const double* w = weight.data() + (size_t)r * num_log;
    int32_t* p2l = phy2log->data() + (size_t)r * num_phy;
    int32_t* pr = phy_rank->data() + (size_t)r * num_phy;
    int32_t* cnt = logcnt->data() + (size_t)r * num_log;
    for (int i = 0; i < num_log; ++i) p2l[i] = i;
    for (int s = num_log; s < num_phy; ++s) {
      int best = 0;
      double best_v = w[0] / cnt[0];
      for (int i = 1; i < num_log; ++i) {
        const double v = w[i] / cnt[i];
        if (v > best_v) { best_v = v; best = i; }
      }
      p2l[s] = best;
      pr[s] = cnt[best];
      cnt[best]++;
    }
  }
}

namespace {

// One layer row of the hierarchical policy; writes phy2log / phy_rank / logcnt of that layer.
void rebalance_hierarchical(const double* w, int num_log, int num_phy, int num_groups, int num_nodes, int num_ranks,
                            int32_t* phy2log, int32_t* phy_rank, int32_t* logcnt) {
  const int group_size = num_log / num_groups;
  const int groups_per_node = num_groups / num_nodes;
  const int phy_per_rank = num_phy / num_ranks;
  const int log_per_node = num_log / num_nodes;
  const int phy_per_node = num_phy / num_nodes;
  const int ranks_per_node = num_ranks / num_nodes;
  // 1. expert groups -> nodes
  std::vector<double> per_group(num_groups, 0.0);
  for (int i = 0; i < num_log; ++i) per_group[i / group_size] += w[i];
  std::vector<int32_t> g_pack, g_rank;
  eplb_balanced_packing(per_group, 1, num_groups, num_nodes, &g_pack, &g_rank);
  // logical expert -> "node-ordered" index (mlog) and back
  std::vector<int> log2mlog(num_log), mlog2log(num_log);
  for (int i = 0; i < num_log; ++i) {
    const int g = i / group_size;
    const int m = (g_pack[g] * groups_per_node + g_rank[g]) * group_size + i % group_size;
    log2mlog[i] = m;
    mlog2log[m] = i;
  }
  // 2. replicas within each node
  std::vector<double> per_mlog((size_t)num_nodes * log_per_node);
  for (int m = 0; m < num_log; ++m) per_mlog[m] = w[mlog2log[m]];
  std::vector<int32_t> p2m, prank, mcnt;
  eplb_replicate(per_mlog, num_nodes, log_per_node, phy_per_node, &p2m, &prank, &mcnt);
  // 3. physical slots of a node -> its ranks
  std::vector<double> per_phy((size_t)num_nodes * phy_per_node);
  for (int nd = 0; nd < num_nodes; ++nd)
    for (int s = 0; s < phy_per_node; ++s) {
      const int m = p2m[(size_t)nd * phy_per_node + s];
      per_phy[(size_t)nd * phy_per_node + s] = per_mlog[(size_t)nd * log_per_node + m] / mcnt[(size_t)nd * log_per_node + m];
    }
  std::vector<int32_t> s_pack, s_rank;
  eplb_balanced_packing(per_phy, num_nodes, phy_per_node, ranks_per_node, &s_pack, &s_rank);
  for (int nd = 0; nd < num_nodes; ++nd)
    for (int s = 0; s < phy_per_node; ++s) {
      const size_t k = (size_t)nd * phy_per_node + s;
      const int final_slot = nd * phy_per_node + s_pack[k] * phy_per_rank + s_rank[k];
      const int mlog = nd * log_per_node + p2m[k];
      phy2log[final_slot] = mlog2log[mlog];
      phy_rank[final_slot] = prank[k];
    }
  for (int i = 0; i < num_log; ++i) {
    const int m = log2mlog[i];
    logcnt[i] = mcnt[m];     // mcnt is laid out [node][log_per_node] = mlog order
  }
}

}  // namespace

EplbPlacement eplb_rebalance(const std::vector<double>& loads, int num_layers, int num_logical, int num_physical,
                             int num_groups, int num_nodes, int num_ranks) {
  if (num_layers <= 0 || num_logical <= 0 || (size_t)num_layers * num_logical != loads.size())
    throw std::invalid_argument("eplb: loads must be [layers][experts]");
  if (num_ranks <= 0 || num_nodes <= 0 || num_ranks % num_nodes || num_physical % num_ranks ||
      num_physical < num_logical)
    throw std::invalid_argument("eplb: physical slots must cover the experts and divide over the ranks");
  if (num_groups <= 0 || num_logical % num_groups) throw std::invalid_argument("eplb: experts do not divide into groups");
  // the group -> node step needs whole groups per node; otherwise one global pool
  if (num_groups % num_nodes || num_logical % num_nodes || num_physical % num_nodes) {
    num_groups = 1;
    if (num_logical % num_nodes || num_physical % num_nodes) num_nodes = 1;
  }
  if (num_groups % num_nodes) { num_groups = 1; num_nodes = 1; }
  EplbPlacement out;
  out.num_layers = num_layers; out.num_logical = num_logical; out.num_physical = num_physical;
  out.phy2log.assign((size_t)num_layers * num_physical, 0);
  out.phy_rank.assign((size_t)num_layers * num_physical, 0);
  out.logcnt.assign((size_t)num_layers * num_logical, 0);
  for (int l = 0; l < num_layers; ++l)
    rebalance_hierarchical(loads.data() + (size_t)l * num_logical, num_logical, num_physical, num_groups, num_nodes,
                           num_ranks, out.phy2log.data() + (size_t)l * num_physical,
                           out.phy_rank.data() + (size_t)l * num_physical, out.logcnt.data() + (size_t)l * num_logical);
  out.max_replicas = *std::max_element(out.logcnt.begin(), out.logcnt.end());
  out.log2phy.assign((size_t)num_layers * num_logical * out.max_replicas, -1);
  for (int l = 0; l < num_layers; ++l)
    for (int s = 0; s < num_physical; ++s) {
      const int e = out.phy2log[(size_t)l * num_physical + s];
      const int r = out.phy_rank[(size_t)l * num_physical + s];
      out.log2phy[((size_t)l * num_logical + e) * out.max_replicas + r] = s;
    }
  return out;
}

}  // namespace b200
