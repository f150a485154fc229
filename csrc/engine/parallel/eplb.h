// Expert-parallel load balancing: from per-layer, per-expert token counts to a placement of
// physical expert slots on ranks. A logical expert that is hot gets several physical replicas; the
// slots are then packed on the ranks so that every rank carries about the same load, and (when the
// model routes within expert groups and the job spans several nodes) the experts of one group stay
// on one node. The reference project has no expert parallelism; this follows the published
// hierarchical / global policy that serving stacks use for DeepSeek-style models.
#pragma once
#include <cstdint>
#include <vector>

namespace b200 {

struct EplbPlacement {
  int num_layers = 0, num_logical = 0, num_physical = 0, max_replicas = 0;
  std::vector<int32_t> phy2log;   // [layers][num_physical]: logical expert held by each slot
  std::vector<int32_t> phy_rank;  // [layers][num_physical]: which replica of its expert the slot is
  std::vector<int32_t> log2phy;   // [layers][num_logical][max_replicas]: slots of an expert, -1 padded
  std::vector<int32_t> logcnt;    // [layers][num_logical]: replicas per expert
};

// items -> packs of exactly n / num_packs items each, heaviest first into the lightest pack that
// still has room. weight: [rows][n]. Writes pack index and position within the pack per item.
void eplb_balanced_packing(const std::vector<double>& weight, int rows, int n, int num_packs,
                           std::vector<int32_t>* pack_index, std::vector<int32_t>* rank_in_pack);

// num_phy >= num_log slots over num_log experts: one each, then every further slot goes to the
// expert whose load per replica is highest. weight: [rows][num_log].
void eplb_replicate(const std::vector<double>& weight, int rows, int num_log, int num_phy,
                    std::vector<int32_t>* phy2log, std::vector<int32_t>* phy_rank, std::vector<int32_t>* logcnt);

// loads: [layers][num_logical] (token counts of a window). num_physical slots in total, a multiple
// of num_ranks; num_groups expert groups (1: no group structure); num_nodes nodes of
// num_ranks / num_nodes ranks. Slots [r * S, (r + 1) * S) belong to rank r, S = num_physical / num_ranks.
// Throws std::invalid_argument on sizes that do not divide.
EplbPlacement eplb_rebalance(const std::vector<double>& loads, int num_layers, int num_logical, int num_physical,
                             int num_groups, int num_nodes, int num_ranks);

}  // namespace b200
