// KV-cache offloading: blocks that leave the GPU cache stay reachable in host memory and on
// disk, keyed by the same chained block hashes as the GPU prefix cache.
//
//   CachePolicy (LRU, ARC)      which resident block to evict
//   CpuTier                     fixed pool of host block slots + hash -> slot map
//   FsTier                      one file per block under a directory, identity-checked header,
//                               size budget with oldest-first eviction
//   TieringManager              lookup across tiers; a disk hit is first promoted to the host
//                               tier ("retry" on the first lookup, "hit" once it is resident);
//                               host evictions cascade down to disk
//   OffloadConnector            scheduler-side KV connector: counts externally cached tokens for
//                               a new request, plans loads into its freshly allocated GPU
//                               blocks and stores of finished requests' blocks; the worker
//                               executes the plan (ConnectorMeta) with plain copies
//
// Reference: include/vllm/v1/kv_offload/{kv_connector,base,tiering_manager,cpu_manager,
// cache_policy,fs_io,fs_tier,cache_identity,kv_block_transfer}.h.
#pragma once
#include <cstdint>
#include <functional>
#include <list>
#include <map>
#include <memory>
#include <mutex>
#include <optional>
#include <string>
#include <unordered_map>
#include <vector>

#include "../core/scheduler.h"

namespace b200 {
namespace offload {

using Key = std::string;   // 32-byte block hash

// ------------------------------------------------------------------------------ policies
class CachePolicy {
 public:
  virtual ~CachePolicy() = default;
  virtual void insert(const Key& k) = 0;
  virtual void touch(const Key& k) = 0;            // hit
  virtual void erase(const Key& k) = 0;
  // Next victim among resident keys for which `evictable(key)` holds; nullopt if none.
  virtual std::optional<Key> victim(const std::function<bool(const Key&)>& evictable) = 0;
  virtual size_t size() const = 0;
  static std::unique_ptr<CachePolicy> make(const std::string& name, size_t capacity);
};

class LruPolicy : public CachePolicy {
 public:
  void insert(const Key& k) override;
  void touch(const Key& k) override;
  void erase(const Key& k) override;
  std::optional<Key> victim(const std::function<bool(const Key&)>& evictable) override;
  size_t size() const override { return order_.size(); }

 private:
  std::list<Key> order_;   // front = coldest
  std::unordered_map<Key, std::list<Key>::iterator> pos_;
};

// Adaptive replacement cache: recency list T1, frequency list T2 and their ghost lists B1 /
// B2; the target size p of T1 moves toward whichever ghost list gets hit.
class ArcPolicy : public CachePolicy {
 public:
  explicit ArcPolicy(size_t capacity) : cap_(capacity) {}
  void insert(const Key& k) override;
  void touch(const Key& k) override;
  void erase(const Key& k) override;
  std::optional<Key> victim(const std::function<bool(const Key&)>& evictable) override;
  size_t size() const override { return t1_.size() + t2_.size(); }
  size_t target_t1() const { return p_; }

 private:
  using List = std::list<Key>;
  struct Where { int list; List::iterator it; };   // 0 T1, 1 T2, 2 B1, 3 B2
  void remove_from(const Key& k);
  void push(int list, const Key& k);
  List& L(int i) { return i == 0 ? t1_ : i == 1 ? t2_ : i == 2 ? b1_ : b2_; }
  size_t cap_, p_ = 0;
  List t1_, t2_, b1_, b2_;
  std::unordered_map<Key, Where> where_;
};

// ------------------------------------------------------------------------------ tiers
struct TierStats {
  uint64_t hits = 0, misses = 0, stores = 0, evictions = 0;
};

class CpuTier {
 public:
  CpuTier(int num_slots, const std::string& policy);
  bool contains(const Key& k) const { return slot_of_.count(k) > 0; }
  int slot(const Key& k) const;                       // -1 if absent
  void touch(const Key& k);
  // Reserves a slot for `k` (evicting if needed; *evicted receives the victim's key and the
  // slot it occupied so that the caller can demote it first). -1 when every slot is pinned.
  int reserve(const Key& k, Key* evicted_key, bool* evicted);
  void pin(const Key& k, int delta);                  // loads in flight must not be evicted
  void erase(const Key& k);
  int num_slots() const { return (int)free_.size() + (int)slot_of_.size(); }
  int num_resident() const { return (int)slot_of_.size(); }
  TierStats stats;

 private:
  std::unique_ptr<CachePolicy> policy_;
  std::unordered_map<Key, int> slot_of_;
  std::unordered_map<Key, int> pins_;
  std::vector<int> free_;
};

// Identity of a cache: blocks written for another model / layout / dtype must never be read.
struct CacheIdentity {
  std::string model;     // free-form model id
  int block_size = 0;
  int64_t block_bytes = 0;
  std::string dtype;
  std::string digest() const;   // hex sha256 of the fields
};

class FsTier {
 public:
  FsTier(std::string dir, CacheIdentity id, int64_t max_bytes);
  bool contains(const Key& k) const;
  // Reads the block into `dst` (block_bytes); false if absent, foreign or corrupt (such files
  // are removed).
  bool read(const Key& k, void* dst);
  bool write(const Key& k, const void* src);
  void erase(const Key& k);
  int64_t bytes_used() const { return used_; }
  size_t num_blocks() const { return index_.size(); }
  std::string path_of(const Key& k) const;
  TierStats stats;

 private:
  void scan();
  void enforce_budget();
  std::string dir_;
  CacheIdentity id_;
  std::string id_digest_;
  int64_t max_bytes_, used_ = 0;
  uint64_t clock_ = 0;
  std::map<Key, uint64_t> index_;            // key -> last-use tick
};

enum class Lookup { kMiss, kRetry, kHit };

// One planned copy. kind: 0 = host slot -> GPU block, 1 = GPU block -> host slot.
struct Transfer {
  int kind;
  int cpu_slot;
  int32_t gpu_block;
  Key key;
};

class TieringManager {
 public:
  // `host_base`: address of the host pool (num_slots * block_bytes) owned by the caller; the
  // disk tier reads into / writes from it directly. May be null when there is no disk tier.
  TieringManager(int num_cpu_slots, const std::string& policy, uint8_t* host_base, int64_t block_bytes,
                 std::unique_ptr<FsTier> fs);
  // kHit: resident in the host tier. kRetry: found on disk and now promoted (resident for the
  // next lookup). kMiss: nowhere.
  Lookup lookup(const Key& k);
  CpuTier& cpu() { return cpu_; }
  FsTier* fs() { return fs_.get(); }
  // Reserves a host slot for a block about to be stored; a displaced block is written to disk
  // first (cascade). Returns -1 if nothing can be evicted.
  int reserve_for_store(const Key& k);
  void reset();

 private:
  CpuTier cpu_;
  uint8_t* host_;
  int64_t block_bytes_;
  std::unique_ptr<FsTier> fs_;
  int num_slots_;
  std::string policy_name_;
};

// ------------------------------------------------------------------------------ connector
struct ConnectorMeta {
  std::vector<Transfer> loads;    // before the forward pass
  std::vector<Transfer> stores;   // after it
};

class OffloadConnector : public KVConnectorHook {
 public:
  OffloadConnector(std::shared_ptr<TieringManager> tiers, int block_size);
  std::optional<std::pair<int, bool>> get_num_new_matched_tokens(const Request& req,
                                                                 int num_computed_tokens) override;
  void update_state_after_alloc(const Request& req, const std::vector<std::vector<int32_t>>& block_ids,
                                int num_external_tokens) override;
  std::shared_ptr<void> build_connector_meta(const SchedulerOutput& out) override;
  bool request_finished(const Request& req, const std::vector<std::vector<int32_t>>& block_ids) override;
  // The worker reports finished transfers so that pins are dropped and stores become visible.
  void transfers_done(const ConnectorMeta& meta);
  std::shared_ptr<ConnectorMeta> take_meta();   // the plan of the step just scheduled
  TieringManager& tiers() { return *tiers_; }

 private:
  std::shared_ptr<TieringManager> tiers_;
  int block_size_;
  std::mutex mu_;
  std::vector<Transfer> pending_loads_, pending_stores_;
  std::shared_ptr<ConnectorMeta> last_;
};

}  // namespace offload
}  // namespace b200
