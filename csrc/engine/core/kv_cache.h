// Paged KV-cache bookkeeping (host only): block pool with an intrusive LRU free list and a
// hash -> block prefix cache, per-attention-type block managers, the cross-group
// coordinator and the KVCacheManager facade the scheduler talks to.
//
// Behaviour follows vLLM V1 as restated by the reference
// (src/vllm/v1/core/block_pool.cpp:60-266, single_type_kv_cache_manager.cpp,
// kv_cache_coordinator.cpp, kv_cache_manager.cpp:124-251, include/vllm/v1/kv_cache_interface.h).
#pragma once
#include <deque>
#include <functional>
#include <memory>
#include <optional>
#include <string>
#include <unordered_map>
#include <vector>

#include "core/types.h"

namespace b200 {

// ------------------------------------------------------------------------------- specs
enum class KVSpecKind : int { kFullAttention, kMLA, kSlidingWindow, kChunkedLocal, kMamba };

struct KVCacheSpec {
  KVSpecKind kind = KVSpecKind::kFullAttention;
  int block_size = 16;
  int num_kv_heads = 1;
  int head_size = 128;
  int dtype_bytes = 2;
  int sliding_window = 0;        // kSlidingWindow
  int attention_chunk_size = 0;  // kChunkedLocal
  // kMamba: bytes of recurrent state per request (one "block" holds one request's state)
  int64_t mamba_state_bytes = 0;
  // kMLA: one latent row per token of width head_size (kv_lora_rank + rope dim), no V slab
  int64_t page_size_bytes() const {
    if (kind == KVSpecKind::kMamba) return mamba_state_bytes;
    if (kind == KVSpecKind::kMLA) return (int64_t)block_size * head_size * dtype_bytes;
    return 2ll * block_size * num_kv_heads * head_size * dtype_bytes;
  }
  // Worst-case bytes one request of max_model_len tokens needs in this group.
  int64_t max_memory_usage_bytes(int max_model_len) const;
};

struct KVCacheGroupSpec {
  std::vector<std::string> layer_names;
  KVCacheSpec spec;
};

struct KVCacheConfig {
  int num_blocks = 0;
  std::vector<KVCacheGroupSpec> groups;
};

// ------------------------------------------------------------------------------- blocks
struct KVCacheBlock {
  int block_id = 0;
  int ref_cnt = 0;
  std::optional<std::string> block_hash;  // hash || group id once the block is full & cached
  KVCacheBlock* prev_free = nullptr;
  KVCacheBlock* next_free = nullptr;
  bool is_null = false;
};

// Doubly linked list threaded through the blocks themselves; front = next to evict.
class FreeBlockQueue {
 public:
  explicit FreeBlockQueue(std::vector<KVCacheBlock>& blocks);
  int size() const { return num_free_; }
  KVCacheBlock* popleft();
  std::vector<KVCacheBlock*> popleft_n(int n);
  void remove(KVCacheBlock* b);
  void append(KVCacheBlock* b);
  void prepend(KVCacheBlock* b);
  std::vector<KVCacheBlock*> all_free() const;

 private:
  KVCacheBlock head_, tail_;
  int num_free_ = 0;
};

struct PrefixCacheStats {
  int64_t requests = 0, queries = 0, hits = 0;
  bool reset = false;
};

class BlockPool {
 public:
  BlockPool(int num_gpu_blocks, bool enable_caching);
  KVCacheBlock* null_block() { return null_block_; }
  int num_gpu_blocks() const { return (int)blocks_.size(); }
  bool caching_enabled() const { return enable_caching_; }

  // All groups in `group_ids` must hold the hash; returns one block per group or nullopt.
  std::optional<std::vector<KVCacheBlock*>> get_cached_block(
      const BlockHash& hash, const std::vector<int>& group_ids);
  // Marks blocks [num_cached, num_full) of a request as cached under the request's hashes.
  void cache_full_blocks(const Request& req, const std::vector<KVCacheBlock*>& blocks,
                         int num_cached_blocks, int num_full_blocks, int block_size, int group_id);
  std::vector<KVCacheBlock*> get_new_blocks(int n);  // throws if short
  void touch(const std::vector<KVCacheBlock*>& blocks);
  // `ordered` is in eviction order (first freed = first evicted). Blocks without a hash go
  // to the front of the free list (nothing to lose), hashed ones to the tail.
  void free_blocks(const std::vector<KVCacheBlock*>& ordered);
  bool reset_prefix_cache();
  int get_num_free_blocks() const { return free_.size(); }
  double get_usage() const;
  KVCacheBlock* block(int id) { return &blocks_[id]; }

 private:
  bool maybe_evict_cached_block(KVCacheBlock* b);
  std::vector<KVCacheBlock> blocks_;
  FreeBlockQueue free_;
  bool enable_caching_;
  KVCacheBlock* null_block_ = nullptr;
  // hash||group -> (block id -> block)
  std::unordered_map<std::string, std::unordered_map<int, KVCacheBlock*>> cached_;
};

// ---------------------------------------------------------------- per-type block managers
class SingleTypeKVCacheManager {
 public:
  SingleTypeKVCacheManager(const KVCacheSpec& spec, BlockPool* pool, int group_id)
      : spec_(spec), pool_(pool), group_id_(group_id), block_size_(spec.block_size) {}
  virtual ~SingleTypeKVCacheManager() = default;

  virtual int get_num_blocks_to_allocate(const std::string& req_id, int num_tokens,
                                         const std::vector<KVCacheBlock*>& new_computed);
  virtual void save_new_computed_blocks(const std::string& req_id,
                                        const std::vector<KVCacheBlock*>& new_computed);
  virtual std::vector<KVCacheBlock*> allocate_new_blocks(const std::string& req_id,
                                                         int num_tokens);
  void cache_blocks(const Request& req, int num_tokens);
  virtual void free(const std::string& req_id);
  virtual int get_num_common_prefix_blocks(const std::string& req_id, int num_running) const;
  // Frees blocks that attention will never read again (sliding window / chunked local).
  virtual void remove_skipped_blocks(const std::string& req_id, int num_computed_tokens) {}
  // Longest prefix (in blocks) of `hashes` present in the pool, limited to max_length tokens.
  virtual std::vector<KVCacheBlock*> find_longest_cache_hit(
      const std::vector<BlockHash>& hashes, int max_length) const = 0;
  const std::vector<KVCacheBlock*>& blocks_of(const std::string& req_id) const;
  const KVCacheSpec& spec() const { return spec_; }
  int group_id() const { return group_id_; }

 protected:
  KVCacheSpec spec_;
  BlockPool* pool_;
  int group_id_;
  int block_size_;
  std::unordered_map<std::string, std::vector<KVCacheBlock*>> req_to_blocks_;
  std::unordered_map<std::string, int> num_cached_block_;
};

class FullAttentionManager : public SingleTypeKVCacheManager {
 public:
  using SingleTypeKVCacheManager::SingleTypeKVCacheManager;
  std::vector<KVCacheBlock*> find_longest_cache_hit(const std::vector<BlockHash>& hashes,
                                                    int max_length) const override;
};

class SlidingWindowManager : public SingleTypeKVCacheManager {
 public:
  using SingleTypeKVCacheManager::SingleTypeKVCacheManager;
  std::vector<KVCacheBlock*> find_longest_cache_hit(const std::vector<BlockHash>& hashes,
                                                    int max_length) const override;
  void remove_skipped_blocks(const std::string& req_id, int num_computed_tokens) override;
  int get_num_common_prefix_blocks(const std::string&, int) const override { return 0; }
};

class ChunkedLocalAttentionManager : public SingleTypeKVCacheManager {
 public:
  using SingleTypeKVCacheManager::SingleTypeKVCacheManager;
  std::vector<KVCacheBlock*> find_longest_cache_hit(const std::vector<BlockHash>& hashes,
                                                    int max_length) const override;
  void remove_skipped_blocks(const std::string& req_id, int num_computed_tokens) override;
  int get_num_common_prefix_blocks(const std::string&, int) const override { return 0; }
};

// Recurrent-state group (GDN / Mamba): one state block per request, never prefix-cached.
class MambaManager : public SingleTypeKVCacheManager {
 public:
  using SingleTypeKVCacheManager::SingleTypeKVCacheManager;
  std::vector<KVCacheBlock*> find_longest_cache_hit(const std::vector<BlockHash>&,
                                                    int) const override { return {}; }
  int get_num_blocks_to_allocate(const std::string& req_id, int num_tokens,
                                 const std::vector<KVCacheBlock*>& new_computed) override;
  std::vector<KVCacheBlock*> allocate_new_blocks(const std::string& req_id,
                                                 int num_tokens) override;
  int get_num_common_prefix_blocks(const std::string&, int) const override { return 0; }
};

std::unique_ptr<SingleTypeKVCacheManager> make_single_type_manager(const KVCacheSpec& spec,
                                                                   BlockPool* pool, int group_id);

// ------------------------------------------------------------------------- coordinator
using BlocksPerGroup = std::vector<std::vector<KVCacheBlock*>>;

class KVCacheCoordinator {
 public:
  KVCacheCoordinator(const KVCacheConfig& cfg, int max_model_len, bool enable_caching);
  virtual ~KVCacheCoordinator() = default;
  int get_num_blocks_to_allocate(const std::string& req_id, int num_tokens,
                                 const BlocksPerGroup& new_computed);
  void save_new_computed_blocks(const std::string& req_id, const BlocksPerGroup& new_computed);
  BlocksPerGroup allocate_new_blocks(const std::string& req_id, int num_tokens);
  void cache_blocks(const Request& req, int num_computed_tokens);
  void free(const std::string& req_id);
  std::vector<int> get_num_common_prefix_blocks(const std::string& req_id, int num_running) const;
  void remove_skipped_blocks(const std::string& req_id, int num_computed_tokens);
  BlocksPerGroup get_blocks(const std::string& req_id) const;
  // Returns (blocks per group, number of hit tokens).
  virtual std::pair<BlocksPerGroup, int> find_longest_cache_hit(
      const std::vector<BlockHash>& hashes, int max_cache_hit_length) const = 0;
  BlockPool& pool() { return *pool_; }
  const BlockPool& pool() const { return *pool_; }
  size_t num_groups() const { return managers_.size(); }
  const KVCacheConfig& config() const { return cfg_; }

 protected:
  KVCacheConfig cfg_;
  int max_model_len_;
  bool enable_caching_;
  std::unique_ptr<BlockPool> pool_;
  std::vector<std::unique_ptr<SingleTypeKVCacheManager>> managers_;
};

std::unique_ptr<KVCacheCoordinator> make_kv_cache_coordinator(const KVCacheConfig& cfg,
                                                              int max_model_len,
                                                              bool enable_caching);

// --------------------------------------------------------------------------- the facade
struct KVCacheBlocks {
  BlocksPerGroup blocks;
  std::vector<std::vector<int32_t>> block_ids() const;
  bool empty() const {
    for (auto& g : blocks)
      if (!g.empty()) return false;
    return true;
  }
};

class KVCacheManager {
 public:
  KVCacheManager(const KVCacheConfig& cfg, int max_model_len, bool enable_caching,
                 bool log_stats = true);
  double usage() const { return coord_->pool().get_usage(); }
  // Prefix-cache lookup for a new (num_computed_tokens == 0) request.
  std::pair<KVCacheBlocks, int> get_computed_blocks(Request& req);
  // Returns nullopt when the pool cannot hold the request's new tokens.
  std::optional<KVCacheBlocks> allocate_slots(Request& req, int num_new_tokens,
                                              int num_new_computed_tokens = 0,
                                              const KVCacheBlocks* new_computed_blocks = nullptr,
                                              int num_lookahead_tokens = 0,
                                              bool delay_cache_blocks = false);
  void free(const Request& req);
  bool reset_prefix_cache();
  std::vector<int> get_num_common_prefix_blocks(const Request& req, int num_running) const;
  KVCacheBlocks get_blocks(const std::string& req_id) const;
  std::vector<std::vector<int32_t>> get_block_ids(const std::string& req_id) const;
  void cache_blocks(const Request& req, int num_computed_tokens);
  PrefixCacheStats take_prefix_cache_stats();
  KVCacheBlocks empty_blocks() const;
  BlockPool& pool() { return coord_->pool(); }
  int block_size() const { return block_size_; }
  bool enable_caching() const { return enable_caching_; }
  size_t num_groups() const { return coord_->num_groups(); }
  void new_step_starts() {}

 private:
  int max_model_len_;
  bool enable_caching_;
  bool log_stats_;
  int block_size_ = 16;
  std::unique_ptr<KVCacheCoordinator> coord_;
  PrefixCacheStats stats_;
};

// Appends the hashes of the newly completed blocks of a request to req.block_hashes.
void update_block_hashes(Request& req, int block_size);

}  // namespace b200
