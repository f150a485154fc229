#include "core/kv_cache.h"

#include <algorithm>
#include <cassert>

#include "core/hashing.h"

namespace b200 {

static inline int cdiv(int a, int b) { return (a + b - 1) / b; }

int64_t KVCacheSpec::max_memory_usage_bytes(int max_model_len) const {
  switch (kind) {
    case KVSpecKind::kMamba: return mamba_state_bytes;
    case KVSpecKind::kSlidingWindow: {
      int tokens = std::min(sliding_window - 1 + max_model_len, max_model_len);
      return (int64_t)(cdiv(tokens, block_size) + 1) * page_size_bytes();
    }
    case KVSpecKind::kChunkedLocal: {
      int tokens = std::min(attention_chunk_size + max_model_len, max_model_len);
      return (int64_t)cdiv(tokens, block_size) * page_size_bytes();
    }
    default: return (int64_t)cdiv(max_model_len, block_size) * page_size_bytes();
  }
}

// ------------------------------------------------------------------------ FreeBlockQueue
FreeBlockQueue::FreeBlockQueue(std::vector<KVCacheBlock>& blocks) {
  head_.next_free = &tail_;
  tail_.prev_free = &head_;
  for (auto& b : blocks) append(&b);
}
KVCacheBlock* FreeBlockQueue::popleft() {
  if (num_free_ == 0) throw std::runtime_error("No free blocks available");
  KVCacheBlock* b = head_.next_free;
  remove(b);
  return b;
}
std::vector<KVCacheBlock*> FreeBlockQueue::popleft_n(int n) {
  if (n > num_free_) throw std::runtime_error("Cannot pop more blocks than are free");
  std::vector<KVCacheBlock*> r;
  r.reserve(n);
  for (int i = 0; i < n; ++i) r.push_back(popleft());
  return r;
}
void FreeBlockQueue::remove(KVCacheBlock* b) {
  if (!b->prev_free || !b->next_free) throw std::runtime_error("remove() on a block not in the free list");
  b->prev_free->next_free = b->next_free;
  b->next_free->prev_free = b->prev_free;
  b->prev_free = b->next_free = nullptr;
  --num_free_;
}
void FreeBlockQueue::append(KVCacheBlock* b) {
  KVCacheBlock* last = tail_.prev_free;
  last->next_free = b;
  b->prev_free = last;
  b->next_free = &tail_;
  tail_.prev_free = b;
  ++num_free_;
}
void FreeBlockQueue::prepend(KVCacheBlock* b) {
  KVCacheBlock* first = head_.next_free;
  head_.next_free = b;
  b->prev_free = &head_;
  b->next_free = first;
  first->prev_free = b;
  ++num_free_;
}
std::vector<KVCacheBlock*> FreeBlockQueue::all_free() const {
  std::vector<KVCacheBlock*> r;
  for (KVCacheBlock* b = head_.next_free; b != &tail_; b = b->next_free) r.push_back(b);
  return r;
}

// ----------------------------------------------------------------------------- BlockPool
static std::vector<KVCacheBlock> make_blocks(int n) {
  std::vector<KVCacheBlock> v(n);
  for (int i = 0; i < n; ++i) v[i].block_id = i;
  return v;
}

BlockPool::BlockPool(int num_gpu_blocks, bool enable_caching)
    : blocks_(make_blocks(num_gpu_blocks)), free_(blocks_), enable_caching_(enable_caching) {
  if (num_gpu_blocks <= 0) throw std::invalid_argument("num_gpu_blocks must be positive");
  // Block 0 is reserved as the "null" placeholder (e.g. for slots outside a sliding window).
  null_block_ = free_.popleft();
  null_block_->is_null = true;
}

std::optional<std::vector<KVCacheBlock*>> BlockPool::get_cached_block(
    const BlockHash& hash, const std::vector<int>& group_ids) {
  std::vector<KVCacheBlock*> r;
  for (int g : group_ids) {
    auto it = cached_.find(hash_with_group(hash, (uint32_t)g));
    if (it == cached_.end() || it->second.empty()) return std::nullopt;
    r.push_back(it->second.begin()->second);
  }
  return r;
}

void BlockPool::cache_full_blocks(const Request& req, const std::vector<KVCacheBlock*>& blocks,
                                  int num_cached_blocks, int num_full_blocks, int block_size,
                                  int group_id) {
  (void)block_size;
  if (!enable_caching_ || num_cached_blocks >= num_full_blocks) return;
  if ((int)req.block_hashes.size() < num_full_blocks)
    throw std::runtime_error("cache_full_blocks: request has fewer block hashes than full blocks");
  for (int i = num_cached_blocks; i < num_full_blocks; ++i) {
    KVCacheBlock* b = blocks[i];
    if (b->is_null || b->block_hash) continue;
    std::string key = hash_with_group(req.block_hashes[i], (uint32_t)group_id);
    b->block_hash = key;
    cached_[key][b->block_id] = b;
  }
}

bool BlockPool::maybe_evict_cached_block(KVCacheBlock* b) {
  if (!b->block_hash) return false;
  auto it = cached_.find(*b->block_hash);
  if (it != cached_.end()) {
    it->second.erase(b->block_id);
    if (it->second.empty()) cached_.erase(it);
  }
  b->block_hash.reset();
  return true;
}

std::vector<KVCacheBlock*> BlockPool::get_new_blocks(int n) {
  if (n > free_.size()) throw std::runtime_error("Cannot get " + std::to_string(n) + " free blocks from the pool");
  auto r = free_.popleft_n(n);
  for (KVCacheBlock* b : r) {
    if (enable_caching_) maybe_evict_cached_block(b);
    assert(b->ref_cnt == 0);
    b->ref_cnt = 1;
  }
  return r;
}

void BlockPool::touch(const std::vector<KVCacheBlock*>& blocks) {
  for (KVCacheBlock* b : blocks) {
    if (b->ref_cnt == 0 && !b->is_null) free_.remove(b);
    ++b->ref_cnt;
  }
}

void BlockPool::free_blocks(const std::vector<KVCacheBlock*>& ordered) {
  std::vector<KVCacheBlock*> unhashed;
  for (KVCacheBlock* b : ordered) {
    if (b->is_null) continue;
    --b->ref_cnt;
    if (b->ref_cnt == 0) {
      if (b->block_hash) free_.append(b);
      else unhashed.push_back(b);
    }
  }
  // Keep relative order among the unhashed blocks at the front.
  for (auto it = unhashed.rbegin(); it != unhashed.rend(); ++it) free_.prepend(*it);
}

bool BlockPool::reset_prefix_cache() {
  int used = (int)blocks_.size() - free_.size();
  if (used != 1) return false;  // only the null block may be out
  cached_.clear();
  for (auto& b : blocks_) b.block_hash.reset();
  return true;
}

double BlockPool::get_usage() const {
  int total = (int)blocks_.size() - 1;
  if (total <= 0) return 0.0;
  return 1.0 - (double)free_.size() / total;
}

// ----------------------------------------------------------- SingleTypeKVCacheManager
const std::vector<KVCacheBlock*>& SingleTypeKVCacheManager::blocks_of(
    const std::string& req_id) const {
  static const std::vector<KVCacheBlock*> kEmpty;
  auto it = req_to_blocks_.find(req_id);
  return it == req_to_blocks_.end() ? kEmpty : it->second;
}

int SingleTypeKVCacheManager::get_num_blocks_to_allocate(
    const std::string& req_id, int num_tokens, const std::vector<KVCacheBlock*>& new_computed) {
  int required = cdiv(num_tokens, block_size_);
  int have = (int)blocks_of(req_id).size();
  int num_new = required - (int)new_computed.size() - have;
  // A computed block sitting in the free list (ref_cnt 0) will be taken out of it by touch(),
  // so it costs one free block as well.
  int evictable = 0;
  for (KVCacheBlock* b : new_computed)
    if (b->ref_cnt == 0 && !b->is_null) ++evictable;
  return std::max(num_new, 0) + evictable;
}

void SingleTypeKVCacheManager::save_new_computed_blocks(
    const std::string& req_id, const std::vector<KVCacheBlock*>& new_computed) {
  auto it = req_to_blocks_.find(req_id);
  if (it == req_to_blocks_.end()) {
    auto& v = req_to_blocks_[req_id];
    v = new_computed;
    num_cached_block_[req_id] = (int)new_computed.size();
  } else if (!new_computed.empty()) {
    throw std::runtime_error("a running request cannot receive new computed blocks");
  }
}

std::vector<KVCacheBlock*> SingleTypeKVCacheManager::allocate_new_blocks(
    const std::string& req_id, int num_tokens) {
  auto& v = req_to_blocks_[req_id];
  int required = cdiv(num_tokens, block_size_);
  int n = required - (int)v.size();
  if (n <= 0) return {};
  auto nb = pool_->get_new_blocks(n);
  v.insert(v.end(), nb.begin(), nb.end());
  return nb;
}

void SingleTypeKVCacheManager::cache_blocks(const Request& req, int num_tokens) {
  int& cached = num_cached_block_[req.request_id];
  int full = num_tokens / block_size_;
  if (full <= cached) return;
  pool_->cache_full_blocks(req, req_to_blocks_[req.request_id], cached, full, block_size_,
                           group_id_);
  cached = full;
}

void SingleTypeKVCacheManager::free(const std::string& req_id) {
  auto it = req_to_blocks_.find(req_id);
  if (it != req_to_blocks_.end()) {
    // Free tail blocks first so the prefix survives longest in the LRU order.
    std::vector<KVCacheBlock*> rev(it->second.rbegin(), it->second.rend());
    pool_->free_blocks(rev);
    req_to_blocks_.erase(it);
  }
  num_cached_block_.erase(req_id);
}

int SingleTypeKVCacheManager::get_num_common_prefix_blocks(const std::string& req_id,
                                                           int num_running) const {
  int n = 0;
  for (KVCacheBlock* b : blocks_of(req_id)) {
    if (b->ref_cnt == num_running) ++n;
    else break;
  }
  return n;
}

std::vector<KVCacheBlock*> FullAttentionManager::find_longest_cache_hit(
    const std::vector<BlockHash>& hashes, int max_length) const {
  std::vector<KVCacheBlock*> r;
  int max_blocks = max_length / block_size_;
  for (int i = 0; i < max_blocks && i < (int)hashes.size(); ++i) {
    auto hit = pool_->get_cached_block(hashes[i], {group_id_});
    if (!hit) break;
    r.push_back((*hit)[0]);
  }
  return r;
}

std::vector<KVCacheBlock*> SlidingWindowManager::find_longest_cache_hit(
    const std::vector<BlockHash>& hashes, int max_length) const {
  // A hit of length L needs the last ceil((window-1)/block) blocks before L to be cached
  // contiguously; everything earlier may be the null block. Scan from the right.
  int contiguous_needed = cdiv(std::max(spec_.sliding_window - 1, 0), block_size_);
  int max_blocks = std::min<int>(max_length / block_size_, (int)hashes.size());
  std::vector<KVCacheBlock*> r(max_blocks, pool_->null_block());
  int run = 0;
  bool matched = false;
  for (int i = max_blocks - 1; i >= 0; --i) {
    auto hit = pool_->get_cached_block(hashes[i], {group_id_});
    if (hit) {
      r[i] = (*hit)[0];
      ++run;
      if (run >= contiguous_needed) {
        r.resize(i + run);
        matched = true;
        break;
      }
    } else {
      run = 0;
    }
  }
  if (!matched) {
    // Only a prefix starting at block 0 can still count (the window is not yet full).
    r.resize(run);
  }
  return r;
}

void SlidingWindowManager::remove_skipped_blocks(const std::string& req_id,
                                                 int num_computed_tokens) {
  auto it = req_to_blocks_.find(req_id);
  if (it == req_to_blocks_.end()) return;
  int last_useful_token = num_computed_tokens - spec_.sliding_window + 1;
  int last_useful_block = last_useful_token / block_size_;
  std::vector<KVCacheBlock*> removed;
  auto& blocks = it->second;
  for (int i = std::min(last_useful_block, (int)blocks.size()) - 1; i >= 0; --i) {
    if (blocks[i]->is_null) break;  // everything before is already null
    removed.push_back(blocks[i]);
    blocks[i] = pool_->null_block();
  }
  pool_->free_blocks(removed);
}

std::vector<KVCacheBlock*> ChunkedLocalAttentionManager::find_longest_cache_hit(
    const std::vector<BlockHash>& hashes, int max_length) const {
  // Tokens before the chunk that contains position max_length are never attended: their
  // blocks are represented by the null block; inside the current chunk a plain prefix match.
  int chunk = spec_.attention_chunk_size;
  int local_start_tok = chunk > 0 ? (max_length / chunk) * chunk : 0;
  int local_start_blk = local_start_tok / block_size_;
  int max_blocks = std::min<int>(max_length / block_size_, (int)hashes.size());
  std::vector<KVCacheBlock*> r;
  for (int i = 0; i < std::min(local_start_blk, max_blocks); ++i) r.push_back(pool_->null_block());
  for (int i = local_start_blk; i < max_blocks; ++i) {
    auto hit = pool_->get_cached_block(hashes[i], {group_id_});
    if (!hit) break;
    r.push_back((*hit)[0]);
  }
  return r;
}

void ChunkedLocalAttentionManager::remove_skipped_blocks(const std::string& req_id,
                                                         int num_computed_tokens) {
  auto it = req_to_blocks_.find(req_id);
  if (it == req_to_blocks_.end() || spec_.attention_chunk_size <= 0) return;
  int first_useful_tok = (num_computed_tokens / spec_.attention_chunk_size) * spec_.attention_chunk_size;
  int first_useful_blk = first_useful_tok / block_size_;
  std::vector<KVCacheBlock*> removed;
  auto& blocks = it->second;
  for (int i = std::min(first_useful_blk, (int)blocks.size()) - 1; i >= 0; --i) {
    if (blocks[i]->is_null) break;
    removed.push_back(blocks[i]);
    blocks[i] = pool_->null_block();
  }
  pool_->free_blocks(removed);
}

int MambaManager::get_num_blocks_to_allocate(const std::string& req_id, int,
                                             const std::vector<KVCacheBlock*>&) {
  return blocks_of(req_id).empty() ? 1 : 0;
}
std::vector<KVCacheBlock*> MambaManager::allocate_new_blocks(const std::string& req_id, int) {
  auto& v = req_to_blocks_[req_id];
  if (!v.empty()) return {};
  auto nb = pool_->get_new_blocks(1);
  v = nb;
  return nb;
}

std::unique_ptr<SingleTypeKVCacheManager> make_single_type_manager(const KVCacheSpec& spec,
                                                                   BlockPool* pool, int group_id) {
  switch (spec.kind) {
    case KVSpecKind::kSlidingWindow: return std::make_unique<SlidingWindowManager>(spec, pool, group_id);
    case KVSpecKind::kChunkedLocal: return std::make_unique<ChunkedLocalAttentionManager>(spec, pool, group_id);
    case KVSpecKind::kMamba: return std::make_unique<MambaManager>(spec, pool, group_id);
    default: return std::make_unique<FullAttentionManager>(spec, pool, group_id);
  }
}

// --------------------------------------------------------------------------- coordinator
KVCacheCoordinator::KVCacheCoordinator(const KVCacheConfig& cfg, int max_model_len,
                                       bool enable_caching)
    : cfg_(cfg), max_model_len_(max_model_len), enable_caching_(enable_caching),
      pool_(std::make_unique<BlockPool>(cfg.num_blocks, enable_caching)) {
  for (size_t g = 0; g < cfg.groups.size(); ++g)
    managers_.push_back(make_single_type_manager(cfg.groups[g].spec, pool_.get(), (int)g));
}
int KVCacheCoordinator::get_num_blocks_to_allocate(const std::string& req_id, int num_tokens,
                                                   const BlocksPerGroup& new_computed) {
  int n = 0;
  static const std::vector<KVCacheBlock*> kEmpty;
  for (size_t g = 0; g < managers_.size(); ++g)
    n += managers_[g]->get_num_blocks_to_allocate(
        req_id, num_tokens, g < new_computed.size() ? new_computed[g] : kEmpty);
  return n;
}
void KVCacheCoordinator::save_new_computed_blocks(const std::string& req_id,
                                                  const BlocksPerGroup& new_computed) {
  static const std::vector<KVCacheBlock*> kEmpty;
  for (size_t g = 0; g < managers_.size(); ++g)
    managers_[g]->save_new_computed_blocks(req_id, g < new_computed.size() ? new_computed[g] : kEmpty);
}
BlocksPerGroup KVCacheCoordinator::allocate_new_blocks(const std::string& req_id, int num_tokens) {
  BlocksPerGroup r;
  for (auto& m : managers_) r.push_back(m->allocate_new_blocks(req_id, num_tokens));
  return r;
}
void KVCacheCoordinator::cache_blocks(const Request& req, int num_computed_tokens) {
  for (auto& m : managers_)
    if (m->spec().kind != KVSpecKind::kMamba) m->cache_blocks(req, num_computed_tokens);
}
void KVCacheCoordinator::free(const std::string& req_id) {
  for (auto& m : managers_) m->free(req_id);
}
std::vector<int> KVCacheCoordinator::get_num_common_prefix_blocks(const std::string& req_id,
                                                                  int num_running) const {
  std::vector<int> r;
  for (auto& m : managers_) r.push_back(m->get_num_common_prefix_blocks(req_id, num_running));
  return r;
}
void KVCacheCoordinator::remove_skipped_blocks(const std::string& req_id, int num_computed_tokens) {
  for (auto& m : managers_) m->remove_skipped_blocks(req_id, num_computed_tokens);
}
BlocksPerGroup KVCacheCoordinator::get_blocks(const std::string& req_id) const {
  BlocksPerGroup r;
  for (auto& m : managers_) r.push_back(m->blocks_of(req_id));
  return r;
}

namespace {
class NoPrefixCacheCoordinator : public KVCacheCoordinator {
 public:
  using KVCacheCoordinator::KVCacheCoordinator;
  std::pair<BlocksPerGroup, int> find_longest_cache_hit(const std::vector<BlockHash>&,
                                                        int) const override {
    return {BlocksPerGroup(managers_.size()), 0};
  }
};

class UnitaryCoordinator : public KVCacheCoordinator {
 public:
  using KVCacheCoordinator::KVCacheCoordinator;
  std::pair<BlocksPerGroup, int> find_longest_cache_hit(const std::vector<BlockHash>& hashes,
                                                        int max_len) const override {
    auto hit = managers_[0]->find_longest_cache_hit(hashes, max_len);
    int n = (int)hit.size() * managers_[0]->spec().block_size;
    return {BlocksPerGroup{hit}, n};
  }
};

// Several groups (e.g. full attention + sliding window, or attention + recurrent state):
// shrink the candidate hit length until every cacheable group agrees (fixed point).
// Recurrent-state groups cannot be prefix-cached, so any such group forces a miss.
class HybridCoordinator : public KVCacheCoordinator {
 public:
  using KVCacheCoordinator::KVCacheCoordinator;
  std::pair<BlocksPerGroup, int> find_longest_cache_hit(const std::vector<BlockHash>& hashes,
                                                        int max_len) const override {
    BlocksPerGroup r(managers_.size());
    for (auto& m : managers_)
      if (m->spec().kind == KVSpecKind::kMamba) return {r, 0};
    int len = max_len;
    for (int iter = 0; iter < 64; ++iter) {
      int new_len = len;
      for (size_t g = 0; g < managers_.size(); ++g) {
        r[g] = managers_[g]->find_longest_cache_hit(hashes, new_len);
        new_len = std::min(new_len, (int)r[g].size() * managers_[g]->spec().block_size);
      }
      if (new_len == len) break;
      len = new_len;
      if (len == 0) break;
    }
    for (size_t g = 0; g < managers_.size(); ++g) {
      int keep = len / managers_[g]->spec().block_size;
      if ((int)r[g].size() > keep) r[g].resize(keep);
    }
    return {r, len};
  }
};
}  // namespace

std::unique_ptr<KVCacheCoordinator> make_kv_cache_coordinator(const KVCacheConfig& cfg,
                                                              int max_model_len,
                                                              bool enable_caching) {
  if (!enable_caching) return std::make_unique<NoPrefixCacheCoordinator>(cfg, max_model_len, false);
  if (cfg.groups.size() == 1) return std::make_unique<UnitaryCoordinator>(cfg, max_model_len, true);
  return std::make_unique<HybridCoordinator>(cfg, max_model_len, true);
}

// ------------------------------------------------------------------------------- facade
std::vector<std::vector<int32_t>> KVCacheBlocks::block_ids() const {
  std::vector<std::vector<int32_t>> r;
  for (auto& g : blocks) {
    std::vector<int32_t> ids;
    ids.reserve(g.size());
    for (auto* b : g) ids.push_back(b->block_id);
    r.push_back(std::move(ids));
  }
  return r;
}

KVCacheManager::KVCacheManager(const KVCacheConfig& cfg, int max_model_len, bool enable_caching,
                               bool log_stats)
    : max_model_len_(max_model_len), enable_caching_(enable_caching), log_stats_(log_stats),
      coord_(make_kv_cache_coordinator(cfg, max_model_len, enable_caching)) {
  for (auto& g : cfg.groups)
    if (g.spec.kind != KVSpecKind::kMamba) { block_size_ = g.spec.block_size; break; }
}

KVCacheBlocks KVCacheManager::empty_blocks() const {
  return KVCacheBlocks{BlocksPerGroup(coord_->num_groups())};
}

void update_block_hashes(Request& req, int block_size) {
  int full = req.num_tokens() / block_size;
  while ((int)req.block_hashes.size() < full) {
    size_t i = req.block_hashes.size();
    const std::string& parent = i == 0 ? none_hash() : req.block_hashes.back();
    std::vector<std::string> extra;
    if (i == 0 && req.cache_salt) extra.push_back(*req.cache_salt);
    req.block_hashes.push_back(hash_block_tokens(
        parent, req.all_token_ids.data() + i * block_size, block_size, extra.empty() ? nullptr : &extra));
  }
}

std::pair<KVCacheBlocks, int> KVCacheManager::get_computed_blocks(Request& req) {
  if (!enable_caching_ || req.sampling_params.prompt_logprobs) return {empty_blocks(), 0};
  update_block_hashes(req, block_size_);
  // The last token must always be recomputed so that there are logits to sample from.
  int max_hit = req.num_tokens() - 1;
  auto [blocks, n] = coord_->find_longest_cache_hit(req.block_hashes, max_hit);
  if (log_stats_) {
    stats_.requests += 1;
    stats_.queries += req.num_tokens();
    stats_.hits += n;
  }
  return {KVCacheBlocks{blocks}, n};
}

std::optional<KVCacheBlocks> KVCacheManager::allocate_slots(
    Request& req, int num_new_tokens, int num_new_computed_tokens,
    const KVCacheBlocks* new_computed_blocks, int num_lookahead_tokens, bool delay_cache_blocks) {
  if (num_new_tokens <= 0) throw std::invalid_argument("num_new_tokens must be greater than 0");
  BlocksPerGroup ncb = new_computed_blocks ? new_computed_blocks->blocks
                                           : BlocksPerGroup(coord_->num_groups());
  // Blocks that fell out of every attention window can go back to the pool first.
  coord_->remove_skipped_blocks(req.request_id, req.num_computed_tokens);

  int num_computed = req.num_computed_tokens + num_new_computed_tokens;
  int need_slots = std::min(num_computed + num_new_tokens + num_lookahead_tokens, max_model_len_);
  int to_alloc = coord_->get_num_blocks_to_allocate(req.request_id, need_slots, ncb);
  if (to_alloc > coord_->pool().get_num_free_blocks()) return std::nullopt;

  if (enable_caching_) {
    for (auto& g : ncb) coord_->pool().touch(g);
  }
  coord_->save_new_computed_blocks(req.request_id, ncb);
  BlocksPerGroup nb = coord_->allocate_new_blocks(req.request_id, need_slots);
  if (!enable_caching_ || delay_cache_blocks) return KVCacheBlocks{nb};
  // Speculated tokens may be rejected: only cache up to the tokens that are certain.
  int to_cache = std::min(num_computed + num_new_tokens, req.num_tokens());
  update_block_hashes(req, block_size_);
  coord_->cache_blocks(req, to_cache);
  return KVCacheBlocks{nb};
}

void KVCacheManager::free(const Request& req) { coord_->free(req.request_id); }

bool KVCacheManager::reset_prefix_cache() {
  if (!coord_->pool().reset_prefix_cache()) return false;
  if (log_stats_) stats_.reset = true;
  return true;
}

std::vector<int> KVCacheManager::get_num_common_prefix_blocks(const Request& req,
                                                              int num_running) const {
  return coord_->get_num_common_prefix_blocks(req.request_id, num_running);
}
KVCacheBlocks KVCacheManager::get_blocks(const std::string& req_id) const {
  return KVCacheBlocks{coord_->get_blocks(req_id)};
}
std::vector<std::vector<int32_t>> KVCacheManager::get_block_ids(const std::string& req_id) const {
  return get_blocks(req_id).block_ids();
}
void KVCacheManager::cache_blocks(const Request& req, int num_computed_tokens) {
  if (!enable_caching_) return;
  update_block_hashes(const_cast<Request&>(req), block_size_);
  coord_->cache_blocks(req, num_computed_tokens);
}
PrefixCacheStats KVCacheManager::take_prefix_cache_stats() {
  PrefixCacheStats s = stats_;
  stats_ = PrefixCacheStats{};
  return s;
}

}  // namespace b200
