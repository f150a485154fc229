#include "offload.h"

#include <dirent.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <functional>
#include <stdexcept>

#include "../core/hashing.h"

namespace b200 {
namespace offload {

// ------------------------------------------------------------------------------ LRU
void LruPolicy::insert(const Key& k) {
  erase(k);
  order_.push_back(k);
  pos_[k] = std::prev(order_.end());
}
void LruPolicy::touch(const Key& k) {
  auto it = pos_.find(k);
  if (it == pos_.end()) return;
  order_.splice(order_.end(), order_, it->second);
}
void LruPolicy::erase(const Key& k) {
  auto it = pos_.find(k);
  if (it == pos_.end()) return;
  order_.erase(it->second);
  pos_.erase(it);
}
std::optional<Key> LruPolicy::victim(const std::function<bool(const Key&)>& evictable) {
  for (const Key& k : order_)
    if (evictable(k)) return k;
  return std::nullopt;
}

// ------------------------------------------------------------------------------ ARC
void ArcPolicy::remove_from(const Key& k) {
  auto it = where_.find(k);
  if (it == where_.end()) return;
  L(it->second.list).erase(it->second.it);
  where_.erase(it);
}
void ArcPolicy::push(int list, const Key& k) {
  List& l = L(list);
  l.push_back(k);
  where_[k] = Where{list, std::prev(l.end())};
}
void ArcPolicy::insert(const Key& k) {
  auto it = where_.find(k);
  if (it != where_.end() && it->second.list <= 1) { touch(k); return; }
  if (it != where_.end() && it->second.list == 2) {        // ghost hit in B1: favour recency
    const size_t d = std::max<size_t>(1, b2_.size() / std::max<size_t>(1, b1_.size()));
    p_ = std::min(cap_, p_ + d);
    remove_from(k);
    push(1, k);
    return;
  }
  if (it != where_.end() && it->second.list == 3) {        // ghost hit in B2: favour frequency
    const size_t d = std::max<size_t>(1, b1_.size() / std::max<size_t>(1, b2_.size()));
    p_ = p_ > d ? p_ - d : 0;
    remove_from(k);
    push(1, k);
    return;
  }
  push(0, k);
  // bound the ghost lists
  while (b1_.size() > cap_) { where_.erase(b1_.front()); b1_.pop_front(); }
  while (b2_.size() > cap_) { where_.erase(b2_.front()); b2_.pop_front(); }
}
void ArcPolicy::touch(const Key& k) {
  auto it = where_.find(k);
  if (it == where_.end() || it->second.list > 1) return;
  remove_from(k);
  push(1, k);                                                // seen twice: frequency list
}
void ArcPolicy::erase(const Key& k) { remove_from(k); }
std::optional<Key> ArcPolicy::victim(const std::function<bool(const Key&)>& evictable) {
  // REPLACE: take from T1 when it exceeds its target, else from T2; the victim becomes a ghost.
  auto pick = [&](List& l) -> std::optional<Key> {
    for (const Key& k : l)
      if (evictable(k)) return k;
    return std::nullopt;
  };
  const bool from_t1 = !t1_.empty() && (t1_.size() > p_ || t2_.empty());
  std::optional<Key> v = from_t1 ? pick(t1_) : pick(t2_);
  if (!v) v = from_t1 ? pick(t2_) : pick(t1_);
  if (!v) return v;
  const int src = where_[*v].list;
  remove_from(*v);
  push(src == 0 ? 2 : 3, *v);                                // remember it as a ghost
  return v;
}

std::unique_ptr<CachePolicy> CachePolicy::make(const std::string& name, size_t capacity) {
  if (name == "arc") return std::make_unique<ArcPolicy>(capacity);
  if (name == "lru" || name.empty()) return std::make_unique<LruPolicy>();
  throw std::invalid_argument("unknown cache policy '" + name + "' (lru | arc)");
}

// ------------------------------------------------------------------------------ host tier
CpuTier::CpuTier(int num_slots, const std::string& policy) : policy_(CachePolicy::make(policy, (size_t)num_slots)) {
  for (int i = num_slots - 1; i >= 0; --i) free_.push_back(i);
}
int CpuTier::slot(const Key& k) const {
  auto it = slot_of_.find(k);
  return it == slot_of_.end() ? -1 : it->second;
}
void CpuTier::touch(const Key& k) {
  if (slot_of_.count(k)) policy_->touch(k);
}
void CpuTier::pin(const Key& k, int delta) {
  int& p = pins_[k];
  p += delta;
  if (p <= 0) pins_.erase(k);
}
int CpuTier::reserve(const Key& k, Key* evicted_key, bool* evicted) {
  if (evicted) *evicted = false;
  auto it = slot_of_.find(k);
  if (it != slot_of_.end()) { policy_->touch(k); return it->second; }
  int s;
  if (!free_.empty()) {
    s = free_.back();
    free_.pop_back();
  } else {
    auto v = policy_->victim([&](const Key& c) { return slot_of_.count(c) && !pins_.count(c); });
    if (!v) return -1;
    s = slot_of_[*v];
    slot_of_.erase(*v);
    ++stats.evictions;
    if (evicted_key) *evicted_key = *v;
    if (evicted) *evicted = true;
  }
  slot_of_[k] = s;
  policy_->insert(k);
  ++stats.stores;
  return s;
}
void CpuTier::erase(const Key& k) {
  auto it = slot_of_.find(k);
  if (it == slot_of_.end()) return;
  free_.push_back(it->second);
  slot_of_.erase(it);
  policy_->erase(k);
  pins_.erase(k);
}

// ------------------------------------------------------------------------------ disk tier
static std::string hex(const std::string& bytes) {
  static const char* d = "0123456789abcdef";
  std::string o;
  for (unsigned char c : bytes) { o.push_back(d[c >> 4]); o.push_back(d[c & 15]); }
  return o;
}
static bool unhex(const std::string& h, std::string* out) {
  if (h.size() % 2) return false;
  out->clear();
  auto v = [](char c) { return c >= '0' && c <= '9' ? c - '0' : c >= 'a' && c <= 'f' ? c - 'a' + 10 : -1; };
  for (size_t i = 0; i < h.size(); i += 2) {
    const int a = v(h[i]), b = v(h[i + 1]);
    if (a < 0 || b < 0) return false;
    out->push_back((char)(a * 16 + b));
  }
  return true;
}

std::string CacheIdentity::digest() const {
  const std::string s = model + "|" + std::to_string(block_size) + "|" + std::to_string(block_bytes) + "|" + dtype;
  return hex(sha256(s.data(), s.size()));
}

namespace {
struct FileHeader {
  char magic[8];          // "B2KVBLK1"
  char identity[64];      // hex digest of the cache identity
  uint64_t payload_bytes;
  uint64_t checksum;      // FNV-1a of the payload
};
uint64_t fnv1a(const void* p, size_t n) {
  const unsigned char* b = (const unsigned char*)p;
  uint64_t h = 1469598103934665603ull;
  for (size_t i = 0; i < n; ++i) { h ^= b[i]; h *= 1099511628211ull; }
  return h;
}
}  // namespace

FsTier::FsTier(std::string dir, CacheIdentity id, int64_t max_bytes)
    : dir_(std::move(dir)), id_(std::move(id)), id_digest_(id_.digest()), max_bytes_(max_bytes) {
  ::mkdir(dir_.c_str(), 0755);
  scan();
}
std::string FsTier::path_of(const Key& k) const { return dir_ + "/" + hex(k) + ".kv"; }

void FsTier::scan() {
  DIR* d = ::opendir(dir_.c_str());
  if (!d) return;
  while (dirent* e = ::readdir(d)) {
    const std::string name = e->d_name;
    if (name.size() < 4 || name.substr(name.size() - 3) != ".kv") continue;
    std::string key;
    if (!unhex(name.substr(0, name.size() - 3), &key)) continue;
    struct stat st;
    if (::stat((dir_ + "/" + name).c_str(), &st) != 0) continue;
    index_[key] = ++clock_;
    used_ += st.st_size;
  }
  ::closedir(d);
}
bool FsTier::contains(const Key& k) const { return index_.count(k) > 0; }

bool FsTier::read(const Key& k, void* dst) {
  auto it = index_.find(k);
  if (it == index_.end()) { ++stats.misses; return false; }
  const std::string path = path_of(k);
  FILE* f = std::fopen(path.c_str(), "rb");
  bool ok = false;
  if (f) {
    FileHeader h;
    if (std::fread(&h, sizeof h, 1, f) == 1 && std::memcmp(h.magic, "B2KVBLK1", 8) == 0 &&
        std::memcmp(h.identity, id_digest_.data(), 64) == 0 && (int64_t)h.payload_bytes == id_.block_bytes &&
        std::fread(dst, 1, h.payload_bytes, f) == h.payload_bytes && fnv1a(dst, h.payload_bytes) == h.checksum)
      ok = true;
    std::fclose(f);
  }
  if (!ok) {                    // foreign, truncated or corrupt: never serve it again
    erase(k);
    ++stats.misses;
    return false;
  }
  it->second = ++clock_;
  ++stats.hits;
  return true;
}

bool FsTier::write(const Key& k, const void* src) {
  if (index_.count(k)) { index_[k] = ++clock_; return true; }
  const std::string path = path_of(k), tmp = path + ".tmp";
  FILE* f = std::fopen(tmp.c_str(), "wb");
  if (!f) return false;
  FileHeader h;
  std::memcpy(h.magic, "B2KVBLK1", 8);
  std::memcpy(h.identity, id_digest_.data(), 64);
  h.payload_bytes = (uint64_t)id_.block_bytes;
  h.checksum = fnv1a(src, (size_t)id_.block_bytes);
  const bool ok = std::fwrite(&h, sizeof h, 1, f) == 1 &&
                  std::fwrite(src, 1, (size_t)id_.block_bytes, f) == (size_t)id_.block_bytes;
  std::fclose(f);
  if (!ok || std::rename(tmp.c_str(), path.c_str()) != 0) {   // atomic publish
    ::unlink(tmp.c_str());
    return false;
  }
  index_[k] = ++clock_;
  used_ += (int64_t)sizeof h + id_.block_bytes;
  ++stats.stores;
  enforce_budget();
  return true;
}

void FsTier::erase(const Key& k) {
  auto it = index_.find(k);
  if (it == index_.end()) return;
  ::unlink(path_of(k).c_str());
  used_ -= (int64_t)sizeof(FileHeader) + id_.block_bytes;
  if (used_ < 0) used_ = 0;
  index_.erase(it);
}

void FsTier::enforce_budget() {
  while (max_bytes_ > 0 && used_ > max_bytes_ && index_.size() > 1) {
    auto oldest = std::min_element(index_.begin(), index_.end(),
                                   [](const auto& a, const auto& b) { return a.second < b.second; });
    const Key k = oldest->first;
    erase(k);
    ++stats.evictions;
  }
}

// ------------------------------------------------------------------------------ tiering
TieringManager::TieringManager(int num_cpu_slots, const std::string& policy, uint8_t* host_base,
                               int64_t block_bytes, std::unique_ptr<FsTier> fs)
    : cpu_(num_cpu_slots, policy), host_(host_base), block_bytes_(block_bytes), fs_(std::move(fs)),
      num_slots_(num_cpu_slots), policy_name_(policy) {}

int TieringManager::reserve_for_store(const Key& k) {
  Key victim;
  bool evicted = false;
  // find the victim first so that its bytes can be demoted before the slot is reused
  const int s = cpu_.reserve(k, &victim, &evicted);
  if (s < 0) return -1;
  if (evicted && fs_ && host_) fs_->write(victim, host_ + (int64_t)s * block_bytes_);
  return s;
}

Lookup TieringManager::lookup(const Key& k) {
  if (cpu_.contains(k)) {
    cpu_.touch(k);
    ++cpu_.stats.hits;
    return Lookup::kHit;
  }
  ++cpu_.stats.misses;
  if (fs_ && host_ && fs_->contains(k)) {
    const int s = reserve_for_store(k);
    if (s < 0) return Lookup::kMiss;
    if (!fs_->read(k, host_ + (int64_t)s * block_bytes_)) {
      cpu_.erase(k);
      return Lookup::kMiss;
    }
    return Lookup::kRetry;      // promoted: the next lookup is a host hit
  }
  return Lookup::kMiss;
}

void TieringManager::reset() {
  // host tier first (it may reference nothing on disk), then the disk index stays as is:
  // files are still valid for the same identity
  cpu_ = CpuTier(num_slots_, policy_name_);
}

// ------------------------------------------------------------------------------ connector
OffloadConnector::OffloadConnector(std::shared_ptr<TieringManager> tiers, int block_size)
    : tiers_(std::move(tiers)), block_size_(block_size) {}

std::optional<std::pair<int, bool>> OffloadConnector::get_num_new_matched_tokens(const Request& req,
                                                                                 int num_computed_tokens) {
  std::lock_guard<std::mutex> lock(mu_);
  const int first = num_computed_tokens / block_size_;
  // never cover the whole prompt: the last token must be computed to produce logits
  const int max_blocks = (req.num_tokens() - 1) / block_size_;
  int n = 0;
  bool retry = false;
  for (int b = first; b < max_blocks && b < (int)req.block_hashes.size(); ++b) {
    const Lookup r = tiers_->lookup(req.block_hashes[b]);
    if (r == Lookup::kMiss) break;
    if (r == Lookup::kRetry) retry = true;
    ++n;
  }
  if (retry) return std::nullopt;            // promoted from disk: ask again next step
  return std::make_pair(n * block_size_, false);
}

void OffloadConnector::update_state_after_alloc(const Request& req,
                                                const std::vector<std::vector<int32_t>>& block_ids,
                                                int num_external_tokens) {
  if (num_external_tokens <= 0 || block_ids.empty()) return;
  std::lock_guard<std::mutex> lock(mu_);
  const int n = num_external_tokens / block_size_;
  const std::vector<int32_t>& ids = block_ids[0];
  // the externally cached blocks are the last n of the blocks that precede the new tokens
  const int first = (int)(req.num_computed_tokens / block_size_);
  for (int i = 0; i < n; ++i) {
    const int b = first + i;
    if (b >= (int)ids.size() || b >= (int)req.block_hashes.size()) break;
    const Key& k = req.block_hashes[b];
    const int slot = tiers_->cpu().slot(k);
    if (slot < 0) continue;
    tiers_->cpu().pin(k, +1);
    pending_loads_.push_back(Transfer{0, slot, ids[b], k});
  }
}

std::shared_ptr<void> OffloadConnector::build_connector_meta(const SchedulerOutput&) {
  std::lock_guard<std::mutex> lock(mu_);
  auto m = std::make_shared<ConnectorMeta>();
  m->loads.swap(pending_loads_);
  m->stores.swap(pending_stores_);
  last_ = m;
  return m;
}

std::shared_ptr<ConnectorMeta> OffloadConnector::take_meta() {
  std::lock_guard<std::mutex> lock(mu_);
  auto m = last_;
  last_.reset();
  return m;
}

bool OffloadConnector::request_finished(const Request& req, const std::vector<std::vector<int32_t>>& block_ids) {
  if (block_ids.empty()) return false;
  std::lock_guard<std::mutex> lock(mu_);
  const std::vector<int32_t>& ids = block_ids[0];
  bool any = false;
  for (size_t b = 0; b < req.block_hashes.size() && b < ids.size(); ++b) {
    const Key& k = req.block_hashes[b];
    if (tiers_->cpu().contains(k)) { tiers_->cpu().touch(k); continue; }
    const int slot = tiers_->reserve_for_store(k);
    if (slot < 0) break;
    tiers_->cpu().pin(k, +1);             // not evictable until the copy has happened
    pending_stores_.push_back(Transfer{1, slot, ids[b], k});
    any = true;
  }
  // The copies run at the start of the next step, before any kernel can overwrite a block
  // that was handed out again, so the blocks need not be held back.
  (void)any;
  return false;
}

void OffloadConnector::transfers_done(const ConnectorMeta& meta) {
  std::lock_guard<std::mutex> lock(mu_);
  for (const Transfer& t : meta.loads) tiers_->cpu().pin(t.key, -1);
  for (const Transfer& t : meta.stores) tiers_->cpu().pin(t.key, -1);
}

}  // namespace offload
}  // namespace b200
