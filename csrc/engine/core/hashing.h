// SHA-256 and the canonical-CBOR block hash used for prefix caching.
//
// hash(block) = SHA256(CBOR([parent_hash_bytes, [token ids...], extra_keys | null]))
// which is byte-identical to vLLM's `sha256_cbor` block hash, so cache keys agree with
// external KV stores that speak that format. Reference behaviour:
// src/vllm/v1/core/kv_cache_utils.cpp:393-425.
#pragma once
#include <array>
#include <cstdint>
#include <optional>
#include <string>
#include <vector>

namespace b200 {

std::string sha256(const void* data, size_t len);          // 32 raw bytes
std::string sha256_hex(const void* data, size_t len);
std::string to_hex(const std::string& raw);

// Minimal canonical CBOR writer (definite lengths, shortest-form integers).
class CborWriter {
 public:
  void uint(uint64_t v) { head(0, v); }
  void int_(int64_t v) { v >= 0 ? head(0, (uint64_t)v) : head(1, (uint64_t)(-1 - v)); }
  void bytes(const std::string& b) { head(2, b.size()); buf_.append(b); }
  void text(const std::string& s) { head(3, s.size()); buf_.append(s); }
  void array(uint64_t n) { head(4, n); }
  void null() { buf_.push_back((char)0xf6); }
  const std::string& data() const { return buf_; }

 private:
  void head(int major, uint64_t v);
  std::string buf_;
};

// The seed hash of the first block of every request ("NONE_HASH"). Derived once per process
// from the environment variable PYTHONHASHSEED (vLLM's rule) or the fixed seed "0".
const std::string& none_hash();
void reset_none_hash_for_test(const std::string& seed);

std::string hash_block_tokens(const std::string& parent_hash, const int32_t* tokens, size_t n,
                              const std::vector<std::string>* extra_keys);

// Hash plus KV-cache-group id: hash || 4-byte big-endian group id.
inline std::string hash_with_group(const std::string& h, uint32_t group) {
  std::string r = h;
  r.push_back((char)(group >> 24));
  r.push_back((char)(group >> 16));
  r.push_back((char)(group >> 8));
  r.push_back((char)group);
  return r;
}

}  // namespace b200
