// Client side of an LMCache remote KV server (`lm://host:port`): the rolling BLAKE3 chunk hash
// LMCache keys KV chunks on, the cache-engine key string, the KV_2LTD memory format, the fixed
// size wire messages and a blocking TCP client. Everything here has to agree byte for byte with
// an LMCache server, which is what the tests pin with vectors produced by LMCache itself.
//
// Reference: include/vllm/v1/kv_offload/lmcache/{token_hasher,cache_engine_key,memory_format,
// remote_protocol,remote_client}.h.
#pragma once
#include <array>
#include <cstdint>
#include <optional>
#include <string>
#include <utility>
#include <vector>

namespace b200 {
namespace lmcache {

// ------------------------------------------------------------------ BLAKE3 (portable, hash mode)
std::string blake3(const void* data, size_t len);          // 32-byte digest

// ------------------------------------------------------------------ token hashing
// digest = blake3(prefix || tokens as big-endian uint32); prefix = previous chunk's digest, or
// none_hash = blake3(8 zero bytes || one zero token) for the first chunk.
class TokenHasher {
 public:
  explicit TokenHasher(int chunk_size = 256);
  int chunk_size() const { return chunk_size_; }
  const std::string& none_hash() const { return none_hash_; }
  std::string hash_tokens(const std::vector<uint32_t>& tokens, const std::string& prefix) const;
  // One digest per COMPLETE chunk of token_ids (a trailing partial chunk is dropped).
  std::vector<std::string> chunk_hashes(const std::vector<uint32_t>& token_ids) const;
  static std::string to_hex(const std::string& digest);
  static uint64_t fold(const std::string& digest);          // big-endian first 8 bytes

 private:
  int chunk_size_;
  std::string none_hash_;
};

// ------------------------------------------------------------------ peer-agreeing chunk keys
// The chunk hash a vLLM + LMCache peer keys on (LMCache's ChunkedTokenDatabase with vLLM's
// sha256_cbor hash): prefix = fold8(sha256(cbor(str(seed)))); per chunk
// prefix = fold8(sha256(cbor([prefix, [tokens...], []]))), fold8 = first 8 bytes big-endian.
struct ChunkEntry {
  int start = 0, end = 0;
  uint64_t chunk_hash = 0;
};
uint64_t vllm_none_hash(const std::string& seed = "0");
std::vector<ChunkEntry> vllm_chunk_hashes(const std::vector<uint32_t>& token_ids, int chunk_size = 256,
                                          bool save_unfull_chunk = false, const std::string& seed = "0");

// ------------------------------------------------------------------ wire enums
enum class Command : int32_t { kPut = 1, kGet = 2, kExist = 3, kList = 4, kHealth = 5 };
enum class ReturnCode : int32_t { kSuccess = 200, kFail = 400 };
enum class Location : int32_t { kNone = 0, kLocalCpu = 1, kLocalDisk = 2 };
enum class MemFormat : int32_t { kUndefined = 0, kKv2ltd = 1, kKvt2d = 2, kKv2td = 3, kBinary = 4,
                                 kBinaryBuffer = 5, kKvMla = 6, kEctd = 7, kHstd = 8 };
enum class Dtype : int32_t { kNone = 0, kFloat16 = 2, kBFloat16 = 3, kFloat32 = 4, kFloat64 = 5, kUint8 = 6,
                             kFp8E4m3 = 7, kFp8E5m2 = 8 };
std::string dtype_str(Dtype d);           // "half", "bfloat16", "float", "double", "uint8", ...
Dtype dtype_from_str(const std::string& s);

// ------------------------------------------------------------------ cache key
struct CacheKey {
  std::string model;
  int64_t world_size = 1, worker_id = 0;
  uint64_t chunk_hash = 0;
  Dtype dtype = Dtype::kNone;
  std::vector<std::pair<std::string, std::string>> tags;
  std::string to_string() const;            // model@world@worker@hex(chunk_hash)@dtype[@tag%value...]
  static CacheKey from_string(const std::string& s);
};

// ------------------------------------------------------------------ messages
constexpr int kMaxKeyLength = 150;
struct ClientMeta {                          // 9 little-endian int32 + 150-byte space-padded key = 186 bytes
  Command command = Command::kGet;
  std::string key;
  int32_t length = 0;
  MemFormat fmt = MemFormat::kUndefined;
  Dtype dtype = Dtype::kNone;
  std::vector<int32_t> shape;
  Location location = Location::kNone;
  std::string serialize() const;
  static ClientMeta deserialize(const std::string& bytes);
};
struct ServerMeta {                          // 9 little-endian int32 = 36 bytes (location last)
  ReturnCode code = ReturnCode::kSuccess;
  int32_t length = 0;
  MemFormat fmt = MemFormat::kUndefined;
  Dtype dtype = Dtype::kNone;
  std::vector<int32_t> shape;
  Location location = Location::kNone;
  std::string serialize() const;
  static ServerMeta deserialize(const std::string& bytes);
};

// ------------------------------------------------------------------ KV_2LTD: [2, layers, tokens, hidden]
// k_planes / v_planes: one [tokens, hidden] byte string per layer.
std::string pack_kv2ltd(int layers, int tokens, int hidden, size_t elem_size,
                        const std::vector<std::string>& k_planes, const std::vector<std::string>& v_planes);
void unpack_kv2ltd(int layers, int tokens, int hidden, size_t elem_size, const std::string& packed,
                   std::vector<std::string>* k_planes, std::vector<std::string>* v_planes);

// ------------------------------------------------------------------ blocking TCP client
class RemoteClient {
 public:
  RemoteClient(std::string host, int port, int connect_retries = 20);
  ~RemoteClient();
  RemoteClient(const RemoteClient&) = delete;
  RemoteClient& operator=(const RemoteClient&) = delete;
  void connect();
  void close();
  bool connected() const { return fd_ >= 0; }
  struct GetResult {
    std::string bytes;
    MemFormat fmt = MemFormat::kUndefined;
    Dtype dtype = Dtype::kNone;
    std::vector<int32_t> shape;
  };
  void put(const std::string& key, const std::string& bytes, MemFormat fmt, Dtype dtype,
           const std::vector<int32_t>& shape);
  std::optional<GetResult> get(const std::string& key);     // nullopt: the server does not have it
  bool exist(const std::string& key);
  bool health();

 private:
  void send_all(const char* p, size_t n);
  void recv_all(char* p, size_t n);
  std::string host_;
  int port_, retries_, fd_ = -1;
};

}  // namespace lmcache
}  // namespace b200
