#include "lmcache.h"

#include "../core/hashing.h"

#include <arpa/inet.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <sys/socket.h>
#include <unistd.h>

#include <chrono>
#include <cstdio>
#include <cstring>
#include <stdexcept>
#include <thread>

namespace b200 {
namespace lmcache {

// ====================================================================== BLAKE3
namespace {
constexpr uint32_t kIV[8] = {0x6A09E667u, 0xBB67AE85u, 0x3C6EF372u, 0xA54FF53Au,
                             0x510E527Fu, 0x9B05688Cu, 0x1F83D9ABu, 0x5BE0CD19u};
constexpr int kPerm[16] = {2, 6, 3, 10, 7, 0, 4, 13, 1, 11, 12, 5, 9, 14, 15, 8};
constexpr uint32_t kChunkStart = 1, kChunkEnd = 2, kParent = 4, kRoot = 8;

inline uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }
inline void g(uint32_t* s, int a, int b, int c, int d, uint32_t mx, uint32_t my) {
  s[a] = s[a] + s[b] + mx;
  s[d] = rotr(s[d] ^ s[a], 16);
  s[c] = s[c] + s[d];
  s[b] = rotr(s[b] ^ s[c], 12);
  s[a] = s[a] + s[b] + my;
  s[d] = rotr(s[d] ^ s[a], 8);
  s[c] = s[c] + s[d];
  s[b] = rotr(s[b] ^ s[c], 7);
}
// out[0..7] = new chaining value.
void compress(const uint32_t cv[8], const uint8_t block[64], uint64_t counter, uint32_t block_len,
              uint32_t flags, uint32_t out[8]) {
  uint32_t m[16], s[16];
  for (int i = 0; i < 16; ++i)
    m[i] = (uint32_t)block[4 * i] | ((uint32_t)block[4 * i + 1] << 8) | ((uint32_t)block[4 * i + 2] << 16) |
           ((uint32_t)block[4 * i + 3] << 24);
  for (int i = 0; i < 8; ++i) s[i] = cv[i];
  for (int i = 0; i < 4; ++i) s[8 + i] = kIV[i];
  s[12] = (uint32_t)counter;
  s[13] = (uint32_t)(counter >> 32);
  s[14] = block_len;
  s[15] = flags;
  for (int r = 0; r < 7; ++r) {
    g(s, 0, 4, 8, 12, m[0], m[1]);
    g(s, 1, 5, 9, 13, m[2], m[3]);
    g(s, 2, 6, 10, 14, m[4], m[5]);
    g(s, 3, 7, 11, 15, m[6], m[7]);
    g(s, 0, 5, 10, 15, m[8], m[9]);
    g(s, 1, 6, 11, 12, m[10], m[11]);
    g(s, 2, 7, 8, 13, m[12], m[13]);
    g(s, 3, 4, 9, 14, m[14], m[15]);
    if (r < 6) {
      uint32_t t[16];
      for (int i = 0; i < 16; ++i) t[i] = m[kPerm[i]];
      std::memcpy(m, t, sizeof(m));
    }
  }
  for (int i = 0; i < 8; ++i) out[i] = s[i] ^ s[i + 8];
}
// Chaining value of one chunk (<= 1024 bytes); `root`: it is the whole input.
void chunk_cv(const uint8_t* p, size_t len, uint64_t index, bool root, uint32_t out[8]) {
  uint32_t cv[8];
  std::memcpy(cv, kIV, sizeof(cv));
  const size_t nblocks = len == 0 ? 1 : (len + 63) / 64;
  for (size_t b = 0; b < nblocks; ++b) {
    uint8_t block[64] = {0};
    const size_t n = std::min<size_t>(64, len - b * 64);
    if (len) std::memcpy(block, p + b * 64, n);
    uint32_t flags = 0;
    if (b == 0) flags |= kChunkStart;
    if (b + 1 == nblocks) flags |= kChunkEnd | (root ? kRoot : 0);
    uint32_t next[8];
    compress(cv, block, index, (uint32_t)(len ? n : 0), flags, next);
    std::memcpy(cv, next, sizeof(cv));
  }
  std::memcpy(out, cv, sizeof(cv));
}
void parent_cv(const uint32_t l[8], const uint32_t r[8], bool root, uint32_t out[8]) {
  uint8_t block[64];
  for (int i = 0; i < 8; ++i)
    for (int j = 0; j < 4; ++j) {
      block[4 * i + j] = (uint8_t)(l[i] >> (8 * j));
      block[32 + 4 * i + j] = (uint8_t)(r[i] >> (8 * j));
    }
  compress(kIV, block, 0, 64, kParent | (root ? kRoot : 0), out);
}
}  // namespace

std::string blake3(const void* data, size_t len) {
  const uint8_t* p = static_cast<const uint8_t*>(data);
  const size_t nchunks = len == 0 ? 1 : (len + 1023) / 1024;
  uint32_t cv[8];
  if (nchunks == 1) {
    chunk_cv(p, len, 0, true, cv);
  } else {
    // left-to-right merge: completed subtrees wait on a stack, one entry per set bit of the
    // number of chunks seen so far
    std::vector<std::array<uint32_t, 8>> stack;
    for (size_t c = 0; c + 1 < nchunks; ++c) {
      std::array<uint32_t, 8> cur;
      chunk_cv(p + c * 1024, 1024, c, false, cur.data());
      size_t total = c + 1;
      while ((total & 1) == 0) {
        std::array<uint32_t, 8> merged;
        parent_cv(stack.back().data(), cur.data(), false, merged.data());
        stack.pop_back();
        cur = merged;
        total >>= 1;
      }
      stack.push_back(cur);
    }
    std::array<uint32_t, 8> cur;
    const size_t last = nchunks - 1;
    chunk_cv(p + last * 1024, len - last * 1024, last, false, cur.data());
    while (!stack.empty()) {
      std::array<uint32_t, 8> merged;
      parent_cv(stack.back().data(), cur.data(), stack.size() == 1, merged.data());
      stack.pop_back();
      cur = merged;
    }
    std::memcpy(cv, cur.data(), sizeof(cv));
  }
  std::string out(32, '\0');
  for (int i = 0; i < 8; ++i)
    for (int j = 0; j < 4; ++j) out[4 * i + j] = (char)(uint8_t)(cv[i] >> (8 * j));
  return out;
}

// ====================================================================== token hashing
TokenHasher::TokenHasher(int chunk_size) : chunk_size_(chunk_size) {
  const uint8_t zeros[12] = {0};
  none_hash_ = blake3(zeros, sizeof(zeros));
}

std::string TokenHasher::hash_tokens(const std::vector<uint32_t>& tokens, const std::string& prefix) const {
  std::string buf = prefix;
  buf.reserve(prefix.size() + tokens.size() * 4);
  for (uint32_t t : tokens) {
    buf.push_back((char)(uint8_t)(t >> 24));
    buf.push_back((char)(uint8_t)(t >> 16));
    buf.push_back((char)(uint8_t)(t >> 8));
    buf.push_back((char)(uint8_t)t);
  }
  return blake3(buf.data(), buf.size());
}

std::vector<std::string> TokenHasher::chunk_hashes(const std::vector<uint32_t>& ids) const {
  std::vector<std::string> out;
  std::string prefix = none_hash_;
  for (size_t i = 0; i + chunk_size_ <= ids.size(); i += chunk_size_) {
    std::vector<uint32_t> chunk(ids.begin() + i, ids.begin() + i + chunk_size_);
    prefix = hash_tokens(chunk, prefix);
    out.push_back(prefix);
  }
  return out;
}

std::string TokenHasher::to_hex(const std::string& d) {
  static const char* hex = "0123456789abcdef";
  std::string s;
  for (unsigned char c : d) {
    s.push_back(hex[c >> 4]);
    s.push_back(hex[c & 15]);
  }
  return s;
}

uint64_t TokenHasher::fold(const std::string& d) {
  uint64_t v = 0;
  for (int i = 0; i < 8 && i < (int)d.size(); ++i) v = (v << 8) | (uint8_t)d[i];
  return v;
}

// ====================================================================== peer-agreeing chunk keys
uint64_t vllm_none_hash(const std::string& seed) {
  CborWriter w;
  w.text(seed);
  const std::string& b = w.data();
  return TokenHasher::fold(sha256(b.data(), b.size()));
}

std::vector<ChunkEntry> vllm_chunk_hashes(const std::vector<uint32_t>& ids, int chunk_size, bool save_unfull,
                                          const std::string& seed) {
  std::vector<ChunkEntry> out;
  uint64_t prefix = vllm_none_hash(seed);
  for (size_t i = 0; i < ids.size(); i += chunk_size) {
    const size_t end = std::min(ids.size(), i + (size_t)chunk_size);
    if (end - i < (size_t)chunk_size && !save_unfull) break;
    CborWriter w;
    w.array(3);
    w.uint(prefix);
    w.array(end - i);
    for (size_t j = i; j < end; ++j) w.uint(ids[j]);
    w.array(0);
    const std::string& b = w.data();
    prefix = TokenHasher::fold(sha256(b.data(), b.size()));
    out.push_back(ChunkEntry{(int)i, (int)end, prefix});
  }
  return out;
}

// ====================================================================== dtype / key
std::string dtype_str(Dtype d) {
  switch (d) {
    case Dtype::kFloat16: return "half";
    case Dtype::kBFloat16: return "bfloat16";
    case Dtype::kFloat32: return "float";
    case Dtype::kFloat64: return "double";
    case Dtype::kUint8: return "uint8";
    case Dtype::kFp8E4m3: return "fp8_e4m3fn";
    case Dtype::kFp8E5m2: return "fp8_e5m2";
    default: return "none";
  }
}
Dtype dtype_from_str(const std::string& s) {
  for (Dtype d : {Dtype::kFloat16, Dtype::kBFloat16, Dtype::kFloat32, Dtype::kFloat64, Dtype::kUint8,
                  Dtype::kFp8E4m3, Dtype::kFp8E5m2})
    if (dtype_str(d) == s) return d;
  if (s == "float16") return Dtype::kFloat16;
  if (s == "float32") return Dtype::kFloat32;
  return Dtype::kNone;
}

std::string CacheKey::to_string() const {
  char hex[17];
  std::snprintf(hex, sizeof(hex), "%llx", (unsigned long long)chunk_hash);
  std::string s = model + "@" + std::to_string(world_size) + "@" + std::to_string(worker_id) + "@" + hex + "@" +
                  dtype_str(dtype);
  for (auto& t : tags) s += "@" + t.first + "%" + t.second;
  return s;
}

CacheKey CacheKey::from_string(const std::string& s) {
  std::vector<std::string> parts;
  size_t pos = 0;
  while (true) {
    size_t q = s.find('@', pos);
    parts.push_back(s.substr(pos, q == std::string::npos ? std::string::npos : q - pos));
    if (q == std::string::npos) break;
    pos = q + 1;
  }
  if (parts.size() < 5) throw std::invalid_argument("lmcache key: expected model@world@worker@hash@dtype");
  CacheKey k;
  k.model = parts[0];
  k.world_size = std::stoll(parts[1]);
  k.worker_id = std::stoll(parts[2]);
  k.chunk_hash = std::stoull(parts[3], nullptr, 16);
  k.dtype = dtype_from_str(parts[4]);
  for (size_t i = 5; i < parts.size(); ++i) {
    size_t q = parts[i].find('%');
    if (q == std::string::npos) throw std::invalid_argument("lmcache key: tag without '%'");
    k.tags.emplace_back(parts[i].substr(0, q), parts[i].substr(q + 1));
  }
  return k;
}

// ====================================================================== messages
namespace {
void put_i32(std::string* o, int32_t v) {
  for (int j = 0; j < 4; ++j) o->push_back((char)(uint8_t)((uint32_t)v >> (8 * j)));
}
int32_t get_i32(const std::string& b, size_t off) {
  uint32_t v = 0;
  for (int j = 0; j < 4; ++j) v |= (uint32_t)(uint8_t)b[off + j] << (8 * j);
  return (int32_t)v;
}
std::array<int32_t, 4> pad4(const std::vector<int32_t>& shape) {
  if (shape.size() > 4) throw std::invalid_argument("lmcache: shape has more than 4 dimensions");
  std::array<int32_t, 4> a = {0, 0, 0, 0};
  for (size_t i = 0; i < shape.size(); ++i) a[i] = shape[i];
  return a;
}
std::vector<int32_t> strip(const std::array<int32_t, 4>& d, MemFormat fmt) {
  if (fmt == MemFormat::kBinary || fmt == MemFormat::kBinaryBuffer) return {d[0], d[1], d[2], d[3]};
  int end = 4;
  while (end > 1 && d[end - 1] == 0) --end;
  return std::vector<int32_t>(d.begin(), d.begin() + end);
}
}  // namespace

std::string ClientMeta::serialize() const {
  if ((int)key.size() > kMaxKeyLength) throw std::invalid_argument("lmcache: key longer than 150 bytes");
  const auto d = pad4(shape);
  std::string o;
  put_i32(&o, (int32_t)command);
  put_i32(&o, length);
  put_i32(&o, (int32_t)fmt);
  put_i32(&o, (int32_t)dtype);
  put_i32(&o, (int32_t)location);
  for (int i = 0; i < 4; ++i) put_i32(&o, d[i]);
  o += key;
  o.append(kMaxKeyLength - key.size(), ' ');
  return o;
}

ClientMeta ClientMeta::deserialize(const std::string& b) {
  if (b.size() != 36 + kMaxKeyLength) throw std::invalid_argument("lmcache: client message must be 186 bytes");
  ClientMeta m;
  m.command = (Command)get_i32(b, 0);
  m.length = get_i32(b, 4);
  m.fmt = (MemFormat)get_i32(b, 8);
  m.dtype = (Dtype)get_i32(b, 12);
  m.location = (Location)get_i32(b, 16);
  m.shape = strip({get_i32(b, 20), get_i32(b, 24), get_i32(b, 28), get_i32(b, 32)}, m.fmt);
  std::string k = b.substr(36);
  const size_t a = k.find_first_not_of(" \t\n\r\f\v"), z = k.find_last_not_of(" \t\n\r\f\v");
  m.key = a == std::string::npos ? "" : k.substr(a, z - a + 1);
  return m;
}

std::string ServerMeta::serialize() const {
  const auto d = pad4(shape);
  std::string o;
  put_i32(&o, (int32_t)code);
  put_i32(&o, length);
  put_i32(&o, (int32_t)fmt);
  put_i32(&o, (int32_t)dtype);
  for (int i = 0; i < 4; ++i) put_i32(&o, d[i]);
  put_i32(&o, (int32_t)location);
  return o;
}

ServerMeta ServerMeta::deserialize(const std::string& b) {
  if (b.size() != 36) throw std::invalid_argument("lmcache: server message must be 36 bytes");
  ServerMeta m;
  m.code = (ReturnCode)get_i32(b, 0);
  m.length = get_i32(b, 4);
  m.fmt = (MemFormat)get_i32(b, 8);
  m.dtype = (Dtype)get_i32(b, 12);
  m.shape = strip({get_i32(b, 16), get_i32(b, 20), get_i32(b, 24), get_i32(b, 28)}, m.fmt);
  m.location = (Location)get_i32(b, 32);
  return m;
}

// ====================================================================== KV_2LTD
std::string pack_kv2ltd(int layers, int tokens, int hidden, size_t es, const std::vector<std::string>& k,
                        const std::vector<std::string>& v) {
  const size_t plane = (size_t)tokens * hidden * es;
  if ((int)k.size() != layers || (int)v.size() != layers) throw std::invalid_argument("kv2ltd: one plane per layer");
  std::string o;
  o.reserve(2 * layers * plane);
  for (const auto* side : {&k, &v})
    for (const auto& p : *side) {
      if (p.size() != plane) throw std::invalid_argument("kv2ltd: plane size mismatch");
      o += p;
    }
  return o;
}

void unpack_kv2ltd(int layers, int tokens, int hidden, size_t es, const std::string& packed,
                   std::vector<std::string>* k, std::vector<std::string>* v) {
  const size_t plane = (size_t)tokens * hidden * es;
  if (packed.size() != 2 * (size_t)layers * plane) throw std::invalid_argument("kv2ltd: payload size mismatch");
  k->clear();
  v->clear();
  for (int l = 0; l < layers; ++l) k->push_back(packed.substr((size_t)l * plane, plane));
  for (int l = 0; l < layers; ++l) v->push_back(packed.substr(((size_t)layers + l) * plane, plane));
}

// ====================================================================== client
RemoteClient::RemoteClient(std::string host, int port, int retries)
    : host_(std::move(host)), port_(port), retries_(retries) {}
RemoteClient::~RemoteClient() { close(); }

void RemoteClient::close() {
  if (fd_ >= 0) ::close(fd_);
  fd_ = -1;
}

void RemoteClient::connect() {
  close();
  addrinfo hints{}, *res = nullptr;
  hints.ai_family = AF_UNSPEC;
  hints.ai_socktype = SOCK_STREAM;
  const std::string port = std::to_string(port_);
  if (getaddrinfo(host_.c_str(), port.c_str(), &hints, &res) != 0 || !res)
    throw std::runtime_error("lmcache: cannot resolve " + host_);
  for (int attempt = 0; attempt <= retries_ && fd_ < 0; ++attempt) {
    for (addrinfo* a = res; a && fd_ < 0; a = a->ai_next) {
      int fd = ::socket(a->ai_family, a->ai_socktype, a->ai_protocol);
      if (fd < 0) continue;
      if (::connect(fd, a->ai_addr, a->ai_addrlen) == 0) {
        int one = 1;
        setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
        fd_ = fd;
      } else {
        ::close(fd);
      }
    }
    if (fd_ < 0 && attempt < retries_) std::this_thread::sleep_for(std::chrono::milliseconds(100));
  }
  freeaddrinfo(res);
  if (fd_ < 0) throw std::runtime_error("lmcache: cannot connect to " + host_ + ":" + port);
}

void RemoteClient::send_all(const char* p, size_t n) {
  if (fd_ < 0) throw std::runtime_error("lmcache: not connected");
  while (n) {
    ssize_t w = ::send(fd_, p, n, MSG_NOSIGNAL);
    if (w <= 0) throw std::runtime_error("lmcache: send failed");
    p += w;
    n -= (size_t)w;
  }
}
void RemoteClient::recv_all(char* p, size_t n) {
  if (fd_ < 0) throw std::runtime_error("lmcache: not connected");
  while (n) {
    ssize_t r = ::recv(fd_, p, n, 0);
    if (r == 0) throw std::runtime_error("lmcache: connection closed mid-frame");
    if (r < 0) throw std::runtime_error("lmcache: recv failed");
    p += r;
    n -= (size_t)r;
  }
}

void RemoteClient::put(const std::string& key, const std::string& bytes, MemFormat fmt, Dtype dtype,
                       const std::vector<int32_t>& shape) {
  ClientMeta m;
  m.command = Command::kPut;
  m.key = key;
  m.length = (int32_t)bytes.size();
  m.fmt = fmt;
  m.dtype = dtype;
  m.shape = shape;
  const std::string h = m.serialize();
  send_all(h.data(), h.size());
  send_all(bytes.data(), bytes.size());       // a put has no reply
}

std::optional<RemoteClient::GetResult> RemoteClient::get(const std::string& key) {
  ClientMeta m;
  m.command = Command::kGet;
  m.key = key;
  m.shape = {0};
  const std::string h = m.serialize();
  send_all(h.data(), h.size());
  std::string reply(36, '\0');
  recv_all(reply.data(), reply.size());
  const ServerMeta s = ServerMeta::deserialize(reply);
  if (s.code != ReturnCode::kSuccess) return std::nullopt;   // absent keys are not an error
  GetResult r;
  r.fmt = s.fmt;
  r.dtype = s.dtype;
  r.shape = s.shape;
  r.bytes.resize((size_t)s.length);
  if (s.length > 0) recv_all(r.bytes.data(), r.bytes.size());
  return r;
}

bool RemoteClient::exist(const std::string& key) {
  ClientMeta m;
  m.command = Command::kExist;
  m.key = key;
  m.shape = {0};
  const std::string h = m.serialize();
  send_all(h.data(), h.size());
  std::string reply(36, '\0');
  recv_all(reply.data(), reply.size());
  return ServerMeta::deserialize(reply).code == ReturnCode::kSuccess;
}

bool RemoteClient::health() {
  ClientMeta m;
  m.command = Command::kHealth;
  m.key = "";
  m.shape = {0};
  const std::string h = m.serialize();
  send_all(h.data(), h.size());
  std::string reply(36, '\0');
  recv_all(reply.data(), reply.size());
  return ServerMeta::deserialize(reply).code == ReturnCode::kSuccess;
}

}  // namespace lmcache
}  // namespace b200
