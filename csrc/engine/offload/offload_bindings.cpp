// Python bindings of the KV offload subsystem.
#include <pybind11/functional.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "lmcache.h"
#include "offload.h"

namespace py = pybind11;
using namespace b200;
using namespace b200::offload;

// Lets a KV connector be written in Python: the request is handed over as plain data (id, all
// token ids) so that nothing on the Python side aliases scheduler state.
class PyKVConnector : public KVConnectorHook {
 public:
  std::optional<std::pair<int, bool>> get_num_new_matched_tokens(const Request& req, int num_computed) override {
    py::gil_scoped_acquire gil;
    py::function f = py::get_override(static_cast<const KVConnectorHook*>(this), "get_num_new_matched_tokens");
    if (!f) return std::make_pair(0, false);
    py::object r = f(req.request_id, req.all_token_ids, num_computed);
    if (r.is_none()) return std::nullopt;
    auto t = r.cast<std::pair<int, bool>>();
    return t;
  }
  void update_state_after_alloc(const Request& req, const std::vector<std::vector<int32_t>>& block_ids,
                                int num_external_tokens) override {
    py::gil_scoped_acquire gil;
    py::function f = py::get_override(static_cast<const KVConnectorHook*>(this), "update_state_after_alloc");
    if (f) f(req.request_id, req.all_token_ids, block_ids, num_external_tokens);
  }
  std::shared_ptr<void> build_connector_meta(const SchedulerOutput&) override {
    py::gil_scoped_acquire gil;
    py::function f = py::get_override(static_cast<const KVConnectorHook*>(this), "build_connector_meta");
    if (f) f();
    return nullptr;
  }
  bool request_finished(const Request& req, const std::vector<std::vector<int32_t>>& block_ids) override {
    py::gil_scoped_acquire gil;
    py::function f = py::get_override(static_cast<const KVConnectorHook*>(this), "request_finished");
    if (!f) return false;
    return f(req.request_id, req.all_token_ids, block_ids, req.num_computed_tokens).cast<bool>();
  }
};

void bind_offload(py::module_& m) {
  py::class_<CachePolicy>(m, "CachePolicy")
      .def_static("make", &CachePolicy::make)
      .def("insert", [](CachePolicy& p, py::bytes k) { p.insert(std::string(k)); })
      .def("touch", [](CachePolicy& p, py::bytes k) { p.touch(std::string(k)); })
      .def("erase", [](CachePolicy& p, py::bytes k) { p.erase(std::string(k)); })
      .def("victim", [](CachePolicy& p) -> py::object {
        auto v = p.victim([](const Key&) { return true; });
        if (!v) return py::none();
        return py::bytes(*v);
      })
      .def("__len__", &CachePolicy::size);

  py::class_<TierStats>(m, "TierStats")
      .def_readonly("hits", &TierStats::hits)
      .def_readonly("misses", &TierStats::misses)
      .def_readonly("stores", &TierStats::stores)
      .def_readonly("evictions", &TierStats::evictions);

  py::class_<CacheIdentity>(m, "CacheIdentity")
      .def(py::init([](std::string model, int bs, int64_t bytes, std::string dtype) {
        CacheIdentity id;
        id.model = std::move(model); id.block_size = bs; id.block_bytes = bytes; id.dtype = std::move(dtype);
        return id;
      }))
      .def("digest", &CacheIdentity::digest);

  py::enum_<Lookup>(m, "OffloadLookup")
      .value("MISS", Lookup::kMiss).value("RETRY", Lookup::kRetry).value("HIT", Lookup::kHit);

  py::class_<Transfer>(m, "OffloadTransfer")
      .def_readonly("kind", &Transfer::kind)
      .def_readonly("cpu_slot", &Transfer::cpu_slot)
      .def_readonly("gpu_block", &Transfer::gpu_block)
      .def_property_readonly("key", [](const Transfer& t) { return py::bytes(t.key); });
  py::class_<ConnectorMeta, std::shared_ptr<ConnectorMeta>>(m, "OffloadMeta")
      .def_readonly("loads", &ConnectorMeta::loads)
      .def_readonly("stores", &ConnectorMeta::stores);

  py::class_<TieringManager, std::shared_ptr<TieringManager>>(m, "TieringManager")
      .def(py::init([](int slots, const std::string& policy, uintptr_t host_base, int64_t block_bytes,
                       py::object fs_dir, py::object identity, int64_t fs_max_bytes) {
             std::unique_ptr<FsTier> fs;
             if (!fs_dir.is_none())
               fs = std::make_unique<FsTier>(fs_dir.cast<std::string>(), identity.cast<CacheIdentity>(), fs_max_bytes);
             return std::make_shared<TieringManager>(slots, policy, reinterpret_cast<uint8_t*>(host_base),
                                                     block_bytes, std::move(fs));
           }),
           py::arg("num_cpu_slots"), py::arg("policy") = "lru", py::arg("host_base") = 0,
           py::arg("block_bytes") = 0, py::arg("fs_dir") = py::none(), py::arg("identity") = py::none(),
           py::arg("fs_max_bytes") = 0)
      .def("lookup", [](TieringManager& t, py::bytes k) { return t.lookup(std::string(k)); })
      .def("reserve_for_store", [](TieringManager& t, py::bytes k) { return t.reserve_for_store(std::string(k)); })
      .def("cpu_slot", [](TieringManager& t, py::bytes k) { return t.cpu().slot(std::string(k)); })
      .def("reset", &TieringManager::reset)
      .def_property_readonly("cpu_resident", [](TieringManager& t) { return t.cpu().num_resident(); })
      .def_property_readonly("cpu_stats", [](TieringManager& t) { return t.cpu().stats; })
      .def_property_readonly("fs_blocks", [](TieringManager& t) { return t.fs() ? (int)t.fs()->num_blocks() : 0; })
      .def_property_readonly("fs_bytes", [](TieringManager& t) { return t.fs() ? t.fs()->bytes_used() : 0; })
      .def_property_readonly("fs_stats", [](TieringManager& t) { return t.fs() ? t.fs()->stats : TierStats{}; })
      .def("fs_path", [](TieringManager& t, py::bytes k) { return t.fs() ? t.fs()->path_of(std::string(k)) : std::string(); });

  // ---- LMCache remote client (submodule `lmcache`)
  {
    namespace lm = b200::lmcache;
    py::module_ l = m.def_submodule("lmcache", "client side of an LMCache remote KV server");
    l.def("blake3", [](py::bytes b) { std::string s(b); return py::bytes(lm::blake3(s.data(), s.size())); });
    py::class_<lm::TokenHasher>(l, "TokenHasher")
        .def(py::init<int>(), py::arg("chunk_size") = 256)
        .def_property_readonly("chunk_size", &lm::TokenHasher::chunk_size)
        .def_property_readonly("none_hash", [](const lm::TokenHasher& h) { return py::bytes(h.none_hash()); })
        .def("hash_tokens", [](const lm::TokenHasher& h, const std::vector<uint32_t>& t, py::object prefix) {
          return py::bytes(h.hash_tokens(t, prefix.is_none() ? h.none_hash() : std::string(py::bytes(prefix))));
        }, py::arg("tokens"), py::arg("prefix") = py::none())
        .def("chunk_hashes", [](const lm::TokenHasher& h, const std::vector<uint32_t>& t) {
          py::list out;
          for (auto& d : h.chunk_hashes(t)) out.append(py::bytes(d));
          return out;
        })
        .def_static("fold", [](py::bytes d) { return lm::TokenHasher::fold(std::string(d)); });
    l.def("vllm_none_hash", &lm::vllm_none_hash, py::arg("seed") = "0");
    l.def("vllm_chunk_hashes", [](const std::vector<uint32_t>& t, int chunk, bool keep_tail, const std::string& seed) {
      py::list out;
      for (auto& e : lm::vllm_chunk_hashes(t, chunk, keep_tail, seed)) out.append(py::make_tuple(e.start, e.end, e.chunk_hash));
      return out;
    }, py::arg("token_ids"), py::arg("chunk_size") = 256, py::arg("save_unfull_chunk") = false, py::arg("seed") = "0");
    py::enum_<lm::Command>(l, "Command").value("PUT", lm::Command::kPut).value("GET", lm::Command::kGet)
        .value("EXIST", lm::Command::kExist).value("LIST", lm::Command::kList).value("HEALTH", lm::Command::kHealth);
    py::enum_<lm::ReturnCode>(l, "ReturnCode").value("SUCCESS", lm::ReturnCode::kSuccess).value("FAIL", lm::ReturnCode::kFail);
    py::enum_<lm::Location>(l, "Location").value("NONE", lm::Location::kNone).value("LOCAL_CPU", lm::Location::kLocalCpu)
        .value("LOCAL_DISK", lm::Location::kLocalDisk);
    py::enum_<lm::MemFormat>(l, "MemFormat").value("UNDEFINED", lm::MemFormat::kUndefined)
        .value("KV_2LTD", lm::MemFormat::kKv2ltd).value("KV_T2D", lm::MemFormat::kKvt2d).value("KV_2TD", lm::MemFormat::kKv2td)
        .value("BINARY", lm::MemFormat::kBinary).value("BINARY_BUFFER", lm::MemFormat::kBinaryBuffer)
        .value("KV_MLA_FMT", lm::MemFormat::kKvMla).value("EC_TD", lm::MemFormat::kEctd).value("HS_TD", lm::MemFormat::kHstd);
    py::enum_<lm::Dtype>(l, "Dtype").value("NONE", lm::Dtype::kNone).value("FLOAT16", lm::Dtype::kFloat16)
        .value("BFLOAT16", lm::Dtype::kBFloat16).value("FLOAT32", lm::Dtype::kFloat32).value("FLOAT64", lm::Dtype::kFloat64)
        .value("UINT8", lm::Dtype::kUint8).value("FP8_E4M3", lm::Dtype::kFp8E4m3).value("FP8_E5M2", lm::Dtype::kFp8E5m2);
    l.def("dtype_str", &lm::dtype_str);
    l.def("dtype_from_str", &lm::dtype_from_str);
    py::class_<lm::CacheKey>(l, "CacheKey")
        .def(py::init([](std::string model, int64_t world, int64_t worker, uint64_t hash, lm::Dtype dt,
                         std::vector<std::pair<std::string, std::string>> tags) {
          lm::CacheKey k;
          k.model = std::move(model); k.world_size = world; k.worker_id = worker; k.chunk_hash = hash;
          k.dtype = dt; k.tags = std::move(tags);
          return k;
        }), py::arg("model"), py::arg("world_size") = 1, py::arg("worker_id") = 0, py::arg("chunk_hash") = 0,
             py::arg("dtype") = lm::Dtype::kBFloat16, py::arg("tags") = std::vector<std::pair<std::string, std::string>>{})
        .def_readwrite("model", &lm::CacheKey::model)
        .def_readwrite("world_size", &lm::CacheKey::world_size)
        .def_readwrite("worker_id", &lm::CacheKey::worker_id)
        .def_readwrite("chunk_hash", &lm::CacheKey::chunk_hash)
        .def_readwrite("dtype", &lm::CacheKey::dtype)
        .def_readwrite("tags", &lm::CacheKey::tags)
        .def("to_string", &lm::CacheKey::to_string)
        .def_static("from_string", &lm::CacheKey::from_string);
    py::class_<lm::ClientMeta>(l, "ClientMeta")
        .def(py::init<>())
        .def_readwrite("command", &lm::ClientMeta::command)
        .def_readwrite("key", &lm::ClientMeta::key)
        .def_readwrite("length", &lm::ClientMeta::length)
        .def_readwrite("fmt", &lm::ClientMeta::fmt)
        .def_readwrite("dtype", &lm::ClientMeta::dtype)
        .def_readwrite("shape", &lm::ClientMeta::shape)
        .def_readwrite("location", &lm::ClientMeta::location)
        .def("serialize", [](const lm::ClientMeta& c) { return py::bytes(c.serialize()); })
        .def_static("deserialize", [](py::bytes b) { return lm::ClientMeta::deserialize(std::string(b)); });
    py::class_<lm::ServerMeta>(l, "ServerMeta")
        .def(py::init<>())
        .def_readwrite("code", &lm::ServerMeta::code)
        .def_readwrite("length", &lm::ServerMeta::length)
        .def_readwrite("fmt", &lm::ServerMeta::fmt)
        .def_readwrite("dtype", &lm::ServerMeta::dtype)
        .def_readwrite("shape", &lm::ServerMeta::shape)
        .def_readwrite("location", &lm::ServerMeta::location)
        .def("serialize", [](const lm::ServerMeta& c) { return py::bytes(c.serialize()); })
        .def_static("deserialize", [](py::bytes b) { return lm::ServerMeta::deserialize(std::string(b)); });
    l.def("pack_kv2ltd", [](int L, int T, int D, size_t es, const std::vector<py::bytes>& k, const std::vector<py::bytes>& v) {
      std::vector<std::string> ks(k.begin(), k.end()), vs(v.begin(), v.end());
      return py::bytes(lm::pack_kv2ltd(L, T, D, es, ks, vs));
    });
    l.def("unpack_kv2ltd", [](int L, int T, int D, size_t es, py::bytes packed) {
      std::vector<std::string> k, v;
      lm::unpack_kv2ltd(L, T, D, es, std::string(packed), &k, &v);
      py::list pk, pv;
      for (auto& x : k) pk.append(py::bytes(x));
      for (auto& x : v) pv.append(py::bytes(x));
      return py::make_tuple(pk, pv);
    });
    py::class_<lm::RemoteClient>(l, "RemoteClient")
        .def(py::init<std::string, int, int>(), py::arg("host") = "127.0.0.1", py::arg("port") = 65432,
             py::arg("connect_retries") = 20)
        .def("connect", &lm::RemoteClient::connect, py::call_guard<py::gil_scoped_release>())
        .def("close", &lm::RemoteClient::close)
        .def_property_readonly("connected", &lm::RemoteClient::connected)
        .def("put", [](lm::RemoteClient& c, const std::string& key, py::bytes data, lm::MemFormat fmt, lm::Dtype dt,
                       const std::vector<int32_t>& shape) {
          std::string s(data);
          py::gil_scoped_release rel;
          c.put(key, s, fmt, dt, shape);
        })
        .def("get", [](lm::RemoteClient& c, const std::string& key) -> py::object {
          std::optional<lm::RemoteClient::GetResult> r;
          {
            py::gil_scoped_release rel;
            r = c.get(key);
          }
          if (!r) return py::none();
          return py::make_tuple(py::bytes(r->bytes), r->fmt, r->dtype, r->shape);
        })
        .def("exist", &lm::RemoteClient::exist, py::call_guard<py::gil_scoped_release>())
        .def("health", &lm::RemoteClient::health, py::call_guard<py::gil_scoped_release>());
  }

  py::class_<KVConnectorHook, PyKVConnector>(m, "KVConnectorHook").def(py::init<>());
  py::class_<OffloadConnector, KVConnectorHook>(m, "OffloadConnector")
      .def(py::init<std::shared_ptr<TieringManager>, int>(), py::arg("tiers"), py::arg("block_size"))
      .def("take_meta", &OffloadConnector::take_meta)
      .def("transfers_done", &OffloadConnector::transfers_done);
}
