// Python bindings of the KV offload subsystem.
#include <pybind11/functional.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "offload.h"

namespace py = pybind11;
using namespace b200;
using namespace b200::offload;

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

  py::class_<KVConnectorHook>(m, "KVConnectorHook");
  py::class_<OffloadConnector, KVConnectorHook>(m, "OffloadConnector")
      .def(py::init<std::shared_ptr<TieringManager>, int>(), py::arg("tiers"), py::arg("block_size"))
      .def("take_meta", &OffloadConnector::take_meta)
      .def("transfers_done", &OffloadConnector::transfers_done);
}
