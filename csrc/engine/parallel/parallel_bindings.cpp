// Python binding of the expert-placement policy (eplb.h).
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "eplb.h"

namespace py = pybind11;
using namespace b200;

namespace {
py::array_t<int32_t> as_array(const std::vector<int32_t>& v, std::vector<ssize_t> shape) {
  py::array_t<int32_t> a(shape);
  std::copy(v.begin(), v.end(), a.mutable_data());
  return a;
}
}  // namespace

void bind_parallel(py::module_& m) {
  m.def(
      "eplb_rebalance",
      [](py::array_t<double, py::array::c_style | py::array::forcecast> loads, int num_physical, int num_groups,
         int num_nodes, int num_ranks) {
        if (loads.ndim() != 2) throw std::invalid_argument("eplb: loads must be [layers][experts]");
        const int L = (int)loads.shape(0), E = (int)loads.shape(1);
        std::vector<double> w(loads.data(), loads.data() + (size_t)L * E);
        EplbPlacement p = eplb_rebalance(w, L, E, num_physical, num_groups, num_nodes, num_ranks);
        py::dict d;
        d["phy2log"] = as_array(p.phy2log, {L, num_physical});
        d["phy_rank"] = as_array(p.phy_rank, {L, num_physical});
        d["log2phy"] = as_array(p.log2phy, {L, E, p.max_replicas});
        d["logcnt"] = as_array(p.logcnt, {L, E});
        return d;
      },
      py::arg("loads"), py::arg("num_physical"), py::arg("num_groups") = 1, py::arg("num_nodes") = 1,
      py::arg("num_ranks") = 1,
      "Expert placement from a window of per-layer expert loads: {phy2log, phy_rank, log2phy, logcnt}.");
}
