// Python bindings of the structured-output engine.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "../util/json.h"
#include "manager.h"

namespace py = pybind11;
using namespace b200;
using namespace b200::so;

void bind_structured(py::module_& m) {
  py::class_<Grammar, std::shared_ptr<Grammar>>(m, "Grammar")
      .def_static("from_gbnf", &Grammar::from_gbnf, py::arg("text"), py::arg("root") = "root")
      .def_static("from_json_schema", &Grammar::from_json_schema_text)
      .def_static("from_regex", &Grammar::from_regex)
      .def_static("from_choices", &Grammar::from_choices)
      .def_static("any_json_object", &Grammar::any_json_object)
      .def("to_gbnf", &Grammar::to_gbnf)
      .def_property_readonly("num_rules", [](const Grammar& g) { return g.rules().size(); });
  m.def("json_schema_to_gbnf", [](const std::string& s) { return json_schema_to_gbnf(Json::parse(s)); });
  m.def("regex_to_gbnf", &regex_to_gbnf);

  py::class_<Matcher>(m, "GrammarMatcher")
      .def(py::init([](std::shared_ptr<Grammar> g) { return new Matcher(g); }))
      .def("accept_bytes", [](Matcher& mt, py::bytes b) { return mt.accept_bytes(std::string(b)); })
      .def("accept_string", [](Matcher& mt, const std::string& s) { return mt.accept_bytes(s); })
      .def("can_terminate", &Matcher::can_terminate)
      .def("is_dead", &Matcher::is_dead)
      .def("push_checkpoint", &Matcher::push_checkpoint)
      .def("rollback", &Matcher::rollback)
      .def("reset", &Matcher::reset);

  py::class_<RequestGrammar>(m, "RequestGrammar")
      .def_readonly("invalid", &RequestGrammar::invalid)
      .def_readonly("error", &RequestGrammar::error)
      .def_readonly("terminated", &RequestGrammar::terminated)
      .def_readonly("lazy", &RequestGrammar::lazy)
      .def_property_readonly("constrained", [](const RequestGrammar& s) { return s.matcher != nullptr; });

  py::class_<StructuredOutputHook>(m, "StructuredOutputHook");
  py::class_<StructuredOutputManager, StructuredOutputHook>(m, "StructuredOutputManager")
      .def(py::init([](const std::vector<py::bytes>& tokens, int vocab, std::vector<int> eos) {
             std::vector<std::string> t(tokens.begin(), tokens.end());
             return new StructuredOutputManager(std::move(t), vocab, std::move(eos));
           }),
           py::arg("token_bytes"), py::arg("vocab_size"), py::arg("eos_ids"))
      .def("validate", [](StructuredOutputManager& mg, const StructuredOutputsParams& p) {
        auto st = mg.make_state(p);
        if (st->invalid) throw std::invalid_argument(st->error);
      })
      .def("make_state", [](StructuredOutputManager& mg, const StructuredOutputsParams& p) {
        return mg.make_state(p);
      })
      .def("accept", &StructuredOutputManager::accept)
      .def("mask_for", [](StructuredOutputManager& mg, RequestGrammar& st) {
        py::gil_scoped_release rel;
        return mg.mask_for(st);
      })
      .def("allowed_tokens", [](StructuredOutputManager& mg, RequestGrammar& st) {
        std::vector<uint32_t> row = mg.mask_for(st);
        std::vector<int> ids;
        for (size_t w = 0; w < row.size(); ++w)
          for (int b = 0; b < 32; ++b)
            if (row[w] >> b & 1u) ids.push_back((int)w * 32 + b);
        return ids;
      })
      .def_property_readonly("words_per_row", &StructuredOutputManager::words_per_row);
}
