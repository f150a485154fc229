// Python bindings of the tokenizer and the incremental detokenizer.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "tokenizer.h"

namespace py = pybind11;
using namespace b200::tok;

void bind_tokenizer(py::module_& m) {
  py::enum_<PreFamily>(m, "PreFamily")
      .value("NONE", PreFamily::kNone)
      .value("GPT2", PreFamily::kGpt2)
      .value("LLAMA3", PreFamily::kLlama3)
      .value("QWEN2", PreFamily::kQwen2)
      .value("QWEN35", PreFamily::kQwen35)
      .value("DEEPSEEK_V3", PreFamily::kDeepseekV3)
      .value("DEEPSEEK_V2", PreFamily::kDeepseekV2);
  m.def("pretokenize", [](PreFamily f, const std::string& text) {
    std::vector<py::bytes> out;
    for (auto& p : pretokenize(f, text)) out.emplace_back(p);
    return out;
  });
  m.def("family_from_pattern", &family_from_pattern);
  m.def("byte_to_codepoint", [](int b) { return byte_to_codepoint((uint8_t)b); });

  py::class_<Tokenizer, std::shared_ptr<Tokenizer>>(m, "Tokenizer")
      .def_static("from_hf_json", [](const std::string& tj, const std::string& cj) {
        return std::shared_ptr<Tokenizer>(Tokenizer::from_hf_json(tj, cj).release());
      }, py::arg("tokenizer_json"), py::arg("config_json") = "")
      .def_static("from_dir", [](const std::string& d) {
        return std::shared_ptr<Tokenizer>(Tokenizer::from_dir(d).release());
      })
      .def_static("from_gguf", [](const std::string& model, const std::string& pre,
                                  const std::vector<py::bytes>& tokens, const std::vector<py::bytes>& merges,
                                  const std::vector<int>& types, int bos, int eos, bool add_bos, bool add_eos) {
        std::vector<std::string> t(tokens.begin(), tokens.end()), mg(merges.begin(), merges.end());
        return std::shared_ptr<Tokenizer>(
            Tokenizer::from_gguf(model, pre, t, mg, types, bos, eos, add_bos, add_eos).release());
      })
      .def("encode", [](const Tokenizer& t, const std::string& text, bool add_special) {
        py::gil_scoped_release rel;
        return t.encode(text, add_special);
      }, py::arg("text"), py::arg("add_special_tokens") = true)
      .def("encode_ordinary", &Tokenizer::encode_ordinary)
      .def("decode", [](const Tokenizer& t, const std::vector<int>& ids, bool skip) {
        return py::bytes(t.decode(ids, skip)).attr("decode")("utf-8", "replace");
      }, py::arg("ids"), py::arg("skip_special_tokens") = true)
      .def("token_bytes", [](const Tokenizer& t, int id) { return py::bytes(t.token_bytes(id)); })
      .def("id_to_token", [](const Tokenizer& t, int id) { return py::bytes(t.id_to_token(id)); })
      .def("token_to_id", &Tokenizer::token_to_id)
      .def("is_special", &Tokenizer::is_special)
      .def_property_readonly("vocab_size", &Tokenizer::vocab_size)
      .def_property_readonly("bos_id", &Tokenizer::bos_id)
      .def_property_readonly("eos_id", &Tokenizer::eos_id)
      .def_property_readonly("pad_id", &Tokenizer::pad_id)
      .def_property_readonly("unk_id", &Tokenizer::unk_id)
      .def_property_readonly("adds_bos", &Tokenizer::adds_bos)
      .def_property_readonly("byte_level", &Tokenizer::byte_level)
      .def_property_readonly("family", &Tokenizer::family)
      .def_property_readonly("chat_template", &Tokenizer::chat_template)
      .def("pretokenize", [](const Tokenizer& t, const std::string& s) {
        std::vector<py::bytes> out;
        for (auto& p : t.pretokenize_text(s)) out.emplace_back(p);
        return out;
      });

  py::class_<IncrementalDetokenizer>(m, "IncrementalDetokenizer")
      .def(py::init([](std::shared_ptr<Tokenizer> t, const std::vector<int>& prompt, bool skip,
                       std::vector<std::string> stop, bool include_stop, int min_tokens) {
             return new IncrementalDetokenizer(t.get(), prompt, skip, std::move(stop), include_stop, min_tokens);
           }),
           py::arg("tokenizer"), py::arg("prompt_ids"), py::arg("skip_special_tokens") = true,
           py::arg("stop") = std::vector<std::string>{}, py::arg("include_stop_str_in_output") = false,
           py::arg("min_tokens") = 0, py::keep_alive<1, 2>())
      .def("update", [](IncrementalDetokenizer& d, const std::vector<int>& ids, bool stop_terminated) -> py::object {
        std::string s;
        if (d.update(ids, stop_terminated, &s)) return py::str(s);
        return py::none();
      }, py::arg("new_token_ids"), py::arg("stop_terminated") = false)
      .def("get_next_output_text", [](IncrementalDetokenizer& d, bool finished, bool delta) {
        return py::bytes(d.get_next_output_text(finished, delta)).attr("decode")("utf-8", "replace");
      })
      .def_property_readonly("output_text", [](const IncrementalDetokenizer& d) {
        return py::bytes(d.output_text()).attr("decode")("utf-8", "replace");
      })
      .def_property_readonly("token_ids", &IncrementalDetokenizer::token_ids)
      .def_property_readonly("num_output_tokens", &IncrementalDetokenizer::num_output_tokens);
}
