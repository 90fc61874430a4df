// pybind11 surface of the constrained-decoding grammars.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "rt/json_grammar.h"

namespace py = pybind11;
using namespace dgpp;
using namespace dgpp::grammar;

namespace {

std::shared_ptr<const Schema> make_schema(const std::string& schema_json) {
  if (schema_json.empty()) return std::make_shared<const Schema>(Schema::any_object());
  return std::make_shared<const Schema>(Schema::compile(json::parse(schema_json)));
}

}  // namespace

void bind_grammar(py::module_& m) {
  // (accepted as a prefix, complete value) for a text under a schema ("" = any JSON object)
  m.def("json_machine_check", [](const std::string& schema_json, const py::bytes& text) {
    Machine mc(make_schema(schema_json));
    const bool ok = mc.feed(std::string(text));
    return py::make_tuple(ok, ok && mc.can_finish());
  });
  py::class_<TokenGrammar>(m, "JsonGrammar")
      .def(py::init([](const std::string& schema_json, const std::vector<py::bytes>& token_bytes, std::vector<int32_t> eos) {
        auto toks = std::make_shared<std::vector<std::string>>();
        toks->reserve(token_bytes.size());
        for (const auto& b : token_bytes) toks->push_back(std::string(b));
        return new TokenGrammar(make_schema(schema_json), toks, std::move(eos));
      }), py::arg("schema_json"), py::arg("token_bytes"), py::arg("eos_ids"))
      .def("words", &TokenGrammar::words)
      .def("complete", &TokenGrammar::complete)
      .def("accept", &TokenGrammar::accept)
      // allowed-token bitmask: uint32 words, bit i of word i / 32 = token i (the device sampler's mask layout)
      .def("mask", [](TokenGrammar& g) {
        const std::vector<uint32_t>& mk = g.mask();
        py::array_t<uint32_t> out(static_cast<py::ssize_t>(mk.size()));
        std::memcpy(out.mutable_data(), mk.data(), mk.size() * sizeof(uint32_t));
        return out;
      });
}
