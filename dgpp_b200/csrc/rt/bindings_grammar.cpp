// pybind11 surface of the constrained-decoding grammars.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "rt/json_grammar.h"
#include "rt/speculative.h"
#include "rt/tool_grammar.h"
#include "rt/tool_parser.h"

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

  // tools_json: the request's "tools" array ([{"type":"function","function":{"name":..,"parameters":{..}}}, ...])
  py::class_<ToolTokenGrammar>(m, "ToolGrammar")
      .def(py::init([](const std::string& tools_json, bool required, bool parallel, const std::vector<py::bytes>& token_bytes,
                       std::vector<int32_t> eos, const std::string& only) {
        auto specs = std::make_shared<std::vector<ToolSpec>>();
        const json::Value tools = json::parse(tools_json);
        for (const auto& t : tools.items()) {
          const json::Value* fn = t.find("function");
          const json::Value& f = fn ? *fn : t;
          ToolSpec s;
          s.name = f.at("name").as_string();
          if (!only.empty() && s.name != only) continue;
          const json::Value* p = f.find("parameters");
          s.parameters = (p && p->is_object() && p->size() > 0) ? std::make_shared<const Schema>(Schema::compile(*p))
                                                                : std::make_shared<const Schema>(Schema::any_object());
          specs->push_back(std::move(s));
        }
        if (specs->empty()) throw std::invalid_argument("tool grammar: no (matching) tools");
        auto toks = std::make_shared<std::vector<std::string>>();
        toks->reserve(token_bytes.size());
        for (const auto& b : token_bytes) toks->push_back(std::string(b));
        return new ToolTokenGrammar(specs, required ? ToolChoice::Required : ToolChoice::Auto, parallel, toks, std::move(eos));
      }), py::arg("tools_json"), py::arg("required"), py::arg("parallel"), py::arg("token_bytes"), py::arg("eos_ids"),
          py::arg("only") = "")
      .def("words", &ToolTokenGrammar::words)
      .def("complete", &ToolTokenGrammar::complete)
      .def("in_call", &ToolTokenGrammar::in_call)
      .def("calls", &ToolTokenGrammar::calls)
      .def("accept", &ToolTokenGrammar::accept)
      .def("mask", [](ToolTokenGrammar& g) {
        const std::vector<uint32_t>& mk = g.mask();
        py::array_t<uint32_t> out(static_cast<py::ssize_t>(mk.size()));
        std::memcpy(out.mutable_data(), mk.data(), mk.size() * sizeof(uint32_t));
        return out;
      });

  // ---- speculative decoding control
  py::class_<spec::LookupDraft>(m, "LookupDraft")
      .def(py::init<int, int>(), py::arg("min_ngram") = 2, py::arg("max_ngram") = 4)
      .def("reset", &spec::LookupDraft::reset)
      .def("append", &spec::LookupDraft::append)
      .def("push", &spec::LookupDraft::push)
      .def("propose", &spec::LookupDraft::propose)
      .def("size", &spec::LookupDraft::size);
  py::class_<spec::VerifySchedule>(m, "VerifySchedule")
      .def(py::init<int, int, int>(), py::arg("min_draft") = 0, py::arg("max_draft") = 7, py::arg("start") = 3)
      .def("draft_len", &spec::VerifySchedule::draft_len)
      .def("acceptance", &spec::VerifySchedule::acceptance)
      .def("observe", &spec::VerifySchedule::observe)
      .def("steps", &spec::VerifySchedule::steps)
      .def("proposed_total", &spec::VerifySchedule::proposed_total)
      .def("accepted_total", &spec::VerifySchedule::accepted_total);
  py::class_<spec::ConfidenceDepth>(m, "ConfidenceDepth")
      .def(py::init<double, double, double>(), py::arg("base_ms"), py::arg("row_ms"), py::arg("ema") = 0.1)
      .def("lambda_", &spec::ConfidenceDepth::lambda)
      .def("floor", &spec::ConfidenceDepth::floor)
      .def("depth", &spec::ConfidenceDepth::depth, py::arg("conf"), py::arg("accept_scale") = 1.0)
      .def("depth_batch", &spec::ConfidenceDepth::depth_batch, py::arg("conf"), py::arg("accept_scale") = std::vector<double>{})
      .def("observe", &spec::ConfidenceDepth::observe);
  m.def("spec_judge", [](int64_t base, const std::vector<int32_t>& draft, const std::vector<int32_t>& target,
                         const std::vector<int32_t>& stop_ids, int64_t budget) {
    const spec::Verdict v = spec::judge(base, draft, target, stop_ids, budget);
    return py::make_tuple(v.accepted, v.emitted, v.keep_length);
  }, py::arg("base"), py::arg("draft"), py::arg("target"), py::arg("stop_ids") = std::vector<int32_t>{},
     py::arg("budget") = int64_t(-1));

  // ---- streaming tool-call parser
  py::enum_<tools::Format>(m, "ToolFormat").value("JsonTags", tools::Format::JsonTags).value("ArgTags", tools::Format::ArgTags).value("Dsml", tools::Format::Dsml).value("NsXml", tools::Format::NsXml);
  py::class_<tools::ToolParser>(m, "ToolParser")
      .def(py::init<tools::Format, std::string>(), py::arg("format"), py::arg("id_prefix") = "call_")
      .def("calls", &tools::ToolParser::calls)
      .def("set_namespace", &tools::ToolParser::set_namespace)
      .def("set_dsml_spaced", &tools::ToolParser::set_dsml_spaced)
      .def("set_tools", [](tools::ToolParser& p, const std::string& tools_json) { p.set_tools(json::parse(tools_json)); })
      // events: ("content", text) or ("tool_call", index, id, name, arguments_json)
      .def("feed", [](tools::ToolParser& p, const py::bytes& piece) {
        py::list out;
        for (const auto& e : p.feed(std::string(piece))) {
          if (e.is_call) out.append(py::make_tuple("tool_call", e.index, e.id, e.name, e.arguments));
          else out.append(py::make_tuple("content", py::bytes(e.text)));
        }
        return out;
      })
      .def("finish", [](tools::ToolParser& p) {
        py::list out;
        for (const auto& e : p.finish()) out.append(py::make_tuple("content", py::bytes(e.text)));
        return out;
      });
  m.def("render_tools_block", [](const std::string& tools_json) { return tools::render_tools_block(json::parse(tools_json)); });
}
