// Bindings of the text stack (tokenizer, chat template).
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "rt/chat_template.h"
#include "rt/ds_prompt.h"
#include "rt/json.h"
#include "rt/tokenizer.h"

namespace py = pybind11;
using namespace dgpp;

void bind_text(py::module_& m) {
  py::enum_<SplitPattern>(m, "SplitPattern")
      .value("Gpt2", SplitPattern::Gpt2)
      .value("Cl100k", SplitPattern::Cl100k)
      .value("Qwen2", SplitPattern::Qwen2)
      .value("Whole", SplitPattern::Whole);

  py::class_<Tokenizer>(m, "Tokenizer")
      .def_static("from_json", &Tokenizer::from_json)
      .def_static("from_file", [](const std::string& path) {
        FILE* f = fopen(path.c_str(), "rb");
        if (!f) throw std::runtime_error("cannot open " + path);
        std::string s;
        char buf[1 << 16];
        size_t n;
        while ((n = fread(buf, 1, sizeof(buf), f)) > 0) s.append(buf, n);
        fclose(f);
        return Tokenizer::from_json(s);
      })
      .def_static("byte_level", [](const std::vector<std::pair<py::bytes, py::bytes>>& merges,
                                   const std::vector<std::tuple<std::string, int32_t, bool>>& added, SplitPattern pat) {
        std::vector<std::pair<std::string, std::string>> ms;
        for (const auto& p : merges) ms.emplace_back(std::string(p.first), std::string(p.second));
        std::vector<AddedToken> ad;
        for (const auto& a : added) ad.push_back({std::get<0>(a), std::get<1>(a), std::get<2>(a)});
        return Tokenizer::byte_level(ms, ad, pat);
      }, py::arg("merges"), py::arg("added") = std::vector<std::tuple<std::string, int32_t, bool>>{},
         py::arg("pattern") = SplitPattern::Gpt2)
      .def("encode", &Tokenizer::encode, py::arg("text"), py::arg("allow_special") = true)
      .def("decode", [](const Tokenizer& t, const std::vector<int32_t>& ids, bool skip) {
        return py::bytes(t.decode(ids, skip));
      }, py::arg("ids"), py::arg("skip_special") = false)
      .def("token_bytes", [](const Tokenizer& t, int32_t id) { return py::bytes(t.token_bytes(id)); })
      .def("token_to_id", &Tokenizer::token_to_id)
      .def("vocab_size", &Tokenizer::vocab_size)
      .def("is_special", &Tokenizer::is_special)
      .def("pre_tokenize", &Tokenizer::pre_tokenize)
      .def("fingerprint", &Tokenizer::fingerprint)
      .def_static("normalize_nfc", &Tokenizer::normalize_nfc);

  py::class_<StreamDecoder>(m, "StreamDecoder")
      .def(py::init<const Tokenizer*, bool>(), py::arg("tokenizer"), py::arg("skip_special") = true,
           py::keep_alive<1, 2>())
      .def("push", [](StreamDecoder& d, int32_t id) { return py::bytes(d.push(id)); })
      .def("flush", [](StreamDecoder& d) { return py::bytes(d.flush()); });

  py::class_<ChatTemplate>(m, "ChatTemplate")
      .def(py::init([](const std::string& src, size_t max_out, size_t max_iter, int max_depth) {
        TemplateLimits lim;
        lim.max_output_bytes = max_out;
        lim.max_loop_iterations = max_iter;
        lim.max_depth = max_depth;
        return new ChatTemplate(src, lim);
      }), py::arg("source"), py::arg("max_output_bytes") = size_t(64) << 20, py::arg("max_loop_iterations") = size_t(1) << 22,
          py::arg("max_depth") = 64)
      .def("render_json", [](const ChatTemplate& t, const std::string& context_json) {
        return t.render(json::parse(context_json));
      });

  // prompt renderer for checkpoints without a chat template (DeepSeek-V4 style layout); globals as JSON text
  m.def("deepseek_prompt", [](const std::string& globals_json) { return DeepSeekPrompt::render(json::parse(globals_json)); });
  m.def("json_roundtrip", [](const std::string& s, bool reject_dup) { return json::parse(s, reject_dup).dump(); },
        py::arg("text"), py::arg("reject_duplicates") = false);
}
