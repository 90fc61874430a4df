// Bindings of the sampler oracle, the OpenAI request/response layer and the HTTP server.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "rt/http_server.h"
#include "rt/openai.h"
#include "rt/sampler.h"

namespace py = pybind11;
using namespace dgpp;

namespace {

py::dict request_to_dict(const openai::Request& r) {
  py::dict d;
  d["chat"] = r.chat;
  d["model"] = r.model;
  d["messages_json"] = r.messages.is_null() ? std::string("null") : r.messages.dump();
  d["prompt_text"] = r.prompt_text;
  d["prompt_ids"] = r.prompt_ids;
  d["stream"] = r.stream;
  d["include_usage"] = r.include_usage;
  d["max_tokens"] = r.max_tokens;
  d["n"] = r.n;
  d["temperature"] = r.temperature;
  d["top_p"] = r.top_p;
  d["min_p"] = r.min_p;
  d["top_k"] = r.top_k;
  d["presence_penalty"] = r.presence_penalty;
  d["frequency_penalty"] = r.frequency_penalty;
  d["repetition_penalty"] = r.repetition_penalty;
  d["seed"] = r.has_seed ? py::object(py::int_(r.seed)) : py::object(py::none());
  d["stop"] = r.stop;
  d["logprobs"] = r.logprobs;
  d["top_logprobs"] = r.top_logprobs;
  d["logit_bias"] = r.logit_bias;
  d["tools_json"] = r.tools.is_null() ? std::string("null") : r.tools.dump();
  d["tool_choice_json"] = r.tool_choice.is_null() ? std::string("null") : r.tool_choice.dump();
  d["response_format_json"] = r.response_format.is_null() ? std::string("null") : r.response_format.dump();
  d["chat_template_kwargs_json"] = r.chat_template_kwargs.is_null() ? std::string("null") : r.chat_template_kwargs.dump();
  d["parallel_tool_calls"] = r.parallel_tool_calls;
  d["ignore_eos"] = r.ignore_eos;
  d["prefix_cache"] = r.prefix_cache;
  d["prompt_cache_key"] = r.prompt_cache_key;
  d["reasoning_effort"] = r.reasoning_effort;
  d["sse_ping_interval"] = r.sse_ping_interval;
  return d;
}

struct ApiErrorPy : std::runtime_error {
  int status;
  std::string body;
  ApiErrorPy(int s, const std::string& b) : std::runtime_error(b), status(s), body(b) {}
};

openai::Choice make_choice(int index, const std::string& text, const std::string& finish, const std::string& tool_calls_json,
                           const std::vector<std::tuple<std::string, double, std::vector<std::pair<std::string, double>>>>& lps,
                           bool has_lp, const std::string& reasoning) {
  openai::Choice c;
  c.index = index;
  c.text = text;
  c.finish_reason = finish;
  c.reasoning = reasoning;
  if (!tool_calls_json.empty() && tool_calls_json != "null") c.tool_calls = json::parse(tool_calls_json);
  c.has_logprobs = has_lp;
  for (const auto& t : lps) c.logprobs.push_back({std::get<0>(t), std::get<1>(t), std::get<2>(t)});
  return c;
}

}  // namespace

void bind_serve(py::module_& m) {
  // ---------------- sampler oracle
  m.def("det_exp", [](float x) { return det::exp(x); });
  m.def("det_log", [](float x) { return det::log(x); });
  m.def("uniform01", [](uint64_t seed, uint64_t counter) { return det::uniform01(seed, counter); });
  m.def("slice_logsumexp", [](const std::vector<float>& x) { return sample::slice_logsumexp(x.data(), static_cast<int64_t>(x.size())); });
  m.def("slice_max_sum", [](const std::vector<float>& x) { return sample::slice_max_sum(x.data(), static_cast<int64_t>(x.size())); });
  m.def("merge_logsumexp", &sample::merge_logsumexp);
  m.def("judge_verify", &sample::judge_verify);
  m.def("spec_accept_ratio", &sample::spec_accept_ratio);
  m.def("sample_reference",
        [](const std::vector<float>& logits, float temperature, int top_k, float top_p, float min_p, float rep, float pres,
           float freq, uint64_t seed, int top_logprobs, const std::map<int32_t, float>& bias,
           const std::map<int32_t, int>& counts, uint64_t position, py::object allowed, int candidates,
           bool return_width) -> py::object {
          sample::Params p;
          p.temperature = temperature; p.top_k = top_k; p.top_p = top_p; p.min_p = min_p;
          p.repetition_penalty = rep; p.presence_penalty = pres; p.frequency_penalty = freq;
          p.seed = seed; p.top_logprobs = top_logprobs; p.logit_bias = bias;
          std::vector<uint8_t> mask;
          const std::vector<uint8_t>* mp = nullptr;
          if (!allowed.is_none()) { mask = allowed.cast<std::vector<uint8_t>>(); mp = &mask; }
          const sample::Result r = sample::sample(logits, p, counts, position, mp, candidates);
          if (return_width) return py::make_tuple(r.token, r.logprob, r.top, r.candidates_used);
          return py::make_tuple(r.token, r.logprob, r.top);
        },
        py::arg("logits"), py::arg("temperature") = 0.f, py::arg("top_k") = 0, py::arg("top_p") = 1.f,
        py::arg("min_p") = 0.f, py::arg("repetition_penalty") = 1.f, py::arg("presence_penalty") = 0.f,
        py::arg("frequency_penalty") = 0.f, py::arg("seed") = 0, py::arg("top_logprobs") = 0,
        py::arg("logit_bias") = std::map<int32_t, float>{}, py::arg("counts") = std::map<int32_t, int>{},
        py::arg("position") = 0, py::arg("allowed") = py::none(), py::arg("candidates") = 128,
        py::arg("return_width") = false);

  // ---------------- OpenAI layer
  static py::exception<ApiErrorPy> api_error(m, "ApiError");
  py::register_exception_translator([](std::exception_ptr p) {
    try {
      if (p) std::rethrow_exception(p);
    } catch (const openai::ApiError& e) {
      PyErr_SetObject(api_error.ptr(), py::make_tuple(e.status, e.to_json()).ptr());
    }
  });
  m.def("parse_chat_request", [](const std::string& body) { return request_to_dict(openai::parse_chat_request(body)); });
  m.def("parse_completion_request",
        [](const std::string& body) { return request_to_dict(openai::parse_completion_request(body)); });
  m.def("completion_json",
        [](bool chat, const std::string& id, const std::string& model, int64_t created, const std::vector<py::tuple>& choices,
           int64_t prompt_tokens, int64_t completion_tokens, int64_t cached_tokens) {
          std::vector<openai::Choice> cs;
          for (const py::tuple& t : choices) {
            using LP = std::vector<std::tuple<std::string, double, std::vector<std::pair<std::string, double>>>>;
            cs.push_back(make_choice(t[0].cast<int>(), t[1].cast<std::string>(), t[2].cast<std::string>(),
                                     t.size() > 3 ? t[3].cast<std::string>() : std::string(),
                                     t.size() > 4 ? t[4].cast<LP>() : LP(), t.size() > 5 ? t[5].cast<bool>() : false,
                                     t.size() > 6 ? t[6].cast<std::string>() : std::string()));
          }
          openai::Usage u{prompt_tokens, completion_tokens, cached_tokens};
          return openai::completion_json(chat, id, model, created, cs, u);
        });
  m.def("chunk_event",
        [](bool chat, const std::string& id, const std::string& model, int64_t created, int index, const std::string& text,
           bool role_delta, const std::string& finish, const std::string& tool_calls_json, py::object logprob) {
          json::Value tc;
          const json::Value* tcp = nullptr;
          if (!tool_calls_json.empty() && tool_calls_json != "null") { tc = json::parse(tool_calls_json); tcp = &tc; }
          openai::TokenLogprob lp;
          const openai::TokenLogprob* lpp = nullptr;
          if (!logprob.is_none()) {
            py::tuple t = logprob.cast<py::tuple>();
            lp.token = t[0].cast<std::string>();
            lp.logprob = t[1].cast<double>();
            lp.top = t[2].cast<std::vector<std::pair<std::string, double>>>();
            lpp = &lp;
          }
          return openai::chunk_event(chat, id, model, created, index, text, role_delta, finish, tcp, lpp);
        },
        py::arg("chat"), py::arg("id"), py::arg("model"), py::arg("created"), py::arg("index"), py::arg("text"),
        py::arg("role_delta") = false, py::arg("finish_reason") = "", py::arg("tool_calls_json") = "",
        py::arg("logprob") = py::none());
  m.def("usage_event", [](bool chat, const std::string& id, const std::string& model, int64_t created, int64_t p, int64_t c, int64_t cached) {
    return openai::usage_event(chat, id, model, created, openai::Usage{p, c, cached});
  });
  m.def("done_event", &openai::done_event);
  m.def("models_json", &openai::models_json);
  m.def("error_json", [](int status, const std::string& message, const std::string& param, const std::string& code,
                         const std::string& type) {
    openai::ApiError e;
    e.status = status; e.message = message; e.param = param; e.code = code; e.type = type;
    return e.to_json();
  }, py::arg("status"), py::arg("message"), py::arg("param") = "", py::arg("code") = "",
     py::arg("type") = "invalid_request_error");

  py::class_<openai::StopScanner>(m, "StopScanner")
      .def(py::init<std::vector<std::string>>())
      .def("feed", [](openai::StopScanner& s, const py::bytes& b) { return py::bytes(s.feed(std::string(b))); })
      .def("flush", [](openai::StopScanner& s) { return py::bytes(s.flush()); })
      .def("stopped", &openai::StopScanner::stopped);

  // ---------------- HTTP server
  py::class_<HttpServer>(m, "HttpServer")
      .def(py::init([](const std::string& host, int port, size_t max_header, size_t max_body, int keepalive_ms) {
        HttpLimits lim;
        lim.max_header_bytes = max_header;
        lim.max_body_bytes = max_body;
        lim.keepalive_comment_ms = keepalive_ms;
        return new HttpServer(host, port, lim);
      }), py::arg("host") = "127.0.0.1", py::arg("port") = 0, py::arg("max_header_bytes") = 16 * 1024,
          py::arg("max_body_bytes") = size_t(256) << 20, py::arg("keepalive_ms") = 30000)
      .def("start", &HttpServer::start)
      .def("stop", &HttpServer::stop, py::call_guard<py::gil_scoped_release>())
      .def("port", &HttpServer::port)
      .def("poll", [](HttpServer& s, int timeout_ms) {
        std::vector<HttpRequest> reqs;
        {
          py::gil_scoped_release rel;
          reqs = s.poll(timeout_ms);
        }
        py::list out;
        for (auto& r : reqs) {
          py::dict d;
          d["conn"] = r.conn;
          d["method"] = r.method;
          d["path"] = r.path;
          d["query"] = r.query;
          d["headers"] = r.headers;
          d["body"] = py::bytes(r.body);
          out.append(d);
        }
        return out;
      }, py::arg("timeout_ms") = 0)
      .def("poll_disconnects", &HttpServer::poll_disconnects)
      .def("respond", [](HttpServer& s, uint64_t conn, int status, const std::string& ctype, const py::bytes& body) {
        s.respond(conn, status, ctype, std::string(body));
      }, py::arg("conn"), py::arg("status"), py::arg("content_type"), py::arg("body"))
      .def("stream_begin", &HttpServer::stream_begin, py::arg("conn"), py::arg("content_type") = "text/event-stream")
      .def("stream_send", [](HttpServer& s, uint64_t conn, const py::bytes& data) { s.stream_send(conn, std::string(data)); })
      .def("stream_end", &HttpServer::stream_end);
}
