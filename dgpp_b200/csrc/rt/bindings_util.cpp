// pybind11 surface of the small runtime services (logger, trace, crc32c, watchdogs, deployment config, memory plan).
#include <pybind11/functional.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "rt/core_util.h"
#include "rt/jpeg.h"
#include "rt/webp.h"

namespace py = pybind11;
using namespace dgpp;

namespace {

// A Python callable that may be released from a thread that does not hold the GIL.
std::shared_ptr<py::object> keep(py::object fn) {
  return std::shared_ptr<py::object>(new py::object(std::move(fn)), [](py::object* p) {
    py::gil_scoped_acquire g;
    delete p;
  });
}
// The watchdogs join their thread in the destructor; that thread may be waiting for the GIL inside a callback.
template <class T>
struct NoGilDelete {
  void operator()(T* p) const {
    py::gil_scoped_release r;
    delete p;
  }
};

}  // namespace

void bind_util(py::module_& m) {
  m.def("log", [](const std::string& level, const std::string& component, const std::string& msg) {
    Logger::get().log(Logger::parse(level, LogLevel::Info), component, msg);
  });
  m.def("set_log_level", [](const std::string& level) { Logger::get().set_level(Logger::parse(level, LogLevel::Info)); });
  m.def("log_level", [] { return static_cast<int>(Logger::get().level()); });
  m.def("set_log_sink", [](py::object fn) {
    if (fn.is_none()) { Logger::get().set_sink(nullptr); return; }
    auto h = keep(fn);
    Logger::get().set_sink([h](const std::string& line) { py::gil_scoped_acquire g; (*h)(line); });
  });
  m.def("trace_open", [](const std::string& path) { Trace::get().open(path); });
  m.def("trace_close", [] { Trace::get().close(); });
  m.def("trace_enabled", [] { return Trace::get().enabled(); });
  m.def("trace_emit", [](const std::string& name, int64_t ts, int64_t dur, const std::string& args) {
    Trace::get().emit(name, ts, dur, args);
  }, py::arg("name"), py::arg("ts_us"), py::arg("dur_us"), py::arg("args_json") = "{}");
  m.def("trace_now_us", &Trace::now_us);
  m.def("crc32c", [](const py::bytes& b, uint32_t crc) {
    const std::string s = b;
    return crc32c(s.data(), s.size(), crc);
  }, py::arg("data"), py::arg("crc") = 0u);

  py::class_<EngineWatchdog, std::unique_ptr<EngineWatchdog, NoGilDelete<EngineWatchdog>>>(m, "EngineWatchdog")
      .def(py::init([](int deadline_ms, py::object on_stall, int poll_ms) {
        std::function<void(int64_t)> cb;
        if (!on_stall.is_none()) {
          auto h = keep(on_stall);
          cb = [h](int64_t ms) { py::gil_scoped_acquire g; (*h)(ms); };
        }
        return new EngineWatchdog(std::chrono::milliseconds(deadline_ms), cb, std::chrono::milliseconds(poll_ms));
      }), py::arg("deadline_ms") = 120000, py::arg("on_stall") = py::none(), py::arg("poll_ms") = 50)
      .def("progress", &EngineWatchdog::progress)
      .def("set_busy", &EngineWatchdog::set_busy)
      .def("fired", &EngineWatchdog::fired);
  py::class_<ShutdownWatchdog, std::unique_ptr<ShutdownWatchdog, NoGilDelete<ShutdownWatchdog>>>(m, "ShutdownWatchdog")
      .def(py::init([](int limit_ms, py::object on_timeout) {
        std::function<void()> cb;
        if (!on_timeout.is_none()) {
          auto h = keep(on_timeout);
          cb = [h] { py::gil_scoped_acquire g; (*h)(); };
        }
        return new ShutdownWatchdog(std::chrono::milliseconds(limit_ms), cb);
      }), py::arg("limit_ms") = 30000, py::arg("on_timeout") = py::none())
      .def("disarm", &ShutdownWatchdog::disarm)
      .def("timed_out", &ShutdownWatchdog::timed_out);

  m.def("parse_cluster_config", [](const std::string& text) {
    const ClusterConfig c = ClusterConfig::parse(text);
    return py::make_tuple(c.to_json().dump(), c.digest());
  });
  m.def("plan_kv", [](int64_t free_bytes, int64_t headroom, int64_t workspace, int layers, int kv_heads, int head_dim,
                      int block_tokens, bool fp8, int64_t max_blocks) {
    const MemoryPlan p = plan_kv(free_bytes, headroom, workspace, layers, kv_heads, head_dim, block_tokens, fp8, max_blocks);
    return py::make_tuple(p.kv_blocks, p.kv_bytes, p.tokens);
  }, py::arg("free_bytes"), py::arg("headroom_bytes"), py::arg("workspace_bytes"), py::arg("layers"), py::arg("kv_heads"),
     py::arg("head_dim"), py::arg("block_tokens"), py::arg("fp8") = true, py::arg("max_blocks") = int64_t(-1));

  m.def("process_memory", []() {
    const ProcessMemory pm = process_memory();
    py::dict d;
    d["rss_bytes"] = pm.rss_bytes; d["peak_rss_bytes"] = pm.peak_rss_bytes; d["locked_bytes"] = pm.locked_bytes;
    d["memlock_limit_bytes"] = pm.memlock_limit_bytes;
    return d;
  });
  m.def("decode_jpeg", [](const py::bytes& data) {
    // (width, height, channels, pixel bytes): interleaved 8-bit grey or RGB; raises ValueError naming what is wrong
    const std::string buf = data;
    rt::jpeg::Image img;
    {
      py::gil_scoped_release release;
      try {
        img = rt::jpeg::decode(reinterpret_cast<const uint8_t*>(buf.data()), buf.size());
      } catch (const std::runtime_error& e) {
        py::gil_scoped_acquire acquire;
        throw py::value_error(e.what());
      }
    }
    return py::make_tuple(img.width, img.height, img.channels,
                          py::bytes(reinterpret_cast<const char*>(img.pixels.data()), img.pixels.size()));
  });
  m.def("decode_webp", [](const py::bytes& data) {
    // (width, height, RGBA bytes) of a lossless WebP file; raises ValueError naming what is wrong (lossy files too)
    const std::string buf = data;
    rt::webp::Image img;
    {
      py::gil_scoped_release release;
      try {
        img = rt::webp::decode(reinterpret_cast<const uint8_t*>(buf.data()), buf.size());
      } catch (const std::runtime_error& e) {
        py::gil_scoped_acquire acquire;
        throw py::value_error(e.what());
      } catch (const std::bad_alloc&) {
        py::gil_scoped_acquire acquire;
        throw py::value_error("webp: image too large");
      }
    }
    return py::make_tuple(img.width, img.height, py::bytes(reinterpret_cast<const char*>(img.rgba.data()), img.rgba.size()));
  });
  m.def("file_residency", [](const std::string& path) {
    int64_t size = -1;
    const double f = file_residency(path, &size);
    return py::make_tuple(f, size);
  });
  py::class_<PrefillProgress>(m, "PrefillProgress")
      .def(py::init<>())
      .def("begin", &PrefillProgress::begin)
      .def("advance", &PrefillProgress::advance)
      .def("end", &PrefillProgress::end)
      .def("snapshot", [](const PrefillProgress& p, int64_t now_ms) {
        py::list out;
        for (const auto& r : p.snapshot(now_ms)) out.append(py::make_tuple(r.id, r.done, r.total, r.started_ms, r.idle_ms));
        return out;
      })
      .def("most_stalled", [](const PrefillProgress& p, int64_t now_ms) {
        const auto r = p.most_stalled(now_ms);
        return py::make_tuple(r.id, r.done, r.total, r.started_ms, r.idle_ms);
      });
}
