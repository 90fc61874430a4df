// Bindings of the scheduler, prefix cache and fake engine.
#include <pybind11/functional.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "rt/fake_engine.h"
#include "rt/prefix_cache.h"
#include "rt/scheduler.h"

namespace py = pybind11;
using namespace dgpp;

void bind_text(py::module_& m);     // tokenizer, chat template (bindings_text.cpp)
void bind_load(py::module_& m);     // safetensors, hub cache, architecture detect, shard specs (bindings_load.cpp)
void bind_grammar(py::module_& m);  // JSON / schema constrained decoding (bindings_grammar.cpp)
void bind_util(py::module_& m);     // logger, trace, crc32c, watchdogs, config, memory plan (bindings_util.cpp)
void bind_ctl(py::module_& m);      // prefill controller, journal, framed TCP, roster, disk tier (bindings_ctl.cpp)
void bind_serve(py::module_& m);    // sampler oracle, grammars, http server (bindings_serve.cpp)

namespace {

// Engine implemented in Python (the GPU engines): methods are looked up on the Python object.
class PyEngine : public SchedulerEngine {
 public:
  using SchedulerEngine::SchedulerEngine;
  int max_concurrent() const override { PYBIND11_OVERRIDE_PURE(int, SchedulerEngine, max_concurrent); }
  int block_tokens() const override { PYBIND11_OVERRIDE_PURE(int, SchedulerEngine, block_tokens); }
  int64_t total_blocks() const override { PYBIND11_OVERRIDE_PURE(int64_t, SchedulerEngine, total_blocks); }
  int64_t free_blocks() const override { PYBIND11_OVERRIDE_PURE(int64_t, SchedulerEngine, free_blocks); }
  int64_t max_context() const override { PYBIND11_OVERRIDE_PURE(int64_t, SchedulerEngine, max_context); }
  bool reserve(int slot, int64_t tokens) override { PYBIND11_OVERRIDE_PURE(bool, SchedulerEngine, reserve, slot, tokens); }
  void attach_prefix(int slot, const std::vector<int32_t>& blocks) override {
    PYBIND11_OVERRIDE_PURE(void, SchedulerEngine, attach_prefix, slot, blocks);
  }
  int32_t prefill(int slot, const int32_t* tokens, int64_t pos, int64_t count, bool last) override {
    py::gil_scoped_acquire gil;
    py::function f = py::get_override(static_cast<const SchedulerEngine*>(this), "prefill");
    if (!f) throw std::runtime_error("engine.prefill is not implemented");
    std::vector<int32_t> v(tokens, tokens + count);
    return f(slot, v, pos, last).cast<int32_t>();
  }
  std::vector<int32_t> prefill_group(const std::vector<PrefillPiece>& pieces) override {
    py::gil_scoped_acquire gil;
    py::function f = py::get_override(static_cast<const SchedulerEngine*>(this), "prefill_group");
    if (!f) return SchedulerEngine::prefill_group(pieces);       // one prefill() call per piece
    py::list arg;
    for (const auto& p : pieces) arg.append(py::make_tuple(p.slot, std::vector<int32_t>(p.tokens, p.tokens + p.count), p.pos, p.last));
    return f(arg).cast<std::vector<int32_t>>();
  }
  std::vector<std::vector<int32_t>> step_batch(const std::vector<int>& slots) override {
    PYBIND11_OVERRIDE_PURE(std::vector<std::vector<int32_t>>, SchedulerEngine, step_batch, slots);
  }
  // Python: mixed_step((slot, tokens, pos, last), slots) -> None (no such pass) or (first, [[tokens of slots[i]], ...])
  bool mixed_step(const PrefillPiece& p, const std::vector<int>& slots, int32_t* first,
                  std::vector<std::vector<int32_t>>* out) override {
    py::gil_scoped_acquire gil;
    py::function f = py::get_override(static_cast<const SchedulerEngine*>(this), "mixed_step");
    if (!f) return false;
    py::object r = f(py::make_tuple(p.slot, std::vector<int32_t>(p.tokens, p.tokens + p.count), p.pos, p.last), slots);
    if (r.is_none()) return false;
    py::tuple t = r.cast<py::tuple>();
    *first = t[0].cast<int32_t>();
    *out = t[1].cast<std::vector<std::vector<int32_t>>>();
    return true;
  }
  int max_tokens_per_step() const override { PYBIND11_OVERRIDE(int, SchedulerEngine, max_tokens_per_step); }
  int64_t usable_prefix(const std::vector<int32_t>& blocks) const override {
    PYBIND11_OVERRIDE(int64_t, SchedulerEngine, usable_prefix, blocks);
  }
  std::vector<int32_t> slot_blocks(int slot) const override {
    PYBIND11_OVERRIDE_PURE(std::vector<int32_t>, SchedulerEngine, slot_blocks, slot);
  }
  void retain_block(int32_t b) override { PYBIND11_OVERRIDE_PURE(void, SchedulerEngine, retain_block, b); }
  void release_block(int32_t b) override { PYBIND11_OVERRIDE_PURE(void, SchedulerEngine, release_block, b); }
  int block_refcount(int32_t b) const override { PYBIND11_OVERRIDE_PURE(int, SchedulerEngine, block_refcount, b); }
  void open(int slot, const std::string& id) override { PYBIND11_OVERRIDE(void, SchedulerEngine, open, slot, id); }
  void close(int slot) override { PYBIND11_OVERRIDE_PURE(void, SchedulerEngine, close, slot); }
};

struct Event {
  std::string kind, id;
  int64_t a, b;
};

class EventLog : public SchedulerObserver {
 public:
  void on_admit(const std::string& id, int slot, int64_t cached) override { ev.push_back({"admit", id, slot, cached}); }
  void on_token(const std::string& id, int32_t tok, int64_t index) override { ev.push_back({"token", id, tok, index}); }
  void on_retire(const std::string& id, RetireReason why, int64_t generated) override {
    ev.push_back({std::string("retire:") + retire_name(why), id, static_cast<int64_t>(why), generated});
  }
  std::vector<py::tuple> take() {
    std::vector<py::tuple> out;
    for (auto& e : ev) out.push_back(py::make_tuple(e.kind, e.id, e.a, e.b));
    ev.clear();
    return out;
  }
  std::vector<Event> ev;
};

// Owns the observer and keeps the engine alive.
class PyScheduler {
 public:
  PyScheduler(py::object engine, const SchedulerConfig& cfg)
      : engine_obj_(std::move(engine)), log_(new EventLog()),
        sched_(new Scheduler(engine_obj_.cast<SchedulerEngine*>(), cfg, log_.get())) {}
  void submit(const std::string& id, std::vector<int32_t> prompt, int64_t max_tokens, std::vector<int32_t> eos,
              std::vector<int32_t> stop, bool ignore_eos, bool prefix_cache, const std::string& cache_key) {
    SchedRequest r;
    r.id = id;
    r.prompt = std::move(prompt);
    r.max_tokens = max_tokens;
    r.eos_ids = std::move(eos);
    r.stop_ids = std::move(stop);
    r.ignore_eos = ignore_eos;
    r.prefix_cache = prefix_cache;
    r.cache_key = cache_key;
    sched_->submit(std::move(r));
  }
  void cancel(const std::string& id) { sched_->cancel(id); }
  int64_t tick() { return sched_->tick(); }
  int64_t run(int64_t max_ticks) { return sched_->run(max_ticks); }
  bool idle() const { return sched_->idle(); }
  int active() const { return sched_->active_count(); }
  int64_t queued() const { return sched_->queued(); }
  std::vector<py::tuple> events() { return log_->take(); }
  uint64_t op_digest() const { return sched_->op_digest(); }
  uint64_t prefix_digest() const { return sched_->prefix_digest(); }
  py::dict meters() const {
    const SchedMeters& m = sched_->meters();
    const PrefixStats& p = sched_->prefix_stats();
    py::dict d;
    d["ticks"] = m.ticks; d["admitted"] = m.admitted; d["retired"] = m.retired; d["shed"] = m.shed;
    d["decode_passes"] = m.decode_passes; d["decode_tokens"] = m.decode_tokens; d["mixed_passes"] = m.mixed_passes;
    d["prefill_tokens"] = m.prefill_tokens; d["prefill_calls"] = m.prefill_calls;
    d["prefix_hit_tokens"] = m.prefix_hit_tokens; d["cancelled"] = m.cancelled;
    d["queue_peak"] = m.queue_peak; d["active_peak"] = m.active_peak;
    d["prefix_lookups"] = p.lookups; d["prefix_hits"] = p.hits; d["prefix_inserts"] = p.inserts;
    d["prefix_evictions"] = p.evictions; d["prefix_ghost_hits"] = p.ghost_hits;
    d["prefix_check_rejects"] = p.check_rejects;
    return d;
  }

 private:
  py::object engine_obj_;
  std::unique_ptr<EventLog> log_;
  std::unique_ptr<Scheduler> sched_;
};

}  // namespace

void bind_more(py::module_& m) {
  m.def("chain_hash", [](uint64_t parent, const std::vector<int32_t>& ids) {
    return chain_hash(parent, ids.data(), static_cast<int>(ids.size()));
  });
  m.attr("FNV_SEED") = kFnvSeed;

  py::class_<SchedulerEngine, PyEngine>(m, "SchedulerEngine")
      .def(py::init<>());

  py::class_<FakeEngine, SchedulerEngine>(m, "FakeEngine")
      .def(py::init<int, int, int64_t, int64_t, int, int>(), py::arg("slots"), py::arg("block_tokens"),
           py::arg("blocks"), py::arg("max_context"), py::arg("vocab"), py::arg("tokens_per_step") = 1)
      .def("free_blocks", &FakeEngine::free_blocks)
      .def("total_blocks", &FakeEngine::total_blocks)
      .def("max_context", &FakeEngine::max_context)
      .def("max_concurrent", &FakeEngine::max_concurrent)
      .def("block_tokens", &FakeEngine::block_tokens)
      .def_readonly("prefill_calls", &FakeEngine::prefill_calls)
      .def_readonly("prefill_tokens", &FakeEngine::prefill_tokens)
      .def_readonly("decode_passes", &FakeEngine::decode_passes)
      .def_readonly("mixed_calls", &FakeEngine::mixed_calls)
      .def_readwrite("mixed", &FakeEngine::mixed)
      .def_static("expected", &FakeEngine::expected);

  py::enum_<AdmissionPolicy>(m, "AdmissionPolicy")
      .value("FullReserve", AdmissionPolicy::FullReserve)
      .value("GrowOnDemand", AdmissionPolicy::GrowOnDemand);

  py::class_<SchedulerConfig>(m, "SchedulerConfig")
      .def(py::init<>())
      .def_readwrite("policy", &SchedulerConfig::policy)
      .def_readwrite("prefill_budget_idle", &SchedulerConfig::prefill_budget_idle)
      .def_readwrite("prefill_budget_busy", &SchedulerConfig::prefill_budget_busy)
      .def_readwrite("prefill_chunk", &SchedulerConfig::prefill_chunk)
      .def_readwrite("prefix_cache", &SchedulerConfig::prefix_cache)
      .def_readwrite("prefix_min_tokens", &SchedulerConfig::prefix_min_tokens)
      .def_readwrite("prefix_max_entries", &SchedulerConfig::prefix_max_entries)
      .def_readwrite("grow_margin_tokens", &SchedulerConfig::grow_margin_tokens)
      .def_readwrite("prefill_group_max", &SchedulerConfig::prefill_group_max)
      .def_readwrite("mixed_pass", &SchedulerConfig::mixed_pass);

  py::class_<PyScheduler>(m, "Scheduler")
      .def(py::init<py::object, const SchedulerConfig&>())
      .def("submit", &PyScheduler::submit, py::arg("id"), py::arg("prompt"), py::arg("max_tokens"),
           py::arg("eos_ids") = std::vector<int32_t>{}, py::arg("stop_ids") = std::vector<int32_t>{},
           py::arg("ignore_eos") = false, py::arg("prefix_cache") = true, py::arg("cache_key") = "")
      .def("cancel", &PyScheduler::cancel)
      .def("tick", &PyScheduler::tick)
      .def("run", &PyScheduler::run, py::arg("max_ticks") = int64_t(1) << 30)
      .def("idle", &PyScheduler::idle)
      .def("active", &PyScheduler::active)
      .def("queued", &PyScheduler::queued)
      .def("events", &PyScheduler::events)
      .def("op_digest", &PyScheduler::op_digest)
      .def("prefix_digest", &PyScheduler::prefix_digest)
      .def("meters", &PyScheduler::meters);

  bind_text(m);
  bind_serve(m);
  bind_load(m);
  bind_grammar(m);
  bind_ctl(m);
  bind_util(m);
}
