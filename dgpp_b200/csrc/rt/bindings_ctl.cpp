// pybind11 surface of the control plane: prefill quantum controller, operation journal, framed TCP, roster, disk tier.
#include <pybind11/functional.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "rt/control.h"
#include "rt/disk_tier.h"
#include "rt/net.h"

namespace py = pybind11;
using namespace dgpp;

namespace {
template <class T>
struct NoGilDelete {
  void operator()(T* p) const {
    py::gil_scoped_release r;
    delete p;
  }
};
py::dict view_dict(const RosterView& v) {
  py::dict d;
  d["epoch"] = v.epoch;
  d["world"] = v.world;
  py::dict m;
  for (const auto& kv : v.members) m[py::int_(kv.first)] = kv.second;
  d["members"] = m;
  d["complete"] = v.complete();
  return d;
}
py::dict record_dict(const JournalRecord& r) {
  py::dict d;
  d["seq"] = r.seq;
  d["op"] = r.op;
  d["id"] = r.id;
  d["tokens"] = r.tokens;
  d["arg"] = r.arg;
  d["extra"] = r.extra;
  d["digest"] = r.digest;
  d["line"] = r.to_line();
  return d;
}
}  // namespace

void bind_ctl(py::module_& m) {
  py::class_<PrefillController>(m, "PrefillController")
      .def(py::init([](double gap_ms, double first_ms, int64_t start, int64_t floor, int64_t idle_floor, int64_t ceiling,
                       int64_t granule) {
        PrefillControlConfig c;
        c.decode_gap_target_ms = gap_ms; c.first_token_target_ms = first_ms; c.start = start; c.floor = floor;
        c.idle_floor = idle_floor; c.ceiling = ceiling; c.granule = granule;
        return new PrefillController(c);
      }), py::arg("decode_gap_target_ms") = 1000.0, py::arg("first_token_target_ms") = 3000.0, py::arg("start") = 256,
          py::arg("floor") = 64, py::arg("idle_floor") = 1024, py::arg("ceiling") = 8192, py::arg("granule") = 16)
      .def("observe", &PrefillController::observe, py::arg("tokens"), py::arg("pass_ms"), py::arg("decoding"))
      .def("next", &PrefillController::next, py::arg("decoding"), py::arg("waiting_tokens"), py::arg("oldest_wait_ms") = 0.0)
      .def("quantum", &PrefillController::quantum)
      .def("rate_tokens_per_ms", &PrefillController::rate_tokens_per_ms);

  py::class_<Journal>(m, "Journal")
      .def(py::init<>())
      .def("append", [](Journal& j, const std::string& op, const std::string& id, const std::vector<int32_t>& tokens, int64_t arg,
                        const std::string& extra) {
        return record_dict(j.append(op, id, tokens, arg, extra));
      }, py::arg("op"), py::arg("id") = "", py::arg("tokens") = std::vector<int32_t>(), py::arg("arg") = 0,
         py::arg("extra") = "")
      // replays one wire line (order and digest are checked) and returns the record
      .def("replay_line", [](Journal& j, const std::string& line) {
        const JournalRecord r = JournalRecord::from_line(line);
        j.replay(r);
        return record_dict(r);
      })
      .def("since", [](const Journal& j, uint64_t seq) {
        std::vector<std::string> out;
        for (const auto& r : j.since(seq)) out.push_back(r.to_line());
        return out;
      })
      .def("set_keep", &Journal::set_keep)
      .def("digest", &Journal::digest)
      .def("next_seq", &Journal::next_seq);

  py::class_<Listener>(m, "Listener")
      .def(py::init<int, bool>(), py::arg("port") = 0, py::arg("loopback") = true)
      .def("port", &Listener::port)
      .def("accept", [](Listener& l, int timeout_ms) -> py::object {
        FramedSocket s;
        { py::gil_scoped_release r; s = l.accept_one(timeout_ms); }
        if (!s.valid()) return py::none();
        return py::cast(new FramedSocket(std::move(s)), py::return_value_policy::take_ownership);
      }, py::arg("timeout_ms") = 1000);
  py::class_<FramedSocket>(m, "FramedSocket")
      .def_static("connect", [](const std::string& host, int port, int timeout_ms) {
        py::gil_scoped_release r;
        return new FramedSocket(FramedSocket::connect_to(host, port, timeout_ms));
      }, py::arg("host"), py::arg("port"), py::arg("timeout_ms") = 5000, py::return_value_policy::take_ownership)
      .def("send", [](FramedSocket& s, const py::bytes& b) { const std::string p = b; py::gil_scoped_release r; return s.send_frame(p); })
      .def("recv", [](FramedSocket& s, int timeout_ms) -> py::object {
        std::string out;
        int rc;
        { py::gil_scoped_release r; rc = s.recv_frame(&out, timeout_ms); }
        if (rc == 1) return py::bytes(out);
        if (rc == 0) return py::none();
        throw std::runtime_error("peer closed the connection");
      }, py::arg("timeout_ms") = 1000)
      .def("close", &FramedSocket::close);

  py::class_<RosterServer, std::unique_ptr<RosterServer, NoGilDelete<RosterServer>>>(m, "RosterServer")
      .def(py::init<int, int, int>(), py::arg("world"), py::arg("port") = 0, py::arg("deadline_ms") = 3000)
      .def("port", &RosterServer::port)
      .def("view", [](const RosterServer& s) { return view_dict(s.view()); })
      .def("evictions", &RosterServer::evictions)
      .def("stop", [](RosterServer& s) { py::gil_scoped_release r; s.stop(); });
  py::class_<RosterClient, std::unique_ptr<RosterClient, NoGilDelete<RosterClient>>>(m, "RosterClient")
      .def(py::init([](const std::string& host, int port, int rank, int world, const std::string& endpoint, int heartbeat_ms) {
        py::gil_scoped_release r;
        return new RosterClient(host, port, rank, world, endpoint, heartbeat_ms);
      }), py::arg("host"), py::arg("port"), py::arg("rank"), py::arg("world"), py::arg("endpoint") = "-", py::arg("heartbeat_ms") = 1000)
      .def("view", [](const RosterClient& c) { return view_dict(c.view()); })
      .def("wait_complete", [](const RosterClient& c, int ms) { py::gil_scoped_release r; return c.wait_complete(ms); }, py::arg("timeout_ms") = 5000)
      .def("server_lost", &RosterClient::server_lost)
      .def("freeze", &RosterClient::freeze)
      .def("stop", [](RosterClient& c, bool bye) { py::gil_scoped_release r; c.stop(bye); }, py::arg("say_goodbye") = true);

  m.def("probe_cache_storage", [](const std::string& dir) {
    const CacheStorageInfo i = probe_cache_storage(dir);
    py::dict d;
    d["exists"] = i.exists; d["writable"] = i.writable; d["direct_io"] = i.direct_io;
    d["free_bytes"] = i.free_bytes; d["total_bytes"] = i.total_bytes;
    return d;
  });
  py::class_<DiskTier, std::unique_ptr<DiskTier, NoGilDelete<DiskTier>>>(m, "DiskTier")
      .def(py::init<const std::string&, size_t, size_t, bool, bool>(), py::arg("dir"), py::arg("page_bytes") = 1 << 20,
           py::arg("pages") = 1024, py::arg("try_direct") = true, py::arg("adopt") = true)
      .def("direct_io", &DiskTier::direct_io)
      .def("payload_per_page", &DiskTier::payload_per_page)
      .def("free_pages", &DiskTier::free_pages)
      .def("blobs", &DiskTier::blobs)
      .def("contains", &DiskTier::contains)
      .def("put", [](DiskTier& t, uint64_t key, py::buffer b) {
        py::buffer_info i = b.request();
        const size_t n = static_cast<size_t>(i.size * i.itemsize);
        py::gil_scoped_release r;
        return t.put(key, i.ptr, n);
      })
      .def("put_async", [](DiskTier& t, uint64_t key, py::buffer b) {
        py::buffer_info i = b.request();
        return t.put_async(key, i.ptr, static_cast<size_t>(i.size * i.itemsize));
      })
      .def("wait", [](DiskTier& t, uint64_t ticket) { py::gil_scoped_release r; t.wait(ticket); })
      .def("flush", [](DiskTier& t) { py::gil_scoped_release r; t.flush(); })
      .def("get", [](DiskTier& t, uint64_t key) -> py::object {
        std::string out;
        bool ok;
        { py::gil_scoped_release r; ok = t.get(key, &out); }
        if (!ok) return py::none();
        return py::bytes(out);
      })
      .def("erase", &DiskTier::erase)
      .def("commit", [](DiskTier& t) { py::gil_scoped_release r; t.commit(); })
      .def("commit_digest", &DiskTier::commit_digest)
      .def("corrupt_for_test", &DiskTier::corrupt_for_test)
      .def("stats", [](const DiskTier& t) {
        const DiskTierStats s = t.stats();
        py::dict d;
        d["puts"] = s.puts; d["gets"] = s.gets; d["hits"] = s.hits; d["misses"] = s.misses; d["evictions"] = s.evictions;
        d["crc_failures"] = s.crc_failures; d["bytes_written"] = s.bytes_written; d["bytes_read"] = s.bytes_read;
        return d;
      });
}
