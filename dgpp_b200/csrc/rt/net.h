// Control-plane networking: length-framed TCP messages and the roster (who is in the world, who is alive).
//
// Frame: 4-byte big-endian length + payload (<= 16 MiB).  Every blocking call has a deadline; a peer that stops
// answering shows up as a timeout, never as a hang.
//
// Roster: one server (rank 0's process or a side-car) and one client per rank.
//   client -> server   "ANNOUNCE <rank> <world> <endpoint>"   once after connect
//                      "HEARTBEAT <rank>"                      every `heartbeat_ms`
//                      "LEAVE <rank>"                          orderly exit
//   server -> clients  "ROSTER <epoch> <world> <rank>=<endpoint>|- ..." on every change of membership
// A member that has not been heard for `deadline_ms` is evicted: the epoch goes up and the new roster is sent to
// the survivors, whose `on_change` hook runs (the serving process stops launching collectives with that peer).
// The data plane never goes through here.
// (reference counterparts: src/net/tcp.cpp framed sockets, src/net/roster.cpp ANNOUNCE / ROSTER / HEARTBEAT frames,
//  epochs and eviction with a 1 s heartbeat and a 3 s deadline.)
#pragma once
#include <arpa/inet.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstring>
#include <functional>
#include <map>
#include <mutex>
#include <sstream>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

namespace dgpp {

constexpr size_t kMaxFrameBytes = 16u << 20;

inline int64_t steady_ms() {
  return std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

// A connected stream socket with framed send / receive.  Move-only.
class FramedSocket {
 public:
  FramedSocket() = default;
  explicit FramedSocket(int fd) : fd_(fd) { tune(); }
  FramedSocket(FramedSocket&& o) noexcept : fd_(o.fd_), buf_(std::move(o.buf_)) { o.fd_ = -1; }
  FramedSocket& operator=(FramedSocket&& o) noexcept {
    if (this != &o) { close(); fd_ = o.fd_; buf_ = std::move(o.buf_); o.fd_ = -1; }
    return *this;
  }
  FramedSocket(const FramedSocket&) = delete;
  FramedSocket& operator=(const FramedSocket&) = delete;
  ~FramedSocket() { close(); }

  static FramedSocket connect_to(const std::string& host, int port, int timeout_ms) {
    const int64_t deadline = steady_ms() + timeout_ms;
    for (;;) {
      int fd = ::socket(AF_INET, SOCK_STREAM, 0);
      if (fd < 0) throw std::runtime_error("socket() failed");
      sockaddr_in a{};
      a.sin_family = AF_INET;
      a.sin_port = htons(static_cast<uint16_t>(port));
      if (inet_pton(AF_INET, host.c_str(), &a.sin_addr) != 1) { ::close(fd); throw std::runtime_error("bad IPv4 address " + host); }
      if (::connect(fd, reinterpret_cast<sockaddr*>(&a), sizeof(a)) == 0) return FramedSocket(fd);
      ::close(fd);
      if (steady_ms() >= deadline) throw std::runtime_error("connect to " + host + ":" + std::to_string(port) + " timed out");
      std::this_thread::sleep_for(std::chrono::milliseconds(20));
    }
  }
  bool valid() const { return fd_ >= 0; }
  int fd() const { return fd_; }
  void close() {
    if (fd_ >= 0) { ::shutdown(fd_, SHUT_RDWR); ::close(fd_); fd_ = -1; }
  }
  // false when the peer is gone.
  bool send_frame(const std::string& payload) {
    if (fd_ < 0 || payload.size() > kMaxFrameBytes) return false;
    unsigned char head[4];
    const uint32_t n = static_cast<uint32_t>(payload.size());
    head[0] = n >> 24; head[1] = n >> 16; head[2] = n >> 8; head[3] = n;
    return write_all(head, 4) && write_all(payload.data(), payload.size());
  }
  // 1 = frame read, 0 = nothing within timeout_ms, -1 = peer closed / error.
  int recv_frame(std::string* out, int timeout_ms) {
    if (fd_ < 0) return -1;
    const int64_t deadline = steady_ms() + timeout_ms;
    for (;;) {
      if (buf_.size() >= 4) {
        const uint32_t n = (uint32_t(uint8_t(buf_[0])) << 24) | (uint32_t(uint8_t(buf_[1])) << 16) |
                           (uint32_t(uint8_t(buf_[2])) << 8) | uint32_t(uint8_t(buf_[3]));
        if (n > kMaxFrameBytes) return -1;
        if (buf_.size() >= 4 + static_cast<size_t>(n)) {
          out->assign(buf_, 4, n);
          buf_.erase(0, 4 + static_cast<size_t>(n));
          return 1;
        }
      }
      const int64_t left = deadline - steady_ms();
      pollfd p{fd_, POLLIN, 0};
      const int r = ::poll(&p, 1, static_cast<int>(left > 0 ? left : 0));
      if (r == 0) return 0;
      if (r < 0) { if (errno == EINTR) continue; return -1; }
      char tmp[65536];
      const ssize_t got = ::recv(fd_, tmp, sizeof(tmp), 0);
      if (got == 0) return -1;
      if (got < 0) { if (errno == EINTR || errno == EAGAIN) continue; return -1; }
      buf_.append(tmp, static_cast<size_t>(got));
    }
  }

 private:
  void tune() {
    int one = 1;
    setsockopt(fd_, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
  }
  bool write_all(const void* p, size_t n) {
    const char* c = static_cast<const char*>(p);
    while (n) {
      const ssize_t w = ::send(fd_, c, n, MSG_NOSIGNAL);
      if (w < 0) { if (errno == EINTR) continue; return false; }
      c += w; n -= static_cast<size_t>(w);
    }
    return true;
  }
  int fd_ = -1;
  std::string buf_;
};

// A listening socket on 127.0.0.1 / 0.0.0.0 (port 0 = pick one).
class Listener {
 public:
  explicit Listener(int port = 0, bool loopback = true) {
    fd_ = ::socket(AF_INET, SOCK_STREAM, 0);
    if (fd_ < 0) throw std::runtime_error("socket() failed");
    int one = 1;
    setsockopt(fd_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
    sockaddr_in a{};
    a.sin_family = AF_INET;
    a.sin_addr.s_addr = htonl(loopback ? INADDR_LOOPBACK : INADDR_ANY);
    a.sin_port = htons(static_cast<uint16_t>(port));
    if (::bind(fd_, reinterpret_cast<sockaddr*>(&a), sizeof(a)) != 0 || ::listen(fd_, 64) != 0) {
      ::close(fd_);
      throw std::runtime_error("bind/listen on port " + std::to_string(port) + " failed");
    }
    socklen_t len = sizeof(a);
    getsockname(fd_, reinterpret_cast<sockaddr*>(&a), &len);
    port_ = ntohs(a.sin_port);
  }
  ~Listener() { if (fd_ >= 0) ::close(fd_); }
  Listener(const Listener&) = delete;
  Listener& operator=(const Listener&) = delete;
  int port() const { return port_; }
  // An accepted connection, or an invalid socket after timeout_ms.
  FramedSocket accept_one(int timeout_ms) {
    pollfd p{fd_, POLLIN, 0};
    if (::poll(&p, 1, timeout_ms) <= 0) return FramedSocket();
    const int c = ::accept(fd_, nullptr, nullptr);
    return c >= 0 ? FramedSocket(c) : FramedSocket();
  }

 private:
  int fd_ = -1, port_ = 0;
};

// ------------------------------------------------------------------------------------------- roster
struct RosterView {
  uint64_t epoch = 0;
  int world = 0;
  std::map<int, std::string> members;   // rank -> endpoint of the ranks that are alive
  std::string encode() const {
    std::ostringstream o;
    o << "ROSTER " << epoch << ' ' << world;
    for (int r = 0; r < world; ++r) {
      auto it = members.find(r);
      o << ' ' << r << '=' << (it == members.end() ? std::string("-") : it->second);
    }
    return o.str();
  }
  static bool decode(const std::string& s, RosterView* v) {
    std::istringstream in(s);
    std::string tag;
    if (!(in >> tag >> v->epoch >> v->world) || tag != "ROSTER") return false;
    v->members.clear();
    std::string item;
    while (in >> item) {
      const size_t eq = item.find('=');
      if (eq == std::string::npos) return false;
      const std::string ep = item.substr(eq + 1);
      if (ep != "-") v->members[std::stoi(item.substr(0, eq))] = ep;
    }
    return true;
  }
  bool complete() const { return world > 0 && static_cast<int>(members.size()) == world; }
};

class RosterServer {
 public:
  RosterServer(int world, int port = 0, int deadline_ms = 3000) : world_(world), deadline_ms_(deadline_ms), listener_(port) {
    thread_ = std::thread([this] { loop(); });
  }
  ~RosterServer() { stop(); }
  int port() const { return listener_.port(); }
  RosterView view() const { std::lock_guard<std::mutex> g(mu_); return view_; }
  uint64_t evictions() const { return evictions_.load(); }
  void stop() {
    if (stop_.exchange(true)) return;
    if (thread_.joinable()) thread_.join();
  }

 private:
  struct Conn { FramedSocket sock; int rank = -1; int64_t last_ms = 0; };
  void loop() {
    view_.world = world_;
    while (!stop_.load()) {
      FramedSocket s = listener_.accept_one(10);
      if (s.valid()) { Conn c; c.sock = std::move(s); c.last_ms = steady_ms(); conns_.push_back(std::move(c)); }
      bool changed = false;
      for (size_t i = 0; i < conns_.size();) {
        Conn& c = conns_[i];
        bool drop = false;
        std::string f;
        for (;;) {
          const int r = c.sock.recv_frame(&f, 0);
          if (r == 0) break;
          if (r < 0) { drop = true; break; }
          c.last_ms = steady_ms();
          std::istringstream in(f);
          std::string tag;
          in >> tag;
          if (tag == "ANNOUNCE") {
            int rank = -1, world = 0; std::string ep;
            in >> rank >> world >> ep;
            if (rank < 0 || rank >= world_ || world != world_) { drop = true; break; }
            c.rank = rank;
            std::lock_guard<std::mutex> g(mu_);
            view_.members[rank] = ep;
            changed = true;
          } else if (tag == "LEAVE") {
            drop = true;
            break;
          }
        }
        if (!drop && steady_ms() - c.last_ms > deadline_ms_) { drop = true; if (c.rank >= 0) evictions_.fetch_add(1); }
        if (drop) {
          if (c.rank >= 0) {
            std::lock_guard<std::mutex> g(mu_);
            changed |= view_.members.erase(c.rank) > 0;
          }
          conns_.erase(conns_.begin() + static_cast<long>(i));
        } else {
          ++i;
        }
      }
      if (changed) {
        std::string msg;
        { std::lock_guard<std::mutex> g(mu_); ++view_.epoch; msg = view_.encode(); }
        for (auto& c : conns_) if (c.rank >= 0) c.sock.send_frame(msg);
      }
    }
  }
  int world_, deadline_ms_;
  Listener listener_;
  std::vector<Conn> conns_;
  mutable std::mutex mu_;
  RosterView view_;
  std::atomic<bool> stop_{false};
  std::atomic<uint64_t> evictions_{0};
  std::thread thread_;
};

class RosterClient {
 public:
  using ChangeFn = std::function<void(const RosterView&)>;
  RosterClient(const std::string& host, int port, int rank, int world, const std::string& endpoint, int heartbeat_ms = 1000,
               ChangeFn on_change = nullptr, int connect_timeout_ms = 5000)
      : rank_(rank), heartbeat_ms_(heartbeat_ms), on_change_(std::move(on_change)) {
    sock_ = FramedSocket::connect_to(host, port, connect_timeout_ms);
    sock_.send_frame("ANNOUNCE " + std::to_string(rank) + " " + std::to_string(world) + " " + endpoint);
    thread_ = std::thread([this] { loop(); });
  }
  ~RosterClient() { stop(true); }
  RosterView view() const { std::lock_guard<std::mutex> g(mu_); return view_; }
  bool server_lost() const { return lost_.load(); }
  // Stops sending heartbeats WITHOUT saying goodbye (what a wedged process looks like from outside).
  void freeze() { frozen_.store(true); }
  // Block until the roster holds all ranks (true) or the timeout passes.
  bool wait_complete(int timeout_ms) const {
    const int64_t deadline = steady_ms() + timeout_ms;
    while (steady_ms() < deadline) {
      if (view().complete()) return true;
      std::this_thread::sleep_for(std::chrono::milliseconds(5));
    }
    return view().complete();
  }
  void stop(bool say_goodbye) {
    if (stop_.exchange(true)) return;
    if (thread_.joinable()) thread_.join();
    if (say_goodbye && !frozen_.load()) sock_.send_frame("LEAVE " + std::to_string(rank_));
    sock_.close();
  }

 private:
  void loop() {
    int64_t next_beat = steady_ms();
    while (!stop_.load()) {
      if (!frozen_.load() && steady_ms() >= next_beat) {
        if (!sock_.send_frame("HEARTBEAT " + std::to_string(rank_))) { lost_.store(true); return; }
        next_beat = steady_ms() + heartbeat_ms_;
      }
      std::string f;
      const int r = sock_.recv_frame(&f, 10);
      if (r < 0) { lost_.store(true); return; }
      if (r == 1) {
        RosterView v;
        if (RosterView::decode(f, &v)) {
          { std::lock_guard<std::mutex> g(mu_); view_ = v; }
          if (on_change_) on_change_(v);
        }
      }
    }
  }
  int rank_, heartbeat_ms_;
  ChangeFn on_change_;
  FramedSocket sock_;
  mutable std::mutex mu_;
  RosterView view_;
  std::atomic<bool> stop_{false}, frozen_{false}, lost_{false};
  std::thread thread_;
};

}  // namespace dgpp
