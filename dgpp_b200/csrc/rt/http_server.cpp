#include "rt/http_server.h"

#include <arpa/inet.h>
#include <errno.h>
#include <fcntl.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <string.h>
#include <sys/epoll.h>
#include <sys/eventfd.h>
#include <sys/socket.h>
#include <unistd.h>

#include <algorithm>
#include <chrono>
#include <stdexcept>

namespace dgpp {

static int64_t now_ms() {
  return std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now().time_since_epoch()).count();
}
static void set_nonblock(int fd) { fcntl(fd, F_SETFL, fcntl(fd, F_GETFL, 0) | O_NONBLOCK); }

HttpServer::HttpServer(const std::string& host, int port, HttpLimits limits) : host_(host), port_(port), limits_(limits) {
  listen_fd_ = socket(AF_INET, SOCK_STREAM, 0);
  if (listen_fd_ < 0) throw std::runtime_error("http: socket() failed");
  int one = 1;
  setsockopt(listen_fd_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  sockaddr_in addr;
  memset(&addr, 0, sizeof(addr));
  addr.sin_family = AF_INET;
  addr.sin_port = htons(static_cast<uint16_t>(port));
  if (inet_pton(AF_INET, host.c_str(), &addr.sin_addr) != 1) throw std::runtime_error("http: bad listen address " + host);
  if (bind(listen_fd_, reinterpret_cast<sockaddr*>(&addr), sizeof(addr)) != 0)
    throw std::runtime_error(std::string("http: bind failed: ") + strerror(errno));
  if (listen(listen_fd_, 256) != 0) throw std::runtime_error("http: listen failed");
  socklen_t len = sizeof(addr);
  getsockname(listen_fd_, reinterpret_cast<sockaddr*>(&addr), &len);
  port_ = ntohs(addr.sin_port);
  set_nonblock(listen_fd_);
  epoll_fd_ = epoll_create1(0);
  event_fd_ = eventfd(0, EFD_NONBLOCK);
  req_event_fd_ = eventfd(0, EFD_NONBLOCK);
  epoll_event ev;
  memset(&ev, 0, sizeof(ev));
  ev.events = EPOLLIN;
  ev.data.u64 = 0;  // listener
  epoll_ctl(epoll_fd_, EPOLL_CTL_ADD, listen_fd_, &ev);
  ev.data.u64 = ~0ull;  // wake
  epoll_ctl(epoll_fd_, EPOLL_CTL_ADD, event_fd_, &ev);
}

HttpServer::~HttpServer() {
  stop();
  for (auto& kv : conns_) close(kv.second.fd);
  if (listen_fd_ >= 0) close(listen_fd_);
  if (epoll_fd_ >= 0) close(epoll_fd_);
  if (event_fd_ >= 0) close(event_fd_);
  if (req_event_fd_ >= 0) close(req_event_fd_);
}

void HttpServer::start() {
  if (running_.exchange(true)) return;
  thread_ = std::thread([this] { loop(); });
}

void HttpServer::stop() {
  if (!running_.exchange(false)) return;
  wake();
  if (thread_.joinable()) thread_.join();
}

void HttpServer::wake() {
  uint64_t one = 1;
  ssize_t r = write(event_fd_, &one, sizeof(one));
  (void)r;
}

std::string HttpServer::status_line(int s) {
  const char* t = "OK";
  switch (s) {
    case 200: t = "OK"; break;
    case 400: t = "Bad Request"; break;
    case 401: t = "Unauthorized"; break;
    case 404: t = "Not Found"; break;
    case 405: t = "Method Not Allowed"; break;
    case 413: t = "Payload Too Large"; break;
    case 429: t = "Too Many Requests"; break;
    case 431: t = "Request Header Fields Too Large"; break;
    case 500: t = "Internal Server Error"; break;
    case 503: t = "Service Unavailable"; break;
  }
  return "HTTP/1.1 " + std::to_string(s) + " " + t + "\r\n";
}

void HttpServer::loop() {
  std::vector<epoll_event> evs(128);
  while (running_) {
    const int n = epoll_wait(epoll_fd_, evs.data(), static_cast<int>(evs.size()), limits_.poll_ms);
    for (int i = 0; i < n; ++i) {
      const uint64_t id = evs[i].data.u64;
      if (id == 0) { accept_new(); continue; }
      if (id == ~0ull) {
        uint64_t v;
        while (read(event_fd_, &v, sizeof(v)) > 0) {}
        continue;
      }
      if (evs[i].events & (EPOLLHUP | EPOLLERR)) { close_conn(id, true); continue; }
      if (evs[i].events & EPOLLIN) on_readable(id);
      if ((evs[i].events & EPOLLOUT) && conns_.count(id)) flush(id);
    }
    // queued answers from the service
    std::deque<Cmd> cmds;
    {
      std::lock_guard<std::mutex> lk(mu_);
      cmds.swap(cmds_);
    }
    for (const Cmd& c : cmds) apply(c);
    // keep-alive comments on idle streams
    const int64_t t = now_ms();
    for (auto& kv : conns_) {
      Conn& c = kv.second;
      if (c.streaming && c.out.empty() && t - c.last_write_ms > limits_.keepalive_comment_ms) {
        const std::string ka = ": keep-alive\n\n";
        char hdr[32];
        snprintf(hdr, sizeof(hdr), "%zx\r\n", ka.size());
        c.out += hdr + ka + "\r\n";
      }
    }
    std::vector<uint64_t> ids;
    for (auto& kv : conns_) if (!kv.second.out.empty()) ids.push_back(kv.first);
    for (uint64_t id : ids) flush(id);
  }
}

void HttpServer::accept_new() {
  for (;;) {
    const int fd = accept(listen_fd_, nullptr, nullptr);
    if (fd < 0) return;
    set_nonblock(fd);
    int one = 1;
    setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
    const uint64_t id = next_conn_++;
    Conn c;
    c.fd = fd;
    c.last_write_ms = now_ms();
    conns_[id] = c;
    epoll_event ev;
    memset(&ev, 0, sizeof(ev));
    ev.events = EPOLLIN;
    ev.data.u64 = id;
    epoll_ctl(epoll_fd_, EPOLL_CTL_ADD, fd, &ev);
  }
}

void HttpServer::close_conn(uint64_t id, bool notify) {
  auto it = conns_.find(id);
  if (it == conns_.end()) return;
  const bool was_busy = it->second.busy;
  epoll_ctl(epoll_fd_, EPOLL_CTL_DEL, it->second.fd, nullptr);
  close(it->second.fd);
  conns_.erase(it);
  if (notify && was_busy) {
    std::lock_guard<std::mutex> lk(mu_);
    disconnects_.push_back(id);
    uint64_t one = 1;
    ssize_t r = write(req_event_fd_, &one, sizeof(one));
    (void)r;
  }
}

void HttpServer::on_readable(uint64_t id) {
  auto it = conns_.find(id);
  if (it == conns_.end()) return;
  char buf[65536];
  for (;;) {
    const ssize_t n = read(it->second.fd, buf, sizeof(buf));
    if (n > 0) {
      it->second.in.append(buf, static_cast<size_t>(n));
      if (it->second.in.size() > limits_.max_header_bytes + limits_.max_body_bytes + 4) break;
      continue;
    }
    if (n == 0) { close_conn(id, true); return; }
    if (errno == EAGAIN || errno == EWOULDBLOCK) break;
    close_conn(id, true);
    return;
  }
  try_parse(id);
}

void HttpServer::send_error(uint64_t id, int status, const std::string& msg) {
  const std::string body = "{\"error\":{\"message\":\"" + msg + "\",\"type\":\"invalid_request_error\"}}";
  Conn& c = conns_[id];
  c.out += status_line(status) + "Content-Type: application/json\r\nContent-Length: " + std::to_string(body.size()) +
           "\r\nConnection: close\r\n\r\n" + body;
  c.close_after = true;
  flush(id);
}

void HttpServer::try_parse(uint64_t id) {
  auto it = conns_.find(id);
  if (it == conns_.end()) return;
  Conn& c = it->second;
  if (c.busy) return;  // one request at a time per connection
  const size_t he = c.in.find("\r\n\r\n");
  if (he == std::string::npos) {
    if (c.in.size() > limits_.max_header_bytes) send_error(id, 431, "request headers exceed the limit");
    return;
  }
  if (he + 4 > limits_.max_header_bytes) { send_error(id, 431, "request headers exceed the limit"); return; }
  HttpRequest req;
  req.conn = id;
  size_t pos = c.in.find("\r\n");
  {
    const std::string line = c.in.substr(0, pos);
    const size_t s1 = line.find(' '), s2 = line.rfind(' ');
    if (s1 == std::string::npos || s2 == s1) { send_error(id, 400, "malformed request line"); return; }
    req.method = line.substr(0, s1);
    std::string target = line.substr(s1 + 1, s2 - s1 - 1);
    const size_t q = target.find('?');
    req.path = target.substr(0, q);
    if (q != std::string::npos) req.query = target.substr(q + 1);
  }
  pos += 2;
  while (pos < he) {
    size_t e = c.in.find("\r\n", pos);
    if (e == std::string::npos || e > he) e = he;
    const std::string line = c.in.substr(pos, e - pos);
    const size_t colon = line.find(':');
    if (colon != std::string::npos) {
      std::string k = line.substr(0, colon), v = line.substr(colon + 1);
      std::transform(k.begin(), k.end(), k.begin(), [](unsigned char ch) { return static_cast<char>(tolower(ch)); });
      while (!v.empty() && (v.front() == ' ' || v.front() == '\t')) v.erase(v.begin());
      while (!v.empty() && (v.back() == ' ' || v.back() == '\t')) v.pop_back();
      req.headers[k] = v;
    }
    pos = e + 2;
  }
  size_t clen = 0;
  auto cl = req.headers.find("content-length");
  if (cl != req.headers.end()) {
    char* end = nullptr;
    const unsigned long long v = strtoull(cl->second.c_str(), &end, 10);
    if (!end || *end) { send_error(id, 400, "bad Content-Length"); return; }
    clen = static_cast<size_t>(v);
  } else if (req.headers.count("transfer-encoding")) {
    send_error(id, 400, "chunked request bodies are not supported");
    return;
  }
  if (clen > limits_.max_body_bytes) { send_error(id, 413, "request body exceeds the limit"); return; }
  if (c.in.size() < he + 4 + clen) return;  // wait for the rest of the body
  req.body = c.in.substr(he + 4, clen);
  c.in.erase(0, he + 4 + clen);
  auto conn_hdr = req.headers.find("connection");
  c.want_close = conn_hdr != req.headers.end() && conn_hdr->second == "close";
  c.busy = true;
  {
    std::lock_guard<std::mutex> lk(mu_);
    requests_.push_back(std::move(req));
  }
  uint64_t one = 1;
  ssize_t r = write(req_event_fd_, &one, sizeof(one));
  (void)r;
}

void HttpServer::flush(uint64_t id) {
  auto it = conns_.find(id);
  if (it == conns_.end()) return;
  Conn& c = it->second;
  while (!c.out.empty()) {
    const ssize_t n = send(c.fd, c.out.data(), c.out.size(), MSG_NOSIGNAL);
    if (n > 0) {
      c.out.erase(0, static_cast<size_t>(n));
      c.last_write_ms = now_ms();
      continue;
    }
    if (errno == EAGAIN || errno == EWOULDBLOCK) break;
    close_conn(id, true);
    return;
  }
  epoll_event ev;
  memset(&ev, 0, sizeof(ev));
  ev.events = EPOLLIN | (c.out.empty() ? 0 : EPOLLOUT);
  ev.data.u64 = id;
  epoll_ctl(epoll_fd_, EPOLL_CTL_MOD, c.fd, &ev);
  if (c.out.empty() && c.close_after) close_conn(id, false);
}

void HttpServer::apply(const Cmd& cmd) {
  auto it = conns_.find(cmd.conn);
  if (it == conns_.end()) return;
  Conn& c = it->second;
  switch (cmd.kind) {
    case 0:
      c.out += cmd.data;
      c.busy = false;
      if (c.want_close) c.close_after = true;
      break;
    case 1:
      c.out += cmd.data;
      c.streaming = true;
      break;
    case 2: {
      char hdr[32];
      snprintf(hdr, sizeof(hdr), "%zx\r\n", cmd.data.size());
      c.out += hdr + cmd.data + "\r\n";
      break;
    }
    case 3:
      c.out += "0\r\n\r\n";
      c.streaming = false;
      c.busy = false;
      if (c.want_close) c.close_after = true;
      break;
  }
  flush(cmd.conn);
  if (conns_.count(cmd.conn) && !conns_[cmd.conn].busy) try_parse(cmd.conn);  // pipelined next request
}

// ------------------------------------------------------------------ service side
std::vector<HttpRequest> HttpServer::poll(int timeout_ms) {
  {
    std::lock_guard<std::mutex> lk(mu_);
    if (!requests_.empty() || !disconnects_.empty() || timeout_ms <= 0) {
      std::vector<HttpRequest> out(requests_.begin(), requests_.end());
      requests_.clear();
      return out;
    }
  }
  pollfd pfd;
  pfd.fd = req_event_fd_;
  pfd.events = POLLIN;
  ::poll(&pfd, 1, timeout_ms);
  uint64_t v;
  while (read(req_event_fd_, &v, sizeof(v)) > 0) {}
  std::lock_guard<std::mutex> lk(mu_);
  std::vector<HttpRequest> out(requests_.begin(), requests_.end());
  requests_.clear();
  return out;
}

std::vector<uint64_t> HttpServer::poll_disconnects() {
  std::lock_guard<std::mutex> lk(mu_);
  std::vector<uint64_t> out(disconnects_.begin(), disconnects_.end());
  disconnects_.clear();
  return out;
}

void HttpServer::respond(uint64_t conn, int status, const std::string& content_type, const std::string& body,
                         const std::vector<std::pair<std::string, std::string>>& extra) {
  std::string h = status_line(status) + "Content-Type: " + content_type + "\r\nContent-Length: " +
                  std::to_string(body.size()) + "\r\n";
  for (const auto& kv : extra) h += kv.first + ": " + kv.second + "\r\n";
  h += "\r\n";
  {
    std::lock_guard<std::mutex> lk(mu_);
    cmds_.push_back({conn, 0, h + body});
  }
  wake();
}

void HttpServer::stream_begin(uint64_t conn, const std::string& content_type) {
  const std::string h = status_line(200) + "Content-Type: " + content_type +
                        "\r\nCache-Control: no-cache\r\nTransfer-Encoding: chunked\r\n\r\n";
  {
    std::lock_guard<std::mutex> lk(mu_);
    cmds_.push_back({conn, 1, h});
  }
  wake();
}

void HttpServer::stream_send(uint64_t conn, const std::string& data) {
  if (data.empty()) return;
  {
    std::lock_guard<std::mutex> lk(mu_);
    cmds_.push_back({conn, 2, data});
  }
  wake();
}

void HttpServer::stream_end(uint64_t conn) {
  {
    std::lock_guard<std::mutex> lk(mu_);
    cmds_.push_back({conn, 3, ""});
  }
  wake();
}

}  // namespace dgpp
