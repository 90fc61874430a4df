// Single-threaded epoll HTTP/1.1 server with server-sent-event streaming.
//
// The loop thread only does socket work: it parses requests (request line + headers <= 16 KiB, body <=
// 256 MiB by default, Content-Length bodies, keep-alive) and puts them on a queue; the service thread takes
// them with poll(), and answers from any thread with respond() / stream_begin() + stream_send() + stream_end().
// Answers are queued and the loop is woken through an eventfd, so no other thread ever touches a socket.
// Streams get `: keep-alive` comments when idle; a client that disconnects shows up in poll_disconnects() so
// the service can cancel the request.
// (behavioural spec: src/serve/http_server.cpp, http_limits.hpp of the reference -- single epoll thread,
//  eventfd wake, 16 KiB / 256 MiB limits, chunked SSE.)
#pragma once
#include <atomic>
#include <cstdint>
#include <deque>
#include <map>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

namespace dgpp {

struct HttpLimits {
  size_t max_header_bytes = 16 * 1024;
  size_t max_body_bytes = 256ull * 1024 * 1024;
  int keepalive_comment_ms = 30000;
  int poll_ms = 25;
};

struct HttpRequest {
  uint64_t conn = 0;
  std::string method, path, query, body;
  std::map<std::string, std::string> headers;  // lower-case names
};

class HttpServer {
 public:
  HttpServer(const std::string& host, int port, HttpLimits limits = HttpLimits());
  ~HttpServer();
  void start();
  void stop();
  int port() const { return port_; }

  // service side (any thread)
  std::vector<HttpRequest> poll(int timeout_ms);
  std::vector<uint64_t> poll_disconnects();
  void respond(uint64_t conn, int status, const std::string& content_type, const std::string& body,
               const std::vector<std::pair<std::string, std::string>>& extra_headers = {});
  void stream_begin(uint64_t conn, const std::string& content_type = "text/event-stream");
  void stream_send(uint64_t conn, const std::string& data);  // raw bytes of the stream (e.g. "data: {...}\n\n")
  void stream_end(uint64_t conn);

 private:
  struct Conn {
    int fd = -1;
    std::string in, out;
    bool streaming = false, close_after = false, busy = false, want_close = false;
    int64_t last_write_ms = 0;
  };
  struct Cmd {
    uint64_t conn;
    int kind;  // 0 respond bytes, 1 stream begin, 2 stream data, 3 stream end
    std::string data;
  };
  void loop();
  void accept_new();
  void on_readable(uint64_t id);
  void try_parse(uint64_t id);
  void flush(uint64_t id);
  void close_conn(uint64_t id, bool notify);
  void apply(const Cmd& c);
  void wake();
  void send_error(uint64_t id, int status, const std::string& msg);
  static std::string status_line(int status);

  std::string host_;
  int port_;
  HttpLimits limits_;
  int listen_fd_ = -1, epoll_fd_ = -1, event_fd_ = -1;
  std::thread thread_;
  std::atomic<bool> running_{false};
  std::unordered_map<uint64_t, Conn> conns_;
  std::unordered_map<int, uint64_t> fd_to_conn_;
  uint64_t next_conn_ = 1;
  std::mutex mu_;
  std::deque<HttpRequest> requests_;
  std::deque<uint64_t> disconnects_;
  std::deque<Cmd> cmds_;
  int req_event_fd_ = -1;
};

}  // namespace dgpp
