// HTTP/1.1 server with keep-alive, chunked responses and server-sent events.  One thread per connection
// (requests are long lived while tokens stream).  The reference uses axum/hyper (router/src/server.rs); no HTTP
// library is available here, and the subset needed is small: request line, headers, Content-Length bodies.
#pragma once
#include <arpa/inet.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <cstring>
#include <functional>
#include <map>
#include <cstdio>
#include <string>
#include <thread>
#include <vector>

namespace http {

struct Request {
  std::string method, path, query, body;
  std::map<std::string, std::string> headers;      // lower-cased names
  std::string header(const std::string& name) const {
    auto it = headers.find(name);
    return it == headers.end() ? std::string() : it->second;
  }
  std::string query_param(const std::string& name) const {
    size_t pos = 0;
    while (pos < query.size()) {
      size_t amp = query.find('&', pos);
      std::string kv = query.substr(pos, amp == std::string::npos ? std::string::npos : amp - pos);
      size_t eq = kv.find('=');
      if (kv.substr(0, eq) == name) return eq == std::string::npos ? "" : kv.substr(eq + 1);
      if (amp == std::string::npos) break;
      pos = amp + 1;
    }
    return "";
  }
};

class ResponseWriter {
 public:
  explicit ResponseWriter(int fd) : fd_(fd) {}
  using Headers = std::vector<std::pair<std::string, std::string>>;

  bool send(int status, const std::string& body, const std::string& content_type = "application/json", const Headers& extra = {}) {
    std::string h = "HTTP/1.1 " + std::to_string(status) + " " + reason(status) + "\r\nContent-Type: " + content_type +
                    "\r\nContent-Length: " + std::to_string(body.size()) + "\r\n";
    for (auto& kv : extra) h += kv.first + ": " + kv.second + "\r\n";
    for (auto& kv : common_) h += kv.first + ": " + kv.second + "\r\n";
    h += "\r\n";
    started_ = true;
    return write_all(h + body);
  }
  // Server-sent events over a chunked response.
  bool begin_stream(int status = 200, const Headers& extra = {}) {
    std::string h = "HTTP/1.1 " + std::to_string(status) + " " + reason(status) +
                    "\r\nContent-Type: text/event-stream\r\nCache-Control: no-cache\r\nTransfer-Encoding: chunked\r\n";
    for (auto& kv : extra) h += kv.first + ": " + kv.second + "\r\n";
    for (auto& kv : common_) h += kv.first + ": " + kv.second + "\r\n";
    h += "\r\n";
    started_ = streaming_ = true;
    return write_all(h);
  }
  bool event(const std::string& data) { return chunk("data:" + data + "\n\n"); }
  bool chunk(const std::string& payload) {
    char len[24];
    snprintf(len, sizeof len, "%zx\r\n", payload.size());
    return write_all(std::string(len) + payload + "\r\n");
  }
  bool end_stream() { streaming_ = false; return write_all("0\r\n\r\n"); }
  bool started() const { return started_; }
  bool streaming() const { return streaming_; }
  // True when the peer closed the connection (used to cancel generation for disconnected clients).
  bool peer_closed() const {
    pollfd p{fd_, POLLIN | POLLRDHUP, 0};
    if (::poll(&p, 1, 0) <= 0) return false;
    if (p.revents & (POLLRDHUP | POLLHUP | POLLERR)) return true;
    char c;
    return (p.revents & POLLIN) && ::recv(fd_, &c, 1, MSG_PEEK | MSG_DONTWAIT) == 0;
  }
  void add_common(const std::string& k, const std::string& v) { common_.push_back({k, v}); }

  static const char* reason(int s) {
    switch (s) {
      case 200: return "OK"; case 204: return "No Content"; case 400: return "Bad Request"; case 401: return "Unauthorized";
      case 404: return "Not Found"; case 405: return "Method Not Allowed"; case 413: return "Payload Too Large";
      case 422: return "Unprocessable Entity"; case 424: return "Failed Dependency"; case 429: return "Too Many Requests";
      case 500: return "Internal Server Error"; case 503: return "Service Unavailable"; default: return "Status";
    }
  }

 private:
  bool write_all(const std::string& s) {
    const char* p = s.data();
    size_t n = s.size();
    while (n) {
      ssize_t w = ::send(fd_, p, n, MSG_NOSIGNAL);
      if (w <= 0) { if (w < 0 && errno == EINTR) continue; return false; }
      p += w; n -= (size_t)w;
    }
    return true;
  }
  int fd_;
  bool started_ = false, streaming_ = false;
  Headers common_;
};

using Handler = std::function<void(const Request&, ResponseWriter&)>;

class Server {
 public:
  void route(const std::string& method, const std::string& path, Handler h) { routes_[method + " " + path] = std::move(h); }
  void set_cors(const std::vector<std::string>& origins) { cors_ = origins; }
  // Values of the other CORS response headers (comma separated lists as given on the command line; empty: the defaults).
  void set_cors_options(std::string methods, std::string headers, std::string expose, bool credentials) {
    cors_methods_ = methods.empty() ? "GET, POST, OPTIONS" : std::move(methods);
    cors_headers_ = headers.empty() ? "*" : std::move(headers);
    cors_expose_ = std::move(expose);
    cors_credentials_ = credentials;
  }
  size_t max_body = 256u << 20;

  // Returns the bound port (0 on failure).  Serves until stop().
  int listen_and_serve(const std::string& host, int port) {
    int fd = ::socket(AF_INET, SOCK_STREAM, 0);
    if (fd < 0) return 0;
    int one = 1;
    setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof one);
    sockaddr_in addr{};
    addr.sin_family = AF_INET;
    addr.sin_port = htons((uint16_t)port);
    if (host.empty() || host == "0.0.0.0") addr.sin_addr.s_addr = INADDR_ANY;
    else inet_pton(AF_INET, host.c_str(), &addr.sin_addr);
    if (::bind(fd, (sockaddr*)&addr, sizeof addr) != 0 || ::listen(fd, 1024) != 0) { ::close(fd); return 0; }
    socklen_t len = sizeof addr;
    getsockname(fd, (sockaddr*)&addr, &len);
    listen_fd_ = fd;
    bound_port_ = ntohs(addr.sin_port);
    running_ = true;
    accept_thread_ = std::thread([this] { accept_loop(); });
    return bound_port_;
  }
  void stop() {
    if (!running_.exchange(false)) return;
    ::shutdown(listen_fd_, SHUT_RDWR);
    ::close(listen_fd_);
    if (accept_thread_.joinable()) accept_thread_.join();
    // in-flight connections finish on their own; wait a bounded time (graceful shutdown)
    for (int i = 0; i < 300 && active_ > 0; ++i) std::this_thread::sleep_for(std::chrono::milliseconds(10));
  }
  int port() const { return bound_port_; }

 private:
  void accept_loop() {
    while (running_) {
      int c = ::accept(listen_fd_, nullptr, nullptr);
      if (c < 0) { if (!running_) break; continue; }
      int one = 1;
      setsockopt(c, IPPROTO_TCP, TCP_NODELAY, &one, sizeof one);
      active_++;
      std::thread([this, c] { serve(c); ::close(c); active_--; }).detach();
    }
  }
  static std::string lower(std::string s) { std::transform(s.begin(), s.end(), s.begin(), ::tolower); return s; }

  void serve(int fd) {
    std::string buf;
    while (running_) {
      // ---- read the header block
      size_t hdr_end;
      while ((hdr_end = buf.find("\r\n\r\n")) == std::string::npos) {
        char tmp[8192];
        pollfd p{fd, POLLIN, 0};
        int pr = ::poll(&p, 1, 75000);            // keep-alive timeout
        if (pr <= 0) return;
        ssize_t r = ::recv(fd, tmp, sizeof tmp, 0);
        if (r <= 0) return;
        buf.append(tmp, (size_t)r);
        if (buf.size() > (1u << 20) && buf.find("\r\n\r\n") == std::string::npos) return;
      }
      Request req;
      {
        size_t line_end = buf.find("\r\n");
        std::string line = buf.substr(0, line_end);
        size_t s1 = line.find(' '), s2 = line.rfind(' ');
        if (s1 == std::string::npos || s2 == s1) return;
        req.method = line.substr(0, s1);
        std::string target = line.substr(s1 + 1, s2 - s1 - 1);
        size_t q = target.find('?');
        req.path = target.substr(0, q);
        if (q != std::string::npos) req.query = target.substr(q + 1);
        size_t pos = line_end + 2;
        while (pos < hdr_end) {
          size_t e = buf.find("\r\n", pos);
          std::string h = buf.substr(pos, e - pos);
          size_t colon = h.find(':');
          if (colon != std::string::npos) {
            std::string v = h.substr(colon + 1);
            v.erase(0, v.find_first_not_of(" \t"));
            req.headers[lower(h.substr(0, colon))] = v;
          }
          pos = e + 2;
        }
      }
      size_t body_len = 0;
      if (!req.header("content-length").empty()) body_len = (size_t)strtoull(req.header("content-length").c_str(), nullptr, 10);
      ResponseWriter w(fd);
      add_cors(req, w);
      if (body_len > max_body) { w.send(413, "{\"error\":\"payload too large\",\"error_type\":\"validation\"}"); return; }
      size_t have = buf.size() - (hdr_end + 4);
      while (have < body_len) {
        char tmp[65536];
        ssize_t r = ::recv(fd, tmp, sizeof tmp, 0);
        if (r <= 0) return;
        buf.append(tmp, (size_t)r);
        have += (size_t)r;
      }
      req.body = buf.substr(hdr_end + 4, body_len);
      buf.erase(0, hdr_end + 4 + body_len);

      if (req.method == "OPTIONS") {
        w.send(204, "", "text/plain", {{"Access-Control-Allow-Methods", cors_methods_}, {"Access-Control-Allow-Headers", cors_headers_}});
      } else {
        auto it = routes_.find(req.method + " " + req.path);
        if (it == routes_.end()) {
          bool path_known = false;
          for (auto& kv : routes_) if (kv.first.substr(kv.first.find(' ') + 1) == req.path) path_known = true;
          w.send(path_known ? 405 : 404, path_known ? "{\"error\":\"method not allowed\"}" : "{\"error\":\"not found\"}");
        } else {
          try {
            it->second(req, w);
          } catch (const std::exception& ex) {
            if (!w.started()) {
              std::string msg;                     // the message as a JSON string
              for (unsigned char ch : std::string(ex.what())) {
                if (ch == '"' || ch == '\\') { msg.push_back('\\'); msg.push_back((char)ch); }
                else if (ch < 0x20) { char buf[8]; std::snprintf(buf, sizeof buf, "\\u%04x", ch); msg += buf; }
                else msg.push_back((char)ch);
              }
              w.send(500, "{\"error\":\"" + msg + "\",\"error_type\":\"internal\"}");
            }
          }
          if (w.streaming()) w.end_stream();
        }
      }
      if (lower(req.header("connection")) == "close") return;
    }
  }
  void add_cors(const Request& req, ResponseWriter& w) {
    if (cors_.empty()) return;
    std::string origin = req.header("origin");
    for (auto& o : cors_) {
      if (o == "*" || o == origin) {
        // a wildcard origin may not be combined with credentials: echo the caller's origin then
        w.add_common("Access-Control-Allow-Origin", o == "*" && !(cors_credentials_ && !origin.empty()) ? "*" : origin);
        if (cors_credentials_) w.add_common("Access-Control-Allow-Credentials", "true");
        if (!cors_expose_.empty()) w.add_common("Access-Control-Expose-Headers", cors_expose_);
        break;
      }
    }
  }
  std::map<std::string, Handler> routes_;
  std::vector<std::string> cors_;
  std::string cors_methods_ = "GET, POST, OPTIONS", cors_headers_ = "*", cors_expose_;
  bool cors_credentials_ = false;
  int listen_fd_ = -1, bound_port_ = 0;
  std::atomic<bool> running_{false};
  std::atomic<int> active_{0};
  std::thread accept_thread_;
};

}  // namespace http
