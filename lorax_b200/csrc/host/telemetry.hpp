// Request tracing and the request-logger webhook of the router.
//
// Tracing follows the reference's OpenTelemetry set-up (router/src/main.rs:492-541, spans with recorded fields
// server.rs:632-643, batch spans linked to request spans infer.rs:1173-1184, context carried to the shards
// router/grpc-metadata/src/lib.rs:45-63) with two differences of mechanism: spans leave as OTLP/HTTP JSON
// (`POST {endpoint}/v1/traces`, the collector's 4318 port) instead of OTLP/gRPC, and the context travels to the shards as
// a W3C `traceparent` string in front of the framed payload instead of gRPC metadata.
//
//   request span   one per HTTP request, child of the caller's `traceparent` header when there is one; attributes:
//                  total / validation / queue / inference time, prompt and generated tokens, seed, adapter id
//   batch spans    one per Prefill / Decode call of the batching loop, in the trace of the loop, with links to the
//                  request spans whose entries are in the batch; the shards' spans are their children
//
// The request logger (server.rs:1314-1349): when REQUEST_LOGGER_URL is set every finished request is posted there as JSON
// (input, output, token counts, adapter, status), three attempts, from a background thread.
#pragma once
#include <arpa/inet.h>
#include <netdb.h>
#include <sys/socket.h>
#include <sys/time.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstring>
#include <deque>
#include <mutex>
#include <random>
#include <string>
#include <thread>
#include <vector>

#include "json.hpp"

namespace lx::telemetry {

// ------------------------------------------------------------------------------------------------ minimal HTTP/1.1 POST
struct Url {
  std::string host, path = "/";
  int port = 80;
  bool ok = false;
};
inline Url parse_url(const std::string& u) {
  Url r;
  const std::string pre = "http://";
  if (u.compare(0, pre.size(), pre) != 0) return r;      // plain HTTP only: collectors and log sinks on the cluster network
  size_t p = pre.size(), slash = u.find('/', p);
  std::string hp = u.substr(p, slash == std::string::npos ? std::string::npos : slash - p);
  if (slash != std::string::npos) r.path = u.substr(slash);
  size_t colon = hp.rfind(':');
  if (colon != std::string::npos) {
    r.host = hp.substr(0, colon);
    r.port = std::atoi(hp.c_str() + colon + 1);
  } else {
    r.host = hp;
  }
  r.ok = !r.host.empty() && r.port > 0;
  return r;
}

// Blocking POST with a timeout on every socket operation.  Returns the HTTP status, or 0 when the peer could not be reached.
inline int http_post(const Url& url, const std::string& path, const std::string& body, const std::string& content_type, int timeout_ms = 2000) {
  addrinfo hints{}, *res = nullptr;
  hints.ai_family = AF_UNSPEC;
  hints.ai_socktype = SOCK_STREAM;
  if (getaddrinfo(url.host.c_str(), std::to_string(url.port).c_str(), &hints, &res) != 0 || !res) return 0;
  int fd = -1;
  for (addrinfo* a = res; a; a = a->ai_next) {
    fd = ::socket(a->ai_family, a->ai_socktype, a->ai_protocol);
    if (fd < 0) continue;
    timeval tv{timeout_ms / 1000, (timeout_ms % 1000) * 1000};
    setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof tv);
    setsockopt(fd, SOL_SOCKET, SO_SNDTIMEO, &tv, sizeof tv);
    if (::connect(fd, a->ai_addr, a->ai_addrlen) == 0) break;
    ::close(fd);
    fd = -1;
  }
  freeaddrinfo(res);
  if (fd < 0) return 0;
  std::string req = "POST " + path + " HTTP/1.1\r\nHost: " + url.host + ":" + std::to_string(url.port) + "\r\nContent-Type: " + content_type +
                    "\r\nContent-Length: " + std::to_string(body.size()) + "\r\nConnection: close\r\n\r\n" + body;
  size_t off = 0;
  while (off < req.size()) {
    ssize_t w = ::send(fd, req.data() + off, req.size() - off, MSG_NOSIGNAL);
    if (w <= 0) { ::close(fd); return 0; }
    off += (size_t)w;
  }
  char buf[256];
  ssize_t n = ::recv(fd, buf, sizeof buf - 1, 0);
  ::close(fd);
  if (n < 12) return 0;
  buf[n] = 0;
  return std::atoi(buf + 9);                             // "HTTP/1.1 200 ..."
}

// Posts queued bodies from one background thread; a body is dropped after `attempts` failures or when the queue is full.
class BackgroundPoster {
 public:
  BackgroundPoster(Url url, std::string path, int attempts = 3) : url_(std::move(url)), path_(std::move(path)), attempts_(attempts) {
    if (url_.ok) worker_ = std::thread([this] { loop(); });
  }
  ~BackgroundPoster() { stop(); }
  bool enabled() const { return url_.ok; }
  void post(std::string body) {
    if (!url_.ok) return;
    std::lock_guard<std::mutex> g(mu_);
    if (q_.size() >= 4096) { ++dropped_; return; }
    q_.push_back(std::move(body));
    cv_.notify_one();
  }
  void stop() {
    { std::lock_guard<std::mutex> g(mu_); if (stop_) return; stop_ = true; cv_.notify_all(); }
    if (worker_.joinable()) worker_.join();
  }
  size_t sent() const { return sent_; }
  size_t dropped() const { return dropped_; }

 private:
  void loop() {
    while (true) {
      std::string body;
      {
        std::unique_lock<std::mutex> g(mu_);
        cv_.wait(g, [this] { return stop_ || !q_.empty(); });
        if (q_.empty()) return;                           // stop requested and everything flushed
        body = std::move(q_.front());
        q_.pop_front();
      }
      bool ok = false;
      for (int a = 0; a < attempts_ && !ok; ++a) {
        int st = http_post(url_, path_, body, "application/json");
        ok = st >= 200 && st < 300;
        if (!ok && a + 1 < attempts_) std::this_thread::sleep_for(std::chrono::milliseconds(100 << a));
      }
      if (ok) ++sent_; else ++dropped_;
    }
  }
  Url url_;
  std::string path_;
  int attempts_;
  std::thread worker_;
  std::mutex mu_;
  std::condition_variable cv_;
  std::deque<std::string> q_;
  bool stop_ = false;
  std::atomic<size_t> sent_{0}, dropped_{0};
};

// ------------------------------------------------------------------------------------------------ trace context
struct SpanContext {
  std::string trace_id, span_id;                          // 32 and 16 lower-case hex digits
  bool valid() const { return trace_id.size() == 32 && span_id.size() == 16; }
};
inline std::string random_hex(int nbytes) {
  static thread_local std::mt19937_64 rng{std::random_device{}() ^ (uint64_t)std::chrono::steady_clock::now().time_since_epoch().count()};
  static const char* d = "0123456789abcdef";
  std::string s;
  while ((int)s.size() < 2 * nbytes) {
    uint64_t v = rng();
    for (int i = 0; i < 16 && (int)s.size() < 2 * nbytes; ++i, v >>= 4) s.push_back(d[v & 15]);
  }
  return s;
}
// "00-<32 hex>-<16 hex>-<2 hex>"
inline SpanContext parse_traceparent(const std::string& h) {
  SpanContext c;
  if (h.size() != 55 || h[2] != '-' || h[35] != '-' || h[52] != '-') return c;
  auto hex = [](const std::string& s) { for (char ch : s) if (!((ch >= '0' && ch <= '9') || (ch >= 'a' && ch <= 'f'))) return false; return true; };
  std::string t = h.substr(3, 32), s = h.substr(36, 16);
  if (!hex(t) || !hex(s) || t == std::string(32, '0') || s == std::string(16, '0')) return c;
  c.trace_id = t;
  c.span_id = s;
  return c;
}
inline std::string format_traceparent(const SpanContext& c) { return c.valid() ? "00-" + c.trace_id + "-" + c.span_id + "-01" : std::string(); }

inline uint64_t unix_nanos() {
  return (uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::system_clock::now().time_since_epoch()).count();
}

struct Span {
  SpanContext ctx;
  std::string parent_span_id, name;
  uint64_t start_ns = 0, end_ns = 0;
  int kind = 1;                                            // 1 internal, 2 server, 3 client
  bool error = false;
  std::string error_message;
  std::vector<std::pair<std::string, json::Value>> attrs;
  std::vector<SpanContext> links;
  void set(const std::string& k, json::Value v) { attrs.emplace_back(k, std::move(v)); }
  bool recording() const { return ctx.valid(); }
};

inline json::Value otlp_any(const json::Value& v) {
  json::Value o = json::Value::object();
  if (v.is_string()) o.set("stringValue", v);
  else if (v.is_bool()) o.set("boolValue", v);
  else if (v.is_number() && v.as_double() == (double)(long long)v.as_double()) o.set("intValue", std::to_string((long long)v.as_double()));
  else if (v.is_number()) o.set("doubleValue", v);
  else o.set("stringValue", v.dump());
  return o;
}

inline json::Value otlp_span(const Span& s) {
  json::Value o = json::Value::object();
  o.set("traceId", s.ctx.trace_id);
  o.set("spanId", s.ctx.span_id);
  if (!s.parent_span_id.empty()) o.set("parentSpanId", s.parent_span_id);
  o.set("name", s.name);
  o.set("kind", s.kind);
  o.set("startTimeUnixNano", std::to_string(s.start_ns));
  o.set("endTimeUnixNano", std::to_string(s.end_ns));
  json::Value attrs = json::Value::array();
  for (auto& kv : s.attrs) {
    json::Value a = json::Value::object();
    a.set("key", kv.first);
    a.set("value", otlp_any(kv.second));
    attrs.push(a);
  }
  o.set("attributes", attrs);
  if (!s.links.empty()) {
    json::Value links = json::Value::array();
    for (auto& l : s.links) {
      json::Value x = json::Value::object();
      x.set("traceId", l.trace_id);
      x.set("spanId", l.span_id);
      links.push(x);
    }
    o.set("links", links);
  }
  json::Value st = json::Value::object();
  if (s.error) { st.set("code", 2); st.set("message", s.error_message); }
  o.set("status", st);
  return o;
}

// Collects finished spans and ships them in batches (every `flush_ms` or 64 spans).
class Tracer {
 public:
  Tracer(const std::string& endpoint, std::string service, int flush_ms = 500)
      : service_(std::move(service)), flush_ms_(flush_ms), poster_(parse_url(endpoint), trace_path(endpoint)) {
    if (poster_.enabled()) flusher_ = std::thread([this] { loop(); });
  }
  ~Tracer() { shutdown(); }
  bool enabled() const { return poster_.enabled(); }

  // A new span: child of `parent` when valid, else the root of a new trace.  Not recording (empty ids) when tracing is off.
  Span start(const std::string& name, const SpanContext& parent = {}, int kind = 1) const {
    Span s;
    s.name = name;
    s.kind = kind;
    if (!enabled()) return s;
    s.ctx.trace_id = parent.valid() ? parent.trace_id : random_hex(16);
    s.ctx.span_id = random_hex(8);
    if (parent.valid()) s.parent_span_id = parent.span_id;
    s.start_ns = unix_nanos();
    return s;
  }
  void end(Span& s) {
    if (!s.recording()) return;
    s.end_ns = unix_nanos();
    std::lock_guard<std::mutex> g(mu_);
    done_.push_back(std::move(s));
    if (done_.size() >= 64) cv_.notify_one();
  }
  void shutdown() {
    { std::lock_guard<std::mutex> g(mu_); if (stop_) return; stop_ = true; cv_.notify_all(); }
    if (flusher_.joinable()) flusher_.join();
    poster_.stop();
  }
  size_t exported_batches() const { return poster_.sent(); }

 private:
  static std::string trace_path(const std::string& endpoint) {
    Url u = parse_url(endpoint);
    std::string p = u.path == "/" ? "" : u.path;
    while (!p.empty() && p.back() == '/') p.pop_back();
    return p.size() >= 10 && p.compare(p.size() - 10, 10, "/v1/traces") == 0 ? p : p + "/v1/traces";
  }
  void flush_locked(std::unique_lock<std::mutex>& g) {
    if (done_.empty()) return;
    std::vector<Span> batch;
    batch.swap(done_);
    g.unlock();
    json::Value spans = json::Value::array();
    for (auto& s : batch) spans.push(otlp_span(s));
    json::Value scope = json::Value::object();
    json::Value sc = json::Value::object();
    sc.set("name", "lorax_b200");
    scope.set("scope", sc);
    scope.set("spans", spans);
    json::Value scopes = json::Value::array();
    scopes.push(scope);
    json::Value res = json::Value::object();
    json::Value rattrs = json::Value::array();
    json::Value svc = json::Value::object();
    svc.set("key", "service.name");
    svc.set("value", otlp_any(json::Value(service_)));
    rattrs.push(svc);
    json::Value resource = json::Value::object();
    resource.set("attributes", rattrs);
    res.set("resource", resource);
    res.set("scopeSpans", scopes);
    json::Value rs = json::Value::array();
    rs.push(res);
    json::Value root = json::Value::object();
    root.set("resourceSpans", rs);
    poster_.post(root.dump());
    g.lock();
  }
  void loop() {
    std::unique_lock<std::mutex> g(mu_);
    while (!stop_) {
      cv_.wait_for(g, std::chrono::milliseconds(flush_ms_));
      flush_locked(g);
    }
    flush_locked(g);
  }
  std::string service_;
  int flush_ms_;
  BackgroundPoster poster_;
  std::thread flusher_;
  std::mutex mu_;
  std::condition_variable cv_;
  std::vector<Span> done_;
  bool stop_ = false;
};

}  // namespace lx::telemetry
