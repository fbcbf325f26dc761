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

#include <algorithm>
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
  bool grpc = false;                                     // OTLP/gRPC (h2c) instead of OTLP/HTTP JSON
};
// "http://host:port/path" speaks HTTP/1.1; "grpc://host:port" speaks gRPC over clear-text HTTP/2, and so does an http:// URL
// on 4317, the port collectors reserve for OTLP/gRPC.
inline Url parse_url(const std::string& u) {
  Url r;
  std::string pre = "http://";
  if (u.compare(0, 7, "grpc://") == 0) { pre = "grpc://"; r.grpc = true; r.port = 4317; }
  else if (u.compare(0, pre.size(), pre) != 0) return r;  // no TLS: collectors and log sinks on the cluster network
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
  if (r.port == 4317) r.grpc = true;
  return r;
}

inline int connect_tcp(const Url& url, int timeout_ms) {
  addrinfo hints{}, *res = nullptr;
  hints.ai_family = AF_UNSPEC;
  hints.ai_socktype = SOCK_STREAM;
  if (getaddrinfo(url.host.c_str(), std::to_string(url.port).c_str(), &hints, &res) != 0 || !res) return -1;
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
  return fd;
}
inline bool send_all(int fd, const std::string& b) {
  size_t off = 0;
  while (off < b.size()) {
    ssize_t w = ::send(fd, b.data() + off, b.size() - off, MSG_NOSIGNAL);
    if (w <= 0) return false;
    off += (size_t)w;
  }
  return true;
}
inline bool recv_exact(int fd, char* dst, size_t n) {
  size_t off = 0;
  while (off < n) {
    ssize_t r = ::recv(fd, dst + off, n - off, 0);
    if (r <= 0) return false;
    off += (size_t)r;
  }
  return true;
}

// ------------------------------------------------------------------------------------------------ protobuf writer
// The few wire types OTLP's trace messages use (opentelemetry/proto/trace/v1/trace.proto).
struct Pb {
  std::string b;
  void varint(uint64_t v) { while (v >= 0x80) { b.push_back((char)(v | 0x80)); v >>= 7; } b.push_back((char)v); }
  void tag(int field, int wire) { varint(((uint64_t)field << 3) | (uint64_t)wire); }
  void bytes(int field, const std::string& v) { tag(field, 2); varint(v.size()); b += v; }
  void msg(int field, const Pb& m) { bytes(field, m.b); }
  void u64(int field, uint64_t v) { tag(field, 0); varint(v); }
  void fixed64(int field, uint64_t v) { tag(field, 1); for (int i = 0; i < 8; ++i) b.push_back((char)((v >> (8 * i)) & 0xff)); }
  void f64(int field, double d) { uint64_t v; std::memcpy(&v, &d, 8); fixed64(field, v); }
};
inline std::string unhex(const std::string& h) {
  auto nib = [](char c) { return c <= '9' ? c - '0' : c - 'a' + 10; };
  std::string o;
  for (size_t i = 0; i + 1 < h.size(); i += 2) o.push_back((char)((nib(h[i]) << 4) | nib(h[i + 1])));
  return o;
}

// ------------------------------------------------------------------------------------------------ minimal gRPC unary call
// One call per connection over clear-text HTTP/2 with prior knowledge: preface, SETTINGS, HEADERS (HPACK literals without
// indexing, no Huffman), DATA, then frames are read until the stream ends.  A unary call that succeeded answers with headers,
// one DATA frame and trailers; a refusal answers with trailers only, so "a DATA frame arrived before the stream ended" tells
// them apart without an HPACK decoder.  Returns true on success.
inline bool grpc_unary(const Url& url, const std::string& method_path, const std::string& message, int timeout_ms = 2000) {
  if (message.size() + 5 > 60000) return false;          // one flow-control window of the default size; batches here are far smaller
  int fd = connect_tcp(url, timeout_ms);
  if (fd < 0) return false;
  auto frame = [](int type, int flags, uint32_t stream, const std::string& payload) {
    std::string f;
    uint32_t n = (uint32_t)payload.size();
    f.push_back((char)(n >> 16)); f.push_back((char)(n >> 8)); f.push_back((char)n);
    f.push_back((char)type); f.push_back((char)flags);
    f.push_back((char)(stream >> 24)); f.push_back((char)(stream >> 16)); f.push_back((char)(stream >> 8)); f.push_back((char)stream);
    return f + payload;
  };
  auto lit = [](std::string& h, const std::string& name, const std::string& value) {
    auto len = [&h](size_t n) {                           // 7-bit prefix integer, Huffman bit clear
      if (n < 127) { h.push_back((char)n); return; }
      h.push_back((char)127);
      n -= 127;
      while (n >= 128) { h.push_back((char)((n & 127) | 128)); n >>= 7; }
      h.push_back((char)n);
    };
    h.push_back((char)0x00);                              // literal header field without indexing, new name
    len(name.size()); h += name;
    len(value.size()); h += value;
  };
  std::string hdr;
  lit(hdr, ":method", "POST");
  lit(hdr, ":scheme", "http");
  lit(hdr, ":path", method_path);
  lit(hdr, ":authority", url.host + ":" + std::to_string(url.port));
  lit(hdr, "content-type", "application/grpc");
  lit(hdr, "te", "trailers");
  std::string body(5, '\0');
  uint32_t n = (uint32_t)message.size();
  body[1] = (char)(n >> 24); body[2] = (char)(n >> 16); body[3] = (char)(n >> 8); body[4] = (char)n;
  body += message;
  std::string out = "PRI * HTTP/2.0\r\n\r\nSM\r\n\r\n" + frame(4, 0, 0, "") + frame(1, 0x4, 1, hdr);
  for (size_t off = 0; off < body.size(); off += 16384) {
    size_t len = std::min<size_t>(16384, body.size() - off);
    out += frame(0, off + len == body.size() ? 0x1 : 0, 1, body.substr(off, len));
  }
  bool ok = send_all(fd, out), got_data = false, done = false;
  for (int guard = 0; ok && !done && guard < 64; ++guard) {
    unsigned char h[9];
    if (!recv_exact(fd, (char*)h, 9)) { ok = false; break; }
    uint32_t len = ((uint32_t)h[0] << 16) | ((uint32_t)h[1] << 8) | h[2];
    int type = h[3], flags = h[4];
    uint32_t stream = (((uint32_t)h[5] & 0x7f) << 24) | ((uint32_t)h[6] << 16) | ((uint32_t)h[7] << 8) | h[8];
    std::string payload(len, '\0');
    if (len > (1u << 20) || (len && !recv_exact(fd, &payload[0], len))) { ok = false; break; }
    if (type == 4 && !(flags & 0x1)) ok = send_all(fd, frame(4, 0x1, 0, ""));          // SETTINGS -> ACK
    else if (type == 6 && !(flags & 0x1)) ok = send_all(fd, frame(6, 0x1, 0, payload)); // PING -> ACK
    else if (type == 3 || type == 7) ok = false;                                        // RST_STREAM, GOAWAY
    else if (type == 0 && stream == 1) { got_data = got_data || len >= 5; done = flags & 0x1; }
    else if (type == 1 && stream == 1) done = flags & 0x1;                              // trailers end the stream
  }
  ::close(fd);
  return ok && done && got_data;
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
  bool grpc() const { return url_.grpc; }
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
        if (url_.grpc) {
          ok = grpc_unary(url_, "/opentelemetry.proto.collector.trace.v1.TraceService/Export", body);
        } else {
          int st = http_post(url_, path_, body, "application/json");
          ok = st >= 200 && st < 300;
        }
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

// The same span as an opentelemetry.proto.trace.v1.Span message.
inline Pb otlp_any_pb(const json::Value& v) {
  Pb a;                                                    // AnyValue: string 1, bool 2, int 3, double 4
  if (v.is_string()) a.bytes(1, v.as_string());
  else if (v.is_bool()) a.u64(2, v.as_bool() ? 1 : 0);
  else if (v.is_number() && v.as_double() == (double)(long long)v.as_double()) a.u64(3, (uint64_t)(long long)v.as_double());
  else if (v.is_number()) a.f64(4, v.as_double());
  else a.bytes(1, v.dump());
  return a;
}
inline Pb otlp_kv_pb(const std::string& k, const json::Value& v) {
  Pb kv;
  kv.bytes(1, k);
  kv.msg(2, otlp_any_pb(v));
  return kv;
}
inline Pb otlp_span_pb(const Span& s) {
  Pb o;
  o.bytes(1, unhex(s.ctx.trace_id));
  o.bytes(2, unhex(s.ctx.span_id));
  if (!s.parent_span_id.empty()) o.bytes(4, unhex(s.parent_span_id));
  o.bytes(5, s.name);
  o.u64(6, (uint64_t)s.kind);
  o.fixed64(7, s.start_ns);
  o.fixed64(8, s.end_ns);
  for (auto& kv : s.attrs) o.msg(9, otlp_kv_pb(kv.first, kv.second));
  for (auto& l : s.links) {
    Pb x;
    x.bytes(1, unhex(l.trace_id));
    x.bytes(2, unhex(l.span_id));
    o.msg(13, x);
  }
  if (s.error) {
    Pb st;
    st.bytes(2, s.error_message);
    st.u64(3, 2);
    o.msg(15, st);
  }
  return o;
}
// ExportTraceServiceRequest { resource_spans { resource { attributes }, scope_spans { scope { name }, spans } } }
inline std::string otlp_request_pb(const std::string& service, const std::vector<Span>& batch, size_t begin, size_t end) {
  Pb scope_spans, scope, resource, rs, root;
  scope.bytes(1, "lorax_b200");
  scope_spans.msg(1, scope);
  for (size_t i = begin; i < end; ++i) scope_spans.msg(2, otlp_span_pb(batch[i]));
  resource.msg(1, otlp_kv_pb("service.name", json::Value(service)));
  rs.msg(1, resource);
  rs.msg(2, scope_spans);
  root.msg(1, rs);
  return root.b;
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
    if (poster_.grpc()) {                                  // OTLP/gRPC: protobuf, at most 32 spans per call
      for (size_t i = 0; i < batch.size(); i += 32) poster_.post(otlp_request_pb(service_, batch, i, std::min(batch.size(), i + 32)));
      g.lock();
      return;
    }
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
