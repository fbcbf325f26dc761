// gRPC (HTTP/2, clear text with prior knowledge) client of `generate.v1.LoraxService` over a Unix socket.
//
// The reference's router reaches its shards through tonic clients on `unix://{uds_path}-{rank}`
// (router/client/src/client.rs, sharded_client.rs:14-261).  The shards of this tree serve the same service with grpcio next to
// the framed socket the router uses by default; with `--shard-transport grpc` the router speaks the original contract instead.
// One connection per shard, one unary call at a time on it (the batching loop is sequential per shard), streams numbered 1, 3,
// 5, ...  What HTTP/2 needs for that is small enough to write out:
//   * preface, SETTINGS (a 2^31-1 initial stream window, so responses never wait for WINDOW_UPDATE) and a connection-level
//     WINDOW_UPDATE of the same size, topped up by the bytes of every response;
//   * request HEADERS as HPACK literals without indexing and without Huffman coding, DATA frames cut to the peer's frame size and
//     to its stream and connection windows (SETTINGS_INITIAL_WINDOW_SIZE and WINDOW_UPDATE frames are tracked);
//   * the response: HEADERS, DATA frames (one length-prefixed message), trailers.  Trailers are scanned for `grpc-status` and
//     `grpc-message` (literal strings; a Huffman-coded value is reported as undecoded), so that a shard-side exception reaches
//     the caller as text.
// The tokenizer helpers of the framed protocol are not part of the gRPC contract; `GrpcUdsClient` forwards them to the framed
// client it is given.
#pragma once

#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <algorithm>
#include <cctype>
#include <cerrno>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <mutex>
#include <string>
#include <system_error>

#include "shard_client.hpp"

namespace lx {

class GrpcUdsClient : public ShardClient {
 public:
  GrpcUdsClient(std::string path, std::shared_ptr<ShardClient> helpers = nullptr) : path_(std::move(path)), helpers_(std::move(helpers)) {}
  ~GrpcUdsClient() override { close_fd(); }

  static const char* method_name(uint32_t m) {
    switch (m) {
      case gen::M_Info: return "Info";
      case gen::M_ServiceDiscovery: return "ServiceDiscovery";
      case gen::M_ClearCache: return "ClearCache";
      case gen::M_FilterBatch: return "FilterBatch";
      case gen::M_Warmup: return "Warmup";
      case gen::M_Prefill: return "Prefill";
      case gen::M_Embed: return "Embed";
      case gen::M_Classify: return "Classify";
      case gen::M_Decode: return "Decode";
      case gen::M_Health: return "Health";
      case gen::M_DownloadAdapter: return "DownloadAdapter";
      case gen::M_LoadAdapter: return "LoadAdapter";
      case gen::M_OffloadAdapter: return "OffloadAdapter";
      default: return nullptr;
    }
  }

  std::string call(uint32_t method, const std::string& payload) override {
    std::string traceparent, body = payload;
    if (method & kTraceFlag) {                     // the router's span context travels as gRPC metadata
      method &= ~kTraceFlag;
      traceparent = payload.substr(0, 55);
      body = payload.substr(55);
    }
    const char* name = method_name(method);
    if (name == nullptr) {
      if (helpers_) return helpers_->call(method, body);
      throw ShardError("method " + std::to_string(method) + " is not part of the gRPC service");
    }
    std::lock_guard<std::mutex> g(mu_);
    for (int attempt = 0; attempt < 2; ++attempt) {
      try {
        ensure_connected();
        return unary(std::string("/generate.v1.LoraxService/") + name, body, traceparent);
      } catch (const std::system_error&) {
        close_fd();
        if (attempt == 1) throw ShardError("connection to shard " + path_ + " lost");
      }
    }
    throw ShardError("unreachable");
  }

 private:
  // ---------------------------------------------------------------- frames
  static std::string frame(int type, int flags, uint32_t stream, const std::string& payload) {
    std::string f;
    const uint32_t n = (uint32_t)payload.size();
    f.push_back((char)(n >> 16)); f.push_back((char)(n >> 8)); f.push_back((char)n);
    f.push_back((char)type); f.push_back((char)flags);
    f.push_back((char)(stream >> 24)); f.push_back((char)(stream >> 16)); f.push_back((char)(stream >> 8)); f.push_back((char)stream);
    return f + payload;
  }
  static std::string u32(uint32_t v) {
    std::string s;
    s.push_back((char)(v >> 24)); s.push_back((char)(v >> 16)); s.push_back((char)(v >> 8)); s.push_back((char)v);
    return s;
  }
  static void hpack_int(std::string& h, size_t n, int prefix_bits, int first_byte_flags) {
    const size_t cap = (1u << prefix_bits) - 1;
    if (n < cap) { h.push_back((char)(first_byte_flags | (int)n)); return; }
    h.push_back((char)(first_byte_flags | (int)cap));
    n -= cap;
    while (n >= 128) { h.push_back((char)((n & 127) | 128)); n >>= 7; }
    h.push_back((char)n);
  }
  static void literal(std::string& h, const std::string& name, const std::string& value) {
    h.push_back((char)0x00);                       // literal header field without indexing, new name
    hpack_int(h, name.size(), 7, 0);
    h += name;
    hpack_int(h, value.size(), 7, 0);
    h += value;
  }

  struct Frame {
    int type = 0, flags = 0;
    uint32_t stream = 0;
    std::string payload;
  };
  Frame read_frame() {
    unsigned char h[9];
    read_all(h, 9);
    Frame f;
    const uint32_t len = ((uint32_t)h[0] << 16) | ((uint32_t)h[1] << 8) | h[2];
    f.type = h[3];
    f.flags = h[4];
    f.stream = (((uint32_t)h[5] & 0x7f) << 24) | ((uint32_t)h[6] << 16) | ((uint32_t)h[7] << 8) | h[8];
    if (len > (1u << 24)) throw std::system_error(EPROTO, std::generic_category(), "frame size");
    f.payload.resize(len);
    if (len) read_all(&f.payload[0], len);
    return f;
  }
  // Frames that are about the connection, whoever is waiting for what.  Returns true when the frame was one of those.
  bool connection_frame(const Frame& f) {
    if (f.type == 4) {                                              // SETTINGS
      if (f.flags & 0x1) return true;
      for (size_t i = 0; i + 6 <= f.payload.size(); i += 6) {
        const unsigned char* p = (const unsigned char*)f.payload.data() + i;
        const int id = (p[0] << 8) | p[1];
        const uint32_t v = ((uint32_t)p[2] << 24) | ((uint32_t)p[3] << 16) | ((uint32_t)p[4] << 8) | p[5];
        if (id == 4) { peer_stream_window_ += (long long)v - peer_initial_window_; peer_initial_window_ = v; }
        if (id == 5 && v >= 16384) peer_max_frame_ = v;
      }
      write_str(frame(4, 0x1, 0, ""));
      return true;
    }
    if (f.type == 6) {                                              // PING
      if (!(f.flags & 0x1)) write_str(frame(6, 0x1, 0, f.payload));
      return true;
    }
    if (f.type == 8 && f.payload.size() == 4) {                     // WINDOW_UPDATE
      const unsigned char* p = (const unsigned char*)f.payload.data();
      const uint32_t inc = (((uint32_t)p[0] & 0x7f) << 24) | ((uint32_t)p[1] << 16) | ((uint32_t)p[2] << 8) | p[3];
      if (f.stream == 0) peer_conn_window_ += inc;
      else if (f.stream == stream_) peer_stream_window_ += inc;
      return true;
    }
    if (f.type == 7) throw std::system_error(ECONNRESET, std::generic_category(), "GOAWAY");
    return false;
  }

  // ---------------------------------------------------------------- one call
  std::string unary(const std::string& path, const std::string& message, const std::string& traceparent) {
    stream_ += 2;
    peer_stream_window_ = peer_initial_window_;
    std::string hdr;
    literal(hdr, ":method", "POST");
    literal(hdr, ":scheme", "http");
    literal(hdr, ":path", path);
    literal(hdr, ":authority", "localhost");
    literal(hdr, "content-type", "application/grpc");
    literal(hdr, "te", "trailers");
    if (traceparent.size() == 55) literal(hdr, "traceparent", traceparent);
    write_str(frame(1, 0x4, stream_, hdr));                        // END_HEADERS
    std::string body(5, '\0');
    const uint32_t n = (uint32_t)message.size();
    body[1] = (char)(n >> 24); body[2] = (char)(n >> 16); body[3] = (char)(n >> 8); body[4] = (char)n;
    body += message;
    size_t off = 0;
    while (off < body.size()) {
      long long room = std::min(peer_stream_window_, peer_conn_window_);
      if (room <= 0) {                                              // wait for the peer to open a window
        Frame f = read_frame();
        if (!connection_frame(f) && f.type == 3 && f.stream == stream_) throw ShardError("shard reset the stream while it received the request");
        continue;
      }
      const size_t len = (size_t)std::min<long long>({room, (long long)peer_max_frame_, (long long)(body.size() - off)});
      const bool last = off + len == body.size();
      write_str(frame(0, last ? 0x1 : 0, stream_, body.substr(off, len)));
      off += len;
      peer_stream_window_ -= (long long)len;
      peer_conn_window_ -= (long long)len;
    }
    std::string data, trailers;
    bool done = false, ends = false;
    size_t received = 0;
    while (!done) {
      Frame f = read_frame();
      if (connection_frame(f)) continue;
      if (f.stream != stream_) continue;
      if (f.type == 0) {                                            // DATA (padding is not used by grpc)
        data += f.payload;
        received += f.payload.size();
        done = f.flags & 0x1;
      } else if (f.type == 1 || f.type == 9) {                      // HEADERS / CONTINUATION: the last block before END_STREAM is the trailers
        size_t skip = 0;
        if (f.type == 1 && (f.flags & 0x20)) skip = 5;              // PRIORITY fields
        if (f.type == 1) {
          trailers = f.payload.substr(std::min(skip, f.payload.size()));
          ends = f.flags & 0x1;
        } else {
          trailers += f.payload;
        }
        if (f.flags & 0x4) done = ends;                             // END_HEADERS of a block that carried END_STREAM
      } else if (f.type == 3) {
        throw ShardError("shard reset the stream");
      }
    }
    if (received) write_str(frame(8, 0, 0, u32((uint32_t)received)));          // give the connection window back
    int status = -1;
    std::string msg;
    scan_trailers(trailers, status, msg);
    if (data.size() >= 5 && (status == 0 || status == -1)) {
      if (data[0] != 0) throw ShardError("compressed gRPC message (no compression was offered)");
      const unsigned char* p = (const unsigned char*)data.data();
      const uint32_t len = ((uint32_t)p[1] << 24) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 8) | p[4];
      if (len + 5 != data.size()) throw ShardError("truncated gRPC message");
      return data.substr(5);
    }
    throw ShardError(!msg.empty() ? msg : ("shard error (grpc-status " + (status < 0 ? std::string("unknown") : std::to_string(status)) + ")"));
  }

  // A reader of the HPACK subset grpc servers use for trailers: indexed fields are skipped, literal fields are read when their
  // strings are not Huffman-coded.  grpc-message is percent-encoded.
  static size_t read_int(const std::string& b, size_t& i, int prefix_bits) {
    const size_t cap = (1u << prefix_bits) - 1;
    size_t v = (unsigned char)b[i++] & cap;
    if (v < cap) return v;
    int shift = 0;
    while (i < b.size()) {
      const unsigned char c = (unsigned char)b[i++];
      v += (size_t)(c & 127) << shift;
      shift += 7;
      if (!(c & 128)) break;
    }
    return v;
  }
  static bool read_str(const std::string& b, size_t& i, std::string& out, bool& huffman) {
    if (i >= b.size()) return false;
    huffman = ((unsigned char)b[i] & 0x80) != 0;
    const size_t n = read_int(b, i, 7);
    if (i + n > b.size()) return false;
    out = b.substr(i, n);
    i += n;
    return true;
  }
  static std::string percent_decode(const std::string& s) {
    std::string o;
    for (size_t i = 0; i < s.size(); ++i) {
      if (s[i] == '%' && i + 2 < s.size() + 0 && std::isxdigit((unsigned char)s[i + 1]) && std::isxdigit((unsigned char)s[i + 2])) {
        o.push_back((char)std::stoi(s.substr(i + 1, 2), nullptr, 16));
        i += 2;
      } else {
        o.push_back(s[i]);
      }
    }
    return o;
  }
  static void scan_trailers(const std::string& b, int& status, std::string& msg) {
    size_t i = 0;
    while (i < b.size()) {
      const unsigned char c = (unsigned char)b[i];
      if (c & 0x80) { read_int(b, i, 7); continue; }                // indexed field
      if ((c & 0xe0) == 0x20) { read_int(b, i, 5); continue; }      // dynamic table size update
      const int prefix = (c & 0x40) ? 6 : 4;                        // literal with incremental indexing / without or never indexed
      const size_t name_idx = read_int(b, i, prefix);
      std::string name, value;
      bool hn = false, hv = false;
      if (name_idx == 0 && !read_str(b, i, name, hn)) return;
      if (!read_str(b, i, value, hv)) return;
      if (hn) continue;
      if (name == "grpc-status" && !hv) status = std::atoi(value.c_str());
      if (name == "grpc-message") msg = hv ? std::string("shard error (message not decoded)") : percent_decode(value);
    }
  }

  // ---------------------------------------------------------------- socket
  void ensure_connected() {
    if (fd_ >= 0) return;
    int fd = ::socket(AF_UNIX, SOCK_STREAM, 0);
    if (fd < 0) throw std::system_error(errno, std::generic_category(), "socket");
    sockaddr_un addr{};
    addr.sun_family = AF_UNIX;
    std::strncpy(addr.sun_path, path_.c_str(), sizeof(addr.sun_path) - 1);
    if (::connect(fd, (sockaddr*)&addr, sizeof addr) != 0) {
      int e = errno;
      ::close(fd);
      throw ShardError("cannot connect to shard socket " + path_ + ": " + std::strerror(e));
    }
    fd_ = fd;
    stream_ = (uint32_t)-1;                                          // first call uses stream 1
    peer_initial_window_ = 65535;
    peer_conn_window_ = 65535;
    peer_max_frame_ = 16384;
    std::string settings;
    settings += std::string("\x00\x02", 2) + u32(0);                 // ENABLE_PUSH = 0
    settings += std::string("\x00\x04", 2) + u32(0x7fffffffu);       // INITIAL_WINDOW_SIZE
    write_str(std::string("PRI * HTTP/2.0\r\n\r\nSM\r\n\r\n") + frame(4, 0, 0, settings) + frame(8, 0, 0, u32(0x7fffffffu - 65535u)));
  }
  void close_fd() { if (fd_ >= 0) { ::close(fd_); fd_ = -1; } }
  void write_str(const std::string& s) {
    const char* p = s.data();
    size_t n = s.size();
    while (n) {
      ssize_t w = ::send(fd_, p, n, MSG_NOSIGNAL);
      if (w <= 0) { if (w < 0 && errno == EINTR) continue; throw std::system_error(errno, std::generic_category(), "send"); }
      p += w; n -= (size_t)w;
    }
  }
  void read_all(void* buf, size_t n) {
    char* p = (char*)buf;
    while (n) {
      ssize_t r = ::recv(fd_, p, n, 0);
      if (r <= 0) { if (r < 0 && errno == EINTR) continue; throw std::system_error(r == 0 ? ECONNRESET : errno, std::generic_category(), "recv"); }
      p += r; n -= (size_t)r;
    }
  }

  std::string path_;
  std::shared_ptr<ShardClient> helpers_;
  int fd_ = -1;
  uint32_t stream_ = (uint32_t)-1;
  long long peer_initial_window_ = 65535, peer_stream_window_ = 65535, peer_conn_window_ = 65535;
  uint32_t peer_max_frame_ = 16384;
  std::mutex mu_;
};

}  // namespace lx
