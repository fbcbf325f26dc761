// Router -> shard transport.
//
// Messages are the protobuf messages of proto/generate.proto (generated codec: pb_gen.hpp).  The reference
// router speaks gRPC over unix sockets through tonic (router/client/src/client.rs, sharded_client.rs); this
// router carries the same messages over a length-prefixed frame on `{uds_path}-{rank}.lx`:
//
//     request   u32 method | u32 length | bytes            (little endian; method ids: gen::Method)
//     response  u32 status | u32 length | bytes            (status 0 = ok, otherwise bytes = error text)
//
// With bit 31 of `method` set, the first 55 bytes are a W3C `traceparent` ("00-<trace id>-<span id>-01") naming the
// router span this call belongs to; the message follows (the reference carries the same context in gRPC metadata,
// router/grpc-metadata/src/lib.rs:45-63).
//
// The Python shard serves both this framing and a regular grpc.aio LoraxService endpoint on `{uds_path}-{rank}`.
// `ShardedClient` fans every call out to all shards in parallel and merges the answers the way the reference
// does (sharded_client.rs:112-273): generations are concatenated, the last shard's CachedBatch wins, warmup takes
// the minimum, DownloadAdapter goes to shard 0 only.
#pragma once
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <cerrno>
#include <cstring>
#include <future>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <vector>

#include "image_chunks.hpp"
#include "pb_gen.hpp"
#include "tokenizer.hpp"

namespace lx {

struct ShardError : std::runtime_error {
  using std::runtime_error::runtime_error;
};

class ShardClient {
 public:
  virtual ~ShardClient() = default;
  // Raw call: returns the response payload or throws ShardError.
  virtual std::string call(uint32_t method, const std::string& payload) = 0;

  static constexpr uint32_t kTraceFlag = 0x80000000u;
  template <class Resp, class Req>
  Resp rpc(uint32_t method, const Req& req, const std::string& traceparent = std::string()) {
    Resp resp;
    std::string out = traceparent.size() == 55 ? call(method | kTraceFlag, traceparent + req.serialize()) : call(method, req.serialize());
    if (!resp.parse(out)) throw ShardError("malformed response for method " + std::to_string(method));
    return resp;
  }
};

class FramedUdsClient : public ShardClient {
 public:
  explicit FramedUdsClient(std::string path) : path_(std::move(path)) {}
  ~FramedUdsClient() override { close_fd(); }

  std::string call(uint32_t method, const std::string& payload) override {
    std::lock_guard<std::mutex> g(mu_);
    for (int attempt = 0; attempt < 2; ++attempt) {
      try {
        ensure_connected();
        uint32_t hdr[2] = {method, (uint32_t)payload.size()};
        write_all(hdr, sizeof hdr);
        write_all(payload.data(), payload.size());
        uint32_t rh[2];
        read_all(rh, sizeof rh);
        std::string body(rh[1], '\0');
        if (rh[1]) read_all(&body[0], rh[1]);
        if (rh[0] != 0) throw ShardError(body.empty() ? "shard error" : body);
        return body;
      } catch (const std::system_error&) {
        close_fd();
        if (attempt == 1) throw ShardError("connection to shard " + path_ + " lost");
      }
    }
    throw ShardError("unreachable");
  }

 private:
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
  }
  void close_fd() { if (fd_ >= 0) { ::close(fd_); fd_ = -1; } }
  void write_all(const void* buf, size_t n) {
    const char* p = (const char*)buf;
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
  int fd_ = -1;
  std::mutex mu_;
};

class ShardedClient {
 public:
  explicit ShardedClient(std::vector<std::shared_ptr<ShardClient>> shards) : shards_(std::move(shards)) {}
  static ShardedClient connect_uds(const std::string& uds_path, int num_shards) {
    std::vector<std::shared_ptr<ShardClient>> v;
    for (int r = 0; r < num_shards; ++r) v.push_back(std::make_shared<FramedUdsClient>(uds_path + "-" + std::to_string(r) + ".lx"));
    return ShardedClient(std::move(v));
  }
  size_t size() const { return shards_.size(); }
  // Trace context of the calls that follow (the batching loop sets it around every Prefill / Decode; empty = none).
  void set_trace(std::string traceparent) { std::lock_guard<std::mutex> g(trace_slot_.mu); trace_slot_.tp = std::move(traceparent); }

  gen::InfoResponse info() { return all<gen::InfoResponse>(gen::M_Info, gen::InfoRequest{}).front(); }
  void health() { all<gen::HealthResponse>(gen::M_Health, gen::HealthRequest{}); }
  void clear_cache(std::optional<uint64_t> id) {
    gen::ClearCacheRequest r;
    r.id = id;
    all<gen::ClearCacheResponse>(gen::M_ClearCache, r);
  }
  std::optional<gen::CachedBatch> filter_batch(uint64_t batch_id, const std::vector<uint64_t>& keep) {
    gen::FilterBatchRequest r;
    r.batch_id = batch_id;
    r.request_ids = keep;
    return all<gen::FilterBatchResponse>(gen::M_FilterBatch, r).back().batch;
  }
  std::optional<uint32_t> warmup(const gen::WarmupRequest& r) {
    std::optional<uint32_t> m;
    for (auto& resp : all<gen::WarmupResponse>(gen::M_Warmup, r))
      if (resp.max_supported_total_tokens && (!m || *resp.max_supported_total_tokens < *m)) m = resp.max_supported_total_tokens;
    return m;
  }
  struct StepResult {
    std::vector<gen::Generation> generations;
    std::optional<gen::CachedBatch> batch;
  };
  StepResult prefill(const gen::Batch& b, const std::optional<gen::CachedBatch>& cached,
                     const std::vector<gen::CachedBatch>& decode_batches = {}) {
    gen::PrefillRequest r;
    r.batch = b;
    r.cached_batch = cached;
    r.decode_batches = decode_batches;
    StepResult out;
    for (auto& resp : all<gen::PrefillResponse>(gen::M_Prefill, r)) {
      for (auto& g : resp.generations) out.generations.push_back(std::move(g));
      out.batch = resp.batch;
    }
    return out;
  }
  StepResult decode(const std::vector<gen::CachedBatch>& batches) {
    gen::DecodeRequest r;
    r.batches = batches;
    StepResult out;
    for (auto& resp : all<gen::DecodeResponse>(gen::M_Decode, r)) {
      for (auto& g : resp.generations) out.generations.push_back(std::move(g));
      out.batch = resp.batch;
    }
    return out;
  }
  gen::DownloadAdapterResponse download_adapter(const gen::DownloadAdapterRequest& r) {
    return shards_.front()->rpc<gen::DownloadAdapterResponse>(gen::M_DownloadAdapter, r);
  }
  bool load_adapter(const gen::LoadAdapterRequest& r) {
    bool ok = true;
    for (auto& resp : all<gen::LoadAdapterResponse>(gen::M_LoadAdapter, r)) ok = ok && resp.loaded;
    return ok;
  }
  bool offload_adapter(const gen::OffloadAdapterRequest& r) {
    bool ok = true;
    for (auto& resp : all<gen::OffloadAdapterResponse>(gen::M_OffloadAdapter, r)) ok = ok && resp.offloaded;
    return ok;
  }
  gen::EmbedResponse embed(const gen::Batch& b) {
    gen::EmbedRequest r;
    r.batch = b;
    return all<gen::EmbedResponse>(gen::M_Embed, r).front();
  }
  gen::ClassifyResponse classify(const gen::Batch& b) {
    gen::ClassifyRequest r;
    r.batch = b;
    return all<gen::ClassifyResponse>(gen::M_Classify, r).front();
  }
  // Request text -> ids.  With a local tokenizer (the router read the shard's tokenizer file and implements every component
  // it uses) this runs on the router's tokenizer workers; otherwise shard 0 is asked.  Chat templating and `/tokenize` with
  // character offsets are always helper calls to shard 0.
  void set_local_tokenizer(std::shared_ptr<tok::TokenizerPool> pool, bool images_to_shard = false, img::ImagePolicy policy = img::ImagePolicy()) {
    local_tok_ = std::move(pool);
    images_to_shard_ = images_to_shard;
    image_policy_ = std::move(policy);
  }
  bool tokenizes_locally() const { return local_tok_ != nullptr; }
  uint64_t local_tokenizations() const { return local_tok_ ? local_tok_->served() : 0; }
  std::vector<uint32_t> tokenize(const std::string& text, bool add_special = true) {
    if (local_tok_ && !(images_to_shard_ && text.find("![](") != std::string::npos)) return local_tok_->encode(text, add_special);
    if (local_tok_ && image_policy_.kind != img::ImagePolicy::None) {
      // a vision-language prompt: text parts through the tokenizer (special tokens with the first part only), every image as its
      // feature tokens; an image the router cannot size (a URL, an unknown format) sends the whole prompt to the shard
      std::vector<uint32_t> ids;
      bool first = true, handled = true;
      for (auto& part : img::split_prompt(text)) {
        if (!part.first) {
          const std::vector<uint32_t> t = local_tok_->encode(part.second, add_special && first);
          ids.insert(ids.end(), t.begin(), t.end());
        } else {
          const long n = image_policy_.count(part.second);
          if (n < 0) { handled = false; break; }
          ids.insert(ids.end(), (size_t)n, image_policy_.image_token);
        }
        first = false;
      }
      if (handled) return ids;
    }
    std::string out = shards_.front()->call(gen::M_Tokenize, std::string(1, add_special ? '\1' : '\0') + text);
    std::vector<uint32_t> ids(out.size() / 4);
    if (!ids.empty()) std::memcpy(ids.data(), out.data(), ids.size() * 4);
    return ids;
  }
  std::string helper(uint32_t method, const std::string& payload) { return shards_.front()->call(method, payload); }

 private:
  template <class Resp, class Req>
  std::vector<Resp> all(uint32_t method, const Req& req) {
    std::string tp;
    if (method == gen::M_Prefill || method == gen::M_Decode) { std::lock_guard<std::mutex> g(trace_slot_.mu); tp = trace_slot_.tp; }
    if (shards_.size() == 1) return {shards_[0]->rpc<Resp>(method, req, tp)};
    std::vector<std::future<Resp>> futs;
    for (auto& s : shards_) futs.push_back(std::async(std::launch::async, [s, method, &req, tp] { return s->template rpc<Resp>(method, req, tp); }));
    std::vector<Resp> out;
    std::exception_ptr err;
    for (auto& f : futs) {
      try { out.push_back(f.get()); } catch (...) { if (!err) err = std::current_exception(); }
    }
    if (err) std::rethrow_exception(err);
    return out;
  }
  std::vector<std::shared_ptr<ShardClient>> shards_;
  std::shared_ptr<tok::TokenizerPool> local_tok_;
  bool images_to_shard_ = false;
  img::ImagePolicy image_policy_;
  struct TraceSlot {                      // movable holder: the client itself is passed around by value once
    std::mutex mu;
    std::string tp;
    TraceSlot() = default;
    TraceSlot(TraceSlot&& o) noexcept : tp(std::move(o.tp)) {}
  } trace_slot_;
};

}  // namespace lx
