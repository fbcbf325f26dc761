// C ABI over the router's data structures, for the Python bindings and the tests (ctypes):
// block allocator / radix trie, adapter queues, JSON, and an in-process Infer driven by a fake shard, which is
// how the scheduler and the batching loop are tested without a GPU or sockets (the reference left those tests
// commented out: router/src/loader.rs:345-564).
#include <cstring>

#include "chat_template.hpp"
#include "encoder_batcher.hpp"
#include "infer.hpp"
#include "json.hpp"
#include "tokenizer.hpp"

using namespace lx;

namespace {

thread_local std::string g_ret;
const char* ret(const std::string& s) { g_ret = s; return g_ret.c_str(); }

// A shard that "generates" deterministic tokens: token k of request id r is (r * 1000 + k) % 50000.  Adapter ids
// containing "missing" fail to download; ids containing "slow" take 50 ms to load.
class FakeShard : public ShardClient {
 public:
  struct Live { uint32_t max_new; uint32_t produced; uint64_t id; };
  std::mutex mu;
  std::map<uint64_t, std::vector<Live>> batches;
  std::vector<std::string> log;                       // method trace
  std::atomic<int> fail_decode_after{-1};
  int decodes = 0;
  uint32_t block_size = 16;
  std::set<uint32_t> loaded;
  std::vector<size_t> embed_batches;                  // sizes of the Embed batches seen

  std::string call(uint32_t method, const std::string& payload) override {
    std::lock_guard<std::mutex> g(mu);
    switch (method) {
      case gen::M_Info: {
        gen::InfoResponse r;
        r.requires_padding = false; r.dtype = "bfloat16"; r.device_type = "cuda"; r.block_size = block_size;
        r.supports_generation = true; r.requires_block_allocator = true;
        return r.serialize();
      }
      case gen::M_Health: return gen::HealthResponse{}.serialize();
      case gen::M_ClearCache: {
        gen::ClearCacheRequest q; q.parse(payload);
        if (q.id) batches.erase(*q.id); else batches.clear();
        log.push_back("clear");
        return gen::ClearCacheResponse{}.serialize();
      }
      case gen::M_Warmup: { gen::WarmupResponse r; r.max_supported_total_tokens = 100000; return r.serialize(); }
      case gen::M_Prefill: {
        gen::PrefillRequest q; q.parse(payload);
        gen::PrefillResponse resp;
        std::vector<Live> live;
        std::string l = "prefill";
        for (auto& r : q.batch->requests) {
          l += " " + std::to_string(r.id) + "@" + std::to_string(r.adapter_index);
          if (r.adapter_index != 0 && !loaded.count(r.adapter_index)) throw ShardError("adapter not loaded");
          Live lv{r.stopping_parameters->max_new_tokens, 1, r.id};
          resp.generations.push_back(make_gen(lv));
          if (lv.produced < lv.max_new) live.push_back(lv);
        }
        log.push_back(l);
        if (!live.empty()) {
          batches[q.batch->id] = live;
          resp.batch = cached(q.batch->id, live);
        }
        return resp.serialize();
      }
      case gen::M_Decode: {
        if (fail_decode_after >= 0 && decodes++ >= fail_decode_after) throw ShardError("injected decode failure");
        gen::DecodeRequest q; q.parse(payload);
        std::vector<Live> merged;
        for (auto& b : q.batches) {
          auto it = batches.find(b.id);
          if (it == batches.end()) throw ShardError("batch not in cache");
          for (auto& lv : it->second) merged.push_back(lv);
          batches.erase(it);
        }
        gen::DecodeResponse resp;
        std::vector<Live> live;
        for (auto& lv : merged) {
          lv.produced++;
          resp.generations.push_back(make_gen(lv));
          if (lv.produced < lv.max_new) live.push_back(lv);
        }
        uint64_t id = q.batches.front().id;
        log.push_back("decode " + std::to_string(merged.size()));
        if (!live.empty()) { batches[id] = live; resp.batch = cached(id, live); }
        return resp.serialize();
      }
      case gen::M_FilterBatch: {
        gen::FilterBatchRequest q; q.parse(payload);
        auto& v = batches[q.batch_id];
        std::vector<Live> keep;
        for (auto& lv : v) if (std::find(q.request_ids.begin(), q.request_ids.end(), lv.id) != q.request_ids.end()) keep.push_back(lv);
        v = keep;
        gen::FilterBatchResponse resp;
        resp.batch = cached(q.batch_id, keep);
        return resp.serialize();
      }
      case gen::M_DownloadAdapter: {
        gen::DownloadAdapterRequest q; q.parse(payload);
        const std::string id = q.adapter_parameters->adapter_ids.empty() ? "" : q.adapter_parameters->adapter_ids[0];
        if (id.find("missing") != std::string::npos) throw ShardError("adapter " + id + " not found");
        gen::DownloadAdapterResponse r; r.downloaded = true; r.memory_fraction = 0.3f;
        log.push_back("download " + id);
        return r.serialize();
      }
      case gen::M_LoadAdapter: {
        gen::LoadAdapterRequest q; q.parse(payload);
        loaded.insert(q.adapter_index);
        log.push_back("load " + std::to_string(q.adapter_index));
        gen::LoadAdapterResponse r; r.loaded = true; return r.serialize();
      }
      case gen::M_OffloadAdapter: {
        gen::OffloadAdapterRequest q; q.parse(payload);
        loaded.erase(q.adapter_index);
        log.push_back("offload " + std::to_string(q.adapter_index));
        gen::OffloadAdapterResponse r; r.offloaded = true; return r.serialize();
      }
      case gen::M_Tokenize: {
        std::vector<uint32_t> ids;
        std::string wd;
        for (size_t i = 1; i <= payload.size(); ++i) {
          if (i == payload.size() || payload[i] == ' ' || payload[i] == '\n' || payload[i] == '\t') {
            if (!wd.empty()) ids.push_back((uint32_t)(std::hash<std::string>{}(wd) % 50000));
            wd.clear();
          } else {
            wd += payload[i];
          }
        }
        return ids.empty() ? std::string() : std::string((const char*)ids.data(), ids.size() * 4);
      }
      case gen::M_Embed: {
        // embedding of request i: [number of input ids, first id, batch size]; a request whose text is "boom" fails the batch
        gen::EmbedRequest q;
        q.parse(payload);
        gen::EmbedResponse r;
        const gen::Batch none;
        const gen::Batch& bt = q.batch ? *q.batch : none;
        embed_batches.push_back(bt.requests.size());
        for (auto& rq : bt.requests) {
          if (rq.inputs == "boom") { r.errorMsg = "the encoder exploded"; r.embeddings.clear(); return r.serialize(); }
          gen::Embedding e;
          e.request_id = rq.id;
          const auto& ids = rq.tokenized_inputs ? rq.tokenized_inputs->ids : std::vector<uint32_t>{};
          e.values = {(float)ids.size(), ids.empty() ? -1.f : (float)ids[0], (float)bt.requests.size()};
          r.embeddings.push_back(e);
        }
        std::this_thread::sleep_for(std::chrono::milliseconds(2));        // long enough for the next batch to fill up
        return r.serialize();
      }
      case gen::M_Classify: {
        gen::ClassifyRequest q;
        q.parse(payload);
        gen::ClassifyResponse r;
        const gen::Batch none;
        const gen::Batch& bt = q.batch ? *q.batch : none;
        for (auto& rq : bt.requests) {
          gen::ClassifyPredictionList l;
          l.request_id = rq.id;
          const size_t n = rq.tokenized_inputs ? rq.tokenized_inputs->ids.size() : 0;
          for (size_t i = 0; i < n; ++i) { l.predictions.push_back("TAG" + std::to_string(i % 3)); l.scores.push_back(0.5f); }
          r.classify_prediction_lists.push_back(l);
        }
        return r.serialize();
      }
      default: throw ShardError("method not implemented by the fake shard");
    }
  }

 private:
  static gen::Generation make_gen(const Live& lv) {
    gen::Generation g;
    g.request_id = lv.id;
    g.next_tokens.emplace();
    uint32_t tok = (uint32_t)((lv.id * 1000 + lv.produced) % 50000);
    g.next_tokens->ids = {tok};
    g.next_tokens->logprobs = {-0.5f};
    g.next_tokens->texts = {" t" + std::to_string(tok)};
    g.next_tokens->is_special = {false};
    if (lv.produced >= lv.max_new) {
      g.generated_text.emplace();
      g.generated_text->text = "done-" + std::to_string(lv.id);
      g.generated_text->generated_tokens = lv.produced;
      g.generated_text->finish_reason = gen::FinishReason_FINISH_REASON_LENGTH;
    }
    return g;
  }
  static gen::CachedBatch cached(uint64_t id, const std::vector<Live>& live) {
    gen::CachedBatch b;
    b.id = id;
    for (auto& lv : live) { b.request_ids.push_back(lv.id); b.max_tokens += lv.max_new; }
    b.size = (uint32_t)live.size();
    return b;
  }
};

}  // namespace

extern "C" {

// ---------------------------------------------------------------- allocators
void* lx_alloc_new(uint32_t num_blocks, uint32_t block_size, int window, int prefix_caching) {
  return make_allocator(num_blocks, block_size, window > 0 ? std::optional<uint32_t>((uint32_t)window) : std::nullopt, prefix_caching != 0).release();
}
void lx_alloc_delete(void* a) { delete static_cast<Allocator*>(a); }
uint64_t lx_alloc_free_blocks(void* a) { return static_cast<Allocator*>(a)->free_blocks(); }
// Returns a handle (BlockAllocation*) or null.  tokens_ptr may be null (no prefix lookup).
void* lx_alloc_allocate(void* a, uint32_t adapter, uint32_t tokens, const uint32_t* prompt, uint32_t prompt_len) {
  std::vector<uint32_t> p;
  if (prompt) p.assign(prompt, prompt + prompt_len);
  auto r = static_cast<Allocator*>(a)->allocate(adapter, tokens, prompt ? &p : nullptr);
  if (!r) return nullptr;
  return new BlockAllocation(std::move(*r));
}
uint32_t lx_allocation_num_blocks(void* h) { return (uint32_t) static_cast<BlockAllocation*>(h)->blocks.size(); }
uint32_t lx_allocation_prefix_len(void* h) { return static_cast<BlockAllocation*>(h)->prefix_len; }
uint32_t lx_allocation_num_slots(void* h) { return (uint32_t) static_cast<BlockAllocation*>(h)->slots.size(); }
void lx_allocation_blocks(void* h, uint32_t* out) { auto& b = static_cast<BlockAllocation*>(h)->blocks; if (!b.empty()) std::memcpy(out, b.data(), b.size() * 4); }
void lx_allocation_slots(void* h, uint32_t* out) { auto& b = static_cast<BlockAllocation*>(h)->slots; if (!b.empty()) std::memcpy(out, b.data(), b.size() * 4); }
void lx_alloc_free(void* a, void* h, uint32_t adapter, const uint32_t* all_tokens, uint32_t n) {
  std::vector<uint32_t> t;
  if (all_tokens) t.assign(all_tokens, all_tokens + n);
  static_cast<Allocator*>(a)->free(*static_cast<BlockAllocation*>(h), adapter, all_tokens ? &t : nullptr);
  delete static_cast<BlockAllocation*>(h);
}

// ---------------------------------------------------------------- JSON round trip (parser conformance tests)
const char* lx_json_roundtrip(const char* s) {
  json::Value v;
  std::string err;
  if (!json::parse(s, v, &err)) return ret("ERROR: " + err);
  return ret(v.dump());
}

// ---------------------------------------------------------------- adapter queues
// Script-driven: ops is a JSON array of [op, args...]; returns a JSON trace.  Ops:
//   ["append", adapter_index]  ["downloaded", idx, cost]  ["ready", idx]  ["update", [in_use...], now_s]  ["next", now_s]
const char* lx_queues_script(int max_active, double cycle_s, const char* ops_json) {
  json::Value ops;
  if (!json::parse(ops_json, ops)) return ret("ERROR: bad script");
  AdapterQueues q((size_t)max_active, cycle_s, 1.0f);
  json::Value out = json::Value::array();
  auto t0 = Clock::now();
  uint64_t next_id = 1;
  for (auto& op : ops.items()) {
    const std::string name = op.items()[0].as_string();
    auto at = [&](double s) { return t0 + std::chrono::microseconds((long long)(s * 1e6)); };
    if (name == "append") {
      auto e = std::make_shared<Entry>();
      e->id = next_id++;
      e->request.adapter.index = (uint32_t)op.items()[1].as_int();
      e->request.adapter.ids = {"a" + std::to_string(e->request.adapter.index)};
      e->queue_time = at(op.items().size() > 2 ? op.items()[2].as_double() : 0.0);
      e->sink = std::make_shared<ResponseSink>();
      out.push(json::Value(q.append(e)));
    } else if (name == "downloaded") {
      q.set_downloaded((uint32_t)op.items()[1].as_int(), (float)op.items()[2].as_double());
      out.push(json::Value());
    } else if (name == "ready") {
      q.set_ready((uint32_t)op.items()[1].as_int());
      out.push(json::Value());
    } else if (name == "update") {
      std::set<uint32_t> in_use;
      for (auto& x : op.items()[1].items()) in_use.insert((uint32_t)x.as_int());
      auto up = q.update_adapters(in_use, at(op.items()[2].as_double()));
      json::Value r = json::Value::object();
      json::Value l = json::Value::array(), o = json::Value::array();
      for (auto& a : up.load) l.push(a.index);
      for (auto& a : up.offload) o.push(a.index);
      r.set("load", l);
      r.set("offload", o);
      r.set("budget", q.budget_remaining());
      out.push(r);
    } else if (name == "next") {
      auto e = q.next_entry(at(op.items()[1].as_double()));
      out.push(e ? json::Value((unsigned long long)e->id) : json::Value());
    }
  }
  return ret(out.dump());
}

// ---------------------------------------------------------------- Infer against a fake shard
// requests_json: [{"inputs": "...", "adapter_id": "...", "max_new_tokens": n}, ...] submitted concurrently.
// Returns {"results": [{"ok":bool,"text":..,"tokens":n,"error":..}], "log": [...shard trace...]}.
const char* lx_infer_fake_run(const char* requests_json, int max_active_adapters, int fail_decode_after, uint32_t num_blocks,
                              int prefix_caching) {
  json::Value reqs;
  if (!json::parse(requests_json, reqs)) return ret("ERROR: bad requests");
  auto fake = std::make_shared<FakeShard>();
  fake->fail_decode_after = fail_decode_after;
  auto client = std::make_shared<ShardedClient>(std::vector<std::shared_ptr<ShardClient>>{fake});
  RouterConfig cfg;
  cfg.max_input_length = 512;
  cfg.max_total_tokens = 1024;
  cfg.max_batch_prefill_tokens = 1024;
  cfg.max_batch_total_tokens = 100000;
  cfg.max_active_adapters = (size_t)max_active_adapters;
  cfg.adapter_cycle_time_s = 0.05;
  cfg.prefix_caching = prefix_caching != 0;
  cfg.waiting_served_ratio = 0.3f;
  Metrics metrics;
  json::Value results = json::Value::array();
  {
    Infer infer(client, cfg, client->info(), num_blocks, &metrics);
    infer.start();
    std::vector<std::future<json::Value>> futs;
    for (auto& r : reqs.items()) {
      futs.push_back(std::async(std::launch::async, [&infer, r] {
        json::Value out = json::Value::object();
        try {
          GenerateParams p;
          if (r["adapter_id"].is_string()) p.adapter_id = r["adapter_id"].as_string();
          p.max_new_tokens = (uint32_t)r["max_new_tokens"].as_int(4);
          if (r["temperature"].is_number()) p.temperature = (float)r["temperature"].as_double();
          if (r["top_p"].is_number()) p.top_p = (float)r["top_p"].as_double();
          auto sink = infer.generate_stream(r["inputs"].as_string(), p);
          int tokens = 0;
          while (true) {
            StreamEvent ev;
            if (!sink->pop(ev, 10000)) { out.set("ok", false); out.set("error", "timeout"); break; }
            if (ev.kind == StreamEvent::Token) { ++tokens; continue; }
            if (ev.kind == StreamEvent::Error) { out.set("ok", false); out.set("error", ev.error); out.set("error_type", ev.error_type); break; }
            if (ev.kind == StreamEvent::End) { out.set("ok", true); out.set("text", ev.generated_text->text); out.set("tokens", tokens); break; }
          }
          infer.request_done();
        } catch (const ApiError& e) {
          out.set("ok", false);
          out.set("error", e.what());
          out.set("error_type", e.type);
          out.set("status", e.status);
        }
        return out;
      }));
    }
    for (auto& f : futs) results.push(f.get());
    infer.stop();
  }
  json::Value out = json::Value::object();
  out.set("results", results);
  json::Value log = json::Value::array();
  for (auto& l : fake->log) log.push(l);
  out.set("log", log);
  out.set("metrics", metrics.render());
  return ret(out.dump());
}

// Feature tokens the router counts for one image reference under an image policy (JSON as shard 0 sends it); -1: left to the shard.
long lx_image_token_count(const char* policy_json, const char* uri) {
  json::Value pol;
  std::string err;
  if (!json::parse(policy_json, pol, &err)) return -2;
  return img::ImagePolicy::from_json(pol).count(uri);
}

// The prompt cut at its image references: JSON [[is_image, text-or-uri], ...].
const char* lx_split_image_prompt(const char* text) {
  json::Value out = json::Value::array();
  for (auto& part : img::split_prompt(text)) {
    json::Value p = json::Value::array();
    p.push(part.first);
    p.push(part.second);
    out.push(p);
  }
  return ret(out.dump());
}

// A chat request rendered by the router's template interpreter.  `request_json`: {"template", "bos_token", "eos_token", "messages",
// "tools"?, "tool_prompt"?, "guideline"?}.  JSON out: {"text": ...}, {"error": ...} (the template raised or misused a value) or
// {"unsupported": ...} (outside the interpreter's subset: the router would ask a shard).
const char* lx_chat_render(const char* request_json) {
  json::Value req, out = json::Value::object();
  std::string err;
  if (!json::parse(request_json, req, &err)) { out.set("error", "bad request json: " + err); return ret(out.dump()); }
  try {
    jinja::ChatRenderer r;
    r.tmpl = jinja::Template::compile(req["template"].as_string());
    r.bos_token = req["bos_token"].as_string();
    r.eos_token = req["eos_token"].as_string();
    out.set("text", r.render(req));
  } catch (const jinja::Unsupported& e) {
    out.set("unsupported", std::string(e.what()));
  } catch (const std::exception& e) {
    out.set("error", std::string(e.what()));
  }
  return ret(out.dump());
}

// Embed / classify inputs from `threads` caller threads, `each` inputs per thread, through the encoder batcher against the fake
// shard.  JSON: {"ok": answers that carried the caller's own input, "failed": answers that were errors, "batches": [sizes]}.  Every
// seventh input of thread 0 is the text that makes the fake shard fail its batch.
const char* lx_encoder_batcher_fake_run(int threads, int each) {
  auto fake = std::make_shared<FakeShard>();
  auto client = std::make_shared<ShardedClient>(std::vector<std::shared_ptr<ShardClient>>{fake});
  Metrics metrics(1024, 2048);
  std::atomic<int> ok{0}, failed{0}, wrong{0};
  {
    EncoderBatcher::Limits lim;
    lim.max_input_length = 64;
    lim.max_batch_tokens = 256;
    EncoderBatcher batcher(client, lim, &metrics);
    std::vector<std::thread> ts;
    for (int t = 0; t < threads; ++t)
      ts.emplace_back([&, t] {
        for (int k = 0; k < each; ++k) {
          const bool boom = t == 0 && k % 7 == 3;
          std::string text = boom ? "boom" : "";
          for (int w = 0; !boom && w <= (t + k) % 5; ++w) text += "w" + std::to_string(t * 1000 + k) + " ";
          const bool classify = (t + k) % 4 == 0 && !boom;
          try {
            auto res = batcher.submit(classify ? EncoderBatcher::Kind::Classify : EncoderBatcher::Kind::Embed, text).get();
            const size_t words = (size_t)((t + k) % 5 + 1);
            if (classify ? res.classes.predictions.size() == words : (res.embedding.size() == 3 && (size_t)res.embedding[0] == words)) ++ok;
            else ++wrong;
          } catch (const std::exception&) {
            ++failed;
          }
        }
      });
    for (auto& th : ts) th.join();
  }
  json::Value out = json::Value::object();
  out.set("ok", ok.load());
  out.set("failed", failed.load());
  out.set("wrong", wrong.load());
  json::Value sizes = json::Value::array();
  for (size_t n : fake->embed_batches) sizes.push((unsigned long long)n);
  out.set("batches", sizes);
  out.set("metrics", metrics.render());
  return ret(out.dump());
}

// ---- tokenizer: load a tokenizer.json, encode through a pool of `workers` threads.  `lx_tokenizer_load` returns null and
// writes the reason (an unsupported component, an unreadable file) to `err`.
struct TokHandle {
  std::shared_ptr<const tok::Tokenizer> tok;
  std::unique_ptr<tok::TokenizerPool> pool;
  std::string last_error;
};
void* lx_tokenizer_load(const char* path, int workers, char* err, int err_cap) {
  try {
    auto h = std::make_unique<TokHandle>();
    h->tok = tok::Tokenizer::load(path);
    h->pool = std::make_unique<tok::TokenizerPool>(h->tok, workers);
    return h.release();
  } catch (const std::exception& e) {
    if (err && err_cap > 0) { std::strncpy(err, e.what(), (size_t)err_cap - 1); err[err_cap - 1] = 0; }
    return nullptr;
  }
}
void lx_tokenizer_free(void* h) { delete static_cast<TokHandle*>(h); }
// Number of ids (the first `cap` are written to `out`), or -1 with the reason in lx_tokenizer_error.
long lx_tokenizer_encode(void* hv, const char* text, size_t len, int add_special, uint32_t* out, size_t cap) {
  auto* h = static_cast<TokHandle*>(hv);
  try {
    const std::vector<uint32_t> ids = h->pool->encode(std::string(text, len), add_special != 0);
    if (!ids.empty() && cap > 0) std::memcpy(out, ids.data(), std::min(cap, ids.size()) * sizeof(uint32_t));
    return (long)ids.size();
  } catch (const std::exception& e) {
    h->last_error = e.what();
    return -1;
  }
}
const char* lx_tokenizer_error(void* h) { return static_cast<TokHandle*>(h)->last_error.c_str(); }
// All matches of `pattern` in `text` as a JSON array of [begin, end) code point offsets (the scan the Split pre-tokenizer and the
// Replace normaliser do); "error: ..." when the pattern is outside the engine's subset.
const char* lx_regex_find_all(const char* pattern, const char* text) {
  std::string err;
  auto re = MiniRegex::compile(pattern, &err);
  if (!re) return ret("error: " + err);
  const uni::Text t = uni::from_utf8(text);
  json::Value out = json::Value::array();
  size_t at = 0;
  while (at <= t.size()) {
    size_t b, e;
    if (!re->search(t.data(), t.size(), at, &b, &e)) break;
    json::Value m = json::Value::array();
    m.push((unsigned long long)b);
    m.push((unsigned long long)e);
    out.push(m);
    at = e > b ? e : b + 1;
  }
  return ret(out.dump());
}
// Normalisation form of a UTF-8 string ("NFC", "NFD", "NFKC", "NFKD", "lower"), for the Unicode tables' own test.
const char* lx_unicode_normalize(const char* text, const char* form) {
  const std::string f = form;
  const uni::Text t = uni::from_utf8(text);
  if (f == "lower") return ret(uni::to_utf8(uni::lowercase(t)));
  const uni::Form which = f == "NFC" ? uni::Form::NFC : f == "NFD" ? uni::Form::NFD : f == "NFKC" ? uni::Form::NFKC : uni::Form::NFKD;
  return ret(uni::to_utf8(uni::normalize(t, which)));
}

}  // extern "C"
