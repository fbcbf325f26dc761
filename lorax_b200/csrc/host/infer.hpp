// Request validation, the adapter scheduler and the continuous-batching loop of the router.
//
// Behavioural counterpart of router/src/{validation.rs, scheduler.rs, loader.rs, infer.rs} of the reference:
//   generate_stream(): concurrency permit -> adapter index assignment -> validation -> per-adapter queue;
//   scheduler next_batch(): update adapter residency, pop the oldest requests of resident adapters, allocate KV
//     blocks, respect the prefill-token and total-token budgets, build the Batch message;
//   batching loop: prefill a new batch, then decode; between decode steps try to admit another batch when enough
//     requests wait (waiting_served_ratio) or the oldest has waited max_waiting_tokens steps;
//   loader thread: DownloadAdapter / LoadAdapter / OffloadAdapter calls off the hot loop, per-adapter error
//     isolation (a failing adapter fails only its own requests).
// Threads instead of tokio tasks; one mutex guards the scheduler state.
#pragma once
#include <atomic>
#include <random>
#include <thread>

#include "adapter_queues.hpp"
#include "metrics.hpp"
#include "shard_client.hpp"
#include "telemetry.hpp"

namespace lx {

struct RouterConfig {
  size_t max_concurrent_requests = 1024;
  uint32_t max_best_of = 2;
  uint32_t max_stop_sequences = 4;
  uint32_t max_input_length = 1024;
  uint32_t max_total_tokens = 2048;
  uint32_t max_batch_prefill_tokens = 4096;
  uint32_t max_batch_total_tokens = 0;       // 0: taken from warmup
  float waiting_served_ratio = 1.2f;
  uint32_t max_waiting_tokens = 20;
  size_t max_active_adapters = 1024;
  double adapter_cycle_time_s = 2.0;
  bool eager_prefill = true;
  bool prefix_caching = false;
  bool chunked_prefill = false;
  std::string default_adapter_source = "hub";
  std::string model_id = "";
};

struct ApiError : std::runtime_error {
  std::string type;     // validation | overloaded | generation | incomplete_generation
  int status;
  ApiError(const std::string& msg, std::string t, int s) : std::runtime_error(msg), type(std::move(t)), status(s) {}
};
inline ApiError validation_error(const std::string& m) { return ApiError(m, "validation", 422); }

struct GenerateParams {
  std::string traceparent;                // the caller's W3C trace context (request header), if any
  std::string trace_id, span_id;          // this request's own span, set by the router when tracing is on
  std::optional<std::string> adapter_id;
  std::optional<std::string> adapter_source;
  std::vector<std::string> merged_ids;
  std::vector<float> merged_weights;
  std::string merge_strategy = "linear";
  float density = 0.f;
  std::string majority_sign_method = "total";
  std::optional<std::string> api_token;
  std::optional<uint32_t> best_of;
  std::optional<float> temperature, repetition_penalty, frequency_penalty, presence_penalty, top_p, typical_p;
  std::optional<int32_t> top_k;
  bool do_sample = false;
  std::optional<uint32_t> max_new_tokens;
  bool ignore_eos_token = false;
  std::optional<bool> return_full_text;
  std::vector<std::string> stop;
  std::optional<uint32_t> truncate;
  bool watermark = false;
  bool details = false;
  bool decoder_input_details = false;
  std::optional<uint32_t> return_k_alternatives;
  std::optional<uint64_t> seed;
  std::optional<std::string> schema;         // JSON schema for structured output
  std::vector<uint32_t> input_ids;           // pre-tokenised prompt (optional)
};

class Infer {
 public:
  Infer(std::shared_ptr<ShardedClient> client, RouterConfig cfg, const gen::InfoResponse& info, uint32_t num_blocks,
        Metrics* metrics)
      : client_(std::move(client)), cfg_(cfg), metrics_(metrics),
        queues_(cfg.max_active_adapters, cfg.adapter_cycle_time_s), block_size_(info.block_size ? info.block_size : 16),
        window_(info.window_size), speculate_(info.speculate), requires_padding_(info.requires_padding),
        fused_prefill_decode_(info.fused_prefill_decode) {
    allocator_ = make_allocator(num_blocks, block_size_, window_, cfg.prefix_caching);
    for (auto& p : info.preloaded_adapters) {
      if (!p.adapter_parameters || p.adapter_parameters->adapter_ids.empty()) continue;
      AdapterKey k;
      k.ids = p.adapter_parameters->adapter_ids;
      k.index = p.adapter_index;
      adapter_index_[k.identity()] = p.adapter_index;
      next_adapter_index_ = std::max(next_adapter_index_, p.adapter_index + 1);
    }
  }
  ~Infer() { stop(); }

  // Must be called before `start`.  Batch spans become children of one "batching_task" span per process.
  void set_tracer(telemetry::Tracer* t) {
    tracer_ = t;
    if (t && t->enabled()) {
      auto root = t->start("batching_task");
      loop_ctx_ = root.ctx;
      t->end(root);
    }
  }
  void start() {
    running_ = true;
    batch_thread_ = std::thread([this] { batching_loop(); });
    loader_thread_ = std::thread([this] { loader_loop(); });
  }
  void stop() {
    if (!running_.exchange(false)) return;
    { std::lock_guard<std::mutex> g(mu_); }
    cv_.notify_all();
    loader_cv_.notify_all();
    if (batch_thread_.joinable()) batch_thread_.join();
    if (loader_thread_.joinable()) loader_thread_.join();
  }
  bool healthy() const { return healthy_; }
  size_t in_flight() const { return in_flight_; }

  // Validate and enqueue.  Throws ApiError.
  std::shared_ptr<ResponseSink> generate_stream(const std::string& inputs, const GenerateParams& p, ValidRequest* out_valid = nullptr) {
    if (in_flight_.fetch_add(1) >= cfg_.max_concurrent_requests) {
      in_flight_--;
      if (metrics_) metrics_->inc("lorax_request_failure", {{"err", "overloaded"}});
      throw ApiError("Model is overloaded", "overloaded", 429);
    }
    try {
      auto entry = std::make_shared<Entry>();
      entry->request = validate(inputs, p);
      entry->sink = std::make_shared<ResponseSink>();
      if (out_valid) *out_valid = entry->request;
      {
        std::lock_guard<std::mutex> g(mu_);
        entry->id = next_id_++;
        bool is_new = queues_.append(entry);
        if (is_new) { loader_queue_.push_back({LoaderCmd::Download, entry->request.adapter}); loader_cv_.notify_one(); }
        if (metrics_) metrics_->set("lorax_queue_length", (double)queues_.queued());
      }
      cv_.notify_one();
      return entry->sink;
    } catch (...) {
      in_flight_--;
      throw;
    }
  }
  void request_done() { in_flight_--; }

  ValidRequest validate(const std::string& inputs, const GenerateParams& p) {
    ValidRequest v;
    if (p.best_of && *p.best_of > 1) {
      if (*p.best_of > cfg_.max_best_of) throw validation_error("`best_of` must be > 0 and <= " + std::to_string(cfg_.max_best_of) + ". Given: " + std::to_string(*p.best_of));
      if (!(p.do_sample || p.temperature || p.top_k || p.top_p || p.typical_p)) throw validation_error("you must use sampling when `best_of` is > 1");
      if (p.seed) throw validation_error("`seed` must not be set when `best_of` > 1");
    }
    auto& np = v.parameters;
    float temperature = p.temperature.value_or(1.0f);
    if (temperature < 0.f) throw validation_error("`temperature` must be non-negative");
    np.do_sample = p.do_sample || p.top_k || p.top_p || p.typical_p || (p.temperature && temperature != 1.0f && temperature != 0.f);
    if (p.temperature && temperature == 0.f) { np.do_sample = false; temperature = 1.0f; }   // temperature 0 means greedy
    np.temperature = temperature;
    float rep = p.repetition_penalty.value_or(1.0f);
    if (rep <= 0.f) throw validation_error("`repetition_penalty` must be strictly positive");
    np.repetition_penalty = rep;
    float fp = p.frequency_penalty.value_or(0.f), pp = p.presence_penalty.value_or(0.f);
    if (fp < -2.f || fp > 2.f) throw validation_error("`frequency_penalty` must be >= -2.0 and <= 2.0");
    if (pp < -2.f || pp > 2.f) throw validation_error("`presence_penalty` must be >= -2.0 and <= 2.0");
    np.frequency_penalty = fp;
    np.presence_penalty = pp;
    if (p.top_p && (*p.top_p <= 0.f || *p.top_p > 1.f)) throw validation_error("`top_p` must be > 0.0 and <= 1.0");
    np.top_p = p.top_p.value_or(1.0f);
    if (p.typical_p && (*p.typical_p <= 0.f || *p.typical_p >= 1.f)) throw validation_error("`typical_p` must be > 0.0 and < 1.0");
    np.typical_p = p.typical_p.value_or(1.0f);
    if (p.top_k && *p.top_k <= 0) throw validation_error("`top_k` must be strictly positive");
    np.top_k = p.top_k ? (uint32_t)*p.top_k : 0;
    np.watermark = p.watermark;
    np.return_k_alternatives = p.return_k_alternatives.value_or(0);
    np.schema = p.schema;
    np.seed = p.seed ? *p.seed : random_seed();
    if (p.stop.size() > cfg_.max_stop_sequences) throw validation_error("`stop` supports up to " + std::to_string(cfg_.max_stop_sequences) + " stop sequences. Given: " + std::to_string(p.stop.size()));
    if (p.truncate && (*p.truncate == 0 || *p.truncate > cfg_.max_input_length)) throw validation_error("`truncate` must be strictly positive and less than " + std::to_string(cfg_.max_input_length) + ". Given: " + std::to_string(*p.truncate));
    if (p.max_new_tokens && *p.max_new_tokens == 0) throw validation_error("`max_new_tokens` must be strictly positive");
    if (!p.adapter_id.value_or("").empty() && !p.merged_ids.empty()) throw validation_error("at most one of `adapter_id` or `merged_adapters` may be provided");
    if (inputs.empty() && p.input_ids.empty()) throw validation_error("`inputs` cannot be empty");

    // tokens
    v.inputs = inputs;
    if (p.input_ids.empty()) {
      try {
        v.input_ids = client_->tokenize(inputs);
      } catch (const ApiError&) {
        throw;
      } catch (const std::exception& e) {       // a word outside a vocabulary without an unknown token, an image that cannot be read ...
        throw validation_error(std::string("tokenizer error ") + e.what());
      }
    } else {
      v.input_ids = p.input_ids;
    }
    if (p.truncate && v.input_ids.size() > *p.truncate) v.input_ids.erase(v.input_ids.begin(), v.input_ids.end() - *p.truncate);
    v.trace_id = p.trace_id;
    v.span_id = p.span_id;
    v.truncate = p.truncate.value_or(cfg_.max_input_length);
    v.input_length = (uint32_t)v.input_ids.size();
    if (v.input_length == 0) throw validation_error("`inputs` cannot be empty");
    if (v.input_length > cfg_.max_input_length) throw validation_error("`inputs` must have less than " + std::to_string(cfg_.max_input_length) + " tokens. Given: " + std::to_string(v.input_length));
    uint32_t max_new = p.max_new_tokens ? *p.max_new_tokens : (cfg_.max_total_tokens > v.input_length ? cfg_.max_total_tokens - v.input_length : 0);
    if (max_new == 0 || v.input_length + max_new > cfg_.max_total_tokens)
      throw validation_error("`inputs` tokens + `max_new_tokens` must be <= " + std::to_string(cfg_.max_total_tokens) + ". Given: " +
                             std::to_string(v.input_length) + " `inputs` tokens and " + std::to_string(max_new) + " `max_new_tokens`");
    v.stopping.max_new_tokens = max_new;
    v.stopping.stop_sequences = p.stop;
    v.stopping.ignore_eos_token = p.ignore_eos_token;
    v.decoder_input_details = p.decoder_input_details;

    // adapter identity -> index (0 = base model)
    AdapterKey k;
    k.source = p.adapter_source.value_or(cfg_.default_adapter_source);
    k.api_token = p.api_token.value_or("");
    if (!p.merged_ids.empty()) {
      k.ids = p.merged_ids;
      k.weights = p.merged_weights;
      k.merge_strategy = p.merge_strategy == "ties" ? 1 : p.merge_strategy == "dare_linear" ? 2 : p.merge_strategy == "dare_ties" ? 3 : 0;
      k.density = p.density;
      k.majority_sign_method = p.majority_sign_method == "frequency" ? 1 : 0;
    } else {
      std::string id = p.adapter_id.value_or("");
      if (id.empty() || id == kBaseModelAdapterId || (!cfg_.model_id.empty() && id == cfg_.model_id)) id = kBaseModelAdapterId;
      k.ids = {id};
    }
    if (k.ids.size() == 1 && k.ids[0] == kBaseModelAdapterId) {
      k.index = 0;
    } else {
      std::lock_guard<std::mutex> g(index_mu_);
      auto it = adapter_index_.find(k.identity());
      if (it == adapter_index_.end()) it = adapter_index_.emplace(k.identity(), next_adapter_index_++).first;
      k.index = it->second;
    }
    np.adapter_id = k.ids.size() == 1 ? k.ids[0] : k.identity();
    v.adapter = k;
    return v;
  }

  // ---------------------------------------------------------------- scheduling (called with mu_ held)
  struct NextBatch {
    gen::Batch batch;
    std::vector<std::shared_ptr<Entry>> entries;
  };
  std::optional<NextBatch> next_batch(const std::set<uint32_t>& adapters_in_use, std::optional<size_t> min_size,
                                      uint32_t prefill_budget, uint32_t token_budget) {
    AdapterUpdate up = queues_.update_adapters(adapters_in_use);
    for (auto& a : up.offload) loader_queue_.push_back({LoaderCmd::Offload, a});
    for (auto& a : up.load) loader_queue_.push_back({LoaderCmd::Load, a});
    if (!up.offload.empty() || !up.load.empty()) loader_cv_.notify_one();
    if (min_size && chunking_.empty() && queues_.queued() < *min_size) return std::nullopt;

    NextBatch nb;
    uint32_t prefill_tokens = 0, decode_tokens = 0, max_blocks = 0;
    uint32_t max_input = 0;
    auto to_request = [&](const std::shared_ptr<Entry>& e) {
      gen::Request r;
      r.id = e->id;
      r.inputs = e->request.inputs;
      r.tokenized_inputs.emplace();
      r.tokenized_inputs->ids = e->request.input_ids;
      r.truncate = e->request.truncate;
      r.parameters = e->request.parameters;
      r.stopping_parameters = e->request.stopping;
      r.prefill_logprobs = e->request.decoder_input_details;
      r.adapter_index = e->request.adapter.index;
      if (e->allocation) {
        r.blocks = e->allocation->blocks;
        r.cache_len = e->allocation->prefix_len;
        // slots are implied by the blocks (slot = block * block_size + offset); sent only for sliding windows
        if (window_) r.slots = e->allocation->slots;
      }
      return r;
    };
    // Chunked prefill: prompts that did not fit the prefill budget of an earlier step continue first.  Every step carries at
    // most `prefill_budget` prompt tokens, so the decode steps of the running batch are never held up by one long prompt.
    bool continued = false;
    while (!chunking_.empty() && prefill_tokens < prefill_budget) {
      auto e = chunking_.front();
      const uint32_t remaining = e->request.input_length - e->prefilled;
      const uint32_t take = std::min(remaining, prefill_budget - prefill_tokens);
      gen::Request r = to_request(e);
      r.cache_len = e->prefilled;
      if (take < remaining) r.chunk_len = take; else chunking_.pop_front();
      e->prefilled += take;
      prefill_tokens += take;
      max_blocks = std::max(max_blocks, (uint32_t)e->allocation->blocks.size());
      nb.batch.requests.push_back(std::move(r));
      nb.entries.push_back(e);
      continued = true;
      if (take < remaining) break;
    }
    while (chunking_.empty() || !continued) {
      auto e = queues_.next_entry();
      if (!e) break;
      const uint32_t in_len = e->request.input_length, max_new = e->request.stopping.max_new_tokens;
      if (requires_padding_) {
        // padded models are budgeted by (n + 1) * longest prompt (scheduler.rs:348-368 of the reference)
        max_input = std::max(max_input, in_len);
        prefill_tokens = (uint32_t)(nb.entries.size() + 1) * max_input;
        decode_tokens += max_new;
        if (prefill_tokens > prefill_budget || prefill_tokens + decode_tokens > token_budget) { queues_.push_front(e); break; }
      } else {
        const uint32_t need = in_len + max_new + (speculate_ ? speculate_ - 1 : 0);
        const bool chunk = cfg_.chunked_prefill && prefill_tokens + in_len > prefill_budget;
        if (chunk && prefill_tokens >= prefill_budget) { queues_.push_front(e); break; }
        if (!chunk && prefill_tokens + in_len > prefill_budget && !nb.entries.empty()) { queues_.push_front(e); break; }
        if (!chunk && in_len > prefill_budget) {          // can never fit: fail it instead of blocking the queue
          StreamEvent ev;
          ev.kind = StreamEvent::Error;
          ev.error = "`inputs` exceed the prefill token budget";
          ev.error_type = "validation";
          e->sink->push(ev);
          continue;
        }
        if (decode_tokens + prefill_tokens + need > token_budget && token_budget > 0) { queues_.push_front(e); break; }
        auto alloc = allocator_->allocate(e->request.adapter.index, need, cfg_.prefix_caching ? &e->request.input_ids : nullptr);
        if (!alloc) { queues_.push_front(e); break; }
        e->allocation = std::move(alloc);
        decode_tokens += max_new;
        max_blocks = std::max(max_blocks, (uint32_t)e->allocation->blocks.size());
        e->batch_time = Clock::now();
        gen::Request r = to_request(e);
        if (chunk && r.cache_len + (prefill_budget - prefill_tokens) < in_len) {
          // only the first part of this prompt fits the step: the rest follows in later steps
          const uint32_t take = prefill_budget - prefill_tokens;
          r.chunk_len = take;
          e->prefilled = r.cache_len + take;
          prefill_tokens += take;
          chunking_.push_back(e);
          continued = true;
          nb.batch.requests.push_back(std::move(r));
          nb.entries.push_back(e);
          break;
        }
        prefill_tokens += in_len;
        nb.batch.requests.push_back(std::move(r));
        nb.entries.push_back(e);
        continue;
      }
      e->batch_time = Clock::now();
      nb.batch.requests.push_back(to_request(e));
      nb.entries.push_back(e);
    }
    if (nb.entries.empty()) return std::nullopt;
    if (min_size && !continued && nb.entries.size() < *min_size) {
      // not worth interrupting decode: put everything back in order
      for (auto it = nb.entries.rbegin(); it != nb.entries.rend(); ++it) {
        if ((*it)->allocation) { allocator_->free(*(*it)->allocation, (*it)->request.adapter.index, nullptr); (*it)->allocation.reset(); }
        queues_.push_front(*it);
      }
      return std::nullopt;
    }
    nb.batch.id = next_batch_id_++;
    nb.batch.size = (uint32_t)nb.entries.size();
    nb.batch.max_tokens = prefill_tokens + decode_tokens;
    nb.batch.max_blocks = max_blocks;
    if (metrics_) {
      metrics_->set("lorax_queue_length", (double)queues_.queued());
      metrics_->observe("lorax_batch_next_size", (double)nb.entries.size());
    }
    return nb;
  }

 private:
  // ---------------------------------------------------------------- batching loop
  using EntryMap = std::unordered_map<uint64_t, std::shared_ptr<Entry>>;

  void fail_all(EntryMap& entries, const std::string& msg) {
    for (auto& kv : entries) {
      StreamEvent ev;
      ev.kind = StreamEvent::Error;
      ev.error = msg;
      ev.error_type = "generation";
      kv.second->sink->push(ev);
      release(kv.second, false);
    }
    entries.clear();
  }
  // Returns the entry's blocks.  Only tokens whose keys / values the shards have written may become a cached prefix:
  // the whole prompt once a first token came back (the prefill finished), plus every generated token except the last,
  // which was sampled but never fed through the model.  After a failed step nothing is known to be written, so
  // nothing is cached (`kv_valid` false).
  void release(const std::shared_ptr<Entry>& e, bool kv_valid = true) {
    std::lock_guard<std::mutex> g(mu_);
    if (e->allocation) {
      std::vector<uint32_t> all;
      const bool cache = cfg_.prefix_caching && kv_valid && !e->generated.empty();
      if (cache) {
        all = e->request.input_ids;
        all.insert(all.end(), e->generated.begin(), e->generated.end() - 1);
      }
      allocator_->free(*e->allocation, e->request.adapter.index, cache ? &all : nullptr);
      e->allocation.reset();
    }
  }

  // Deliver generations; returns the ids of requests still running.
  std::vector<uint64_t> deliver(const std::vector<gen::Generation>& gens, EntryMap& entries, Clock::time_point step_start) {
    for (const auto& g : gens) {
      auto it = entries.find(g.request_id);
      if (it == entries.end()) continue;
      auto& e = it->second;
      bool gone = e->sink->closed();
      const double queue_s = std::chrono::duration<double>(e->batch_time - e->queue_time).count();
      if (g.prefill_tokens && !gone) {
        StreamEvent ev;
        ev.kind = StreamEvent::Prefill;
        ev.prefill_tokens = *g.prefill_tokens;
        ev.queue_seconds = queue_s;
        e->sink->push(std::move(ev));
      }
      if (g.next_tokens) {
        const auto& nt = *g.next_tokens;
        for (size_t i = 0; i < nt.ids.size(); ++i) {
          e->generated.push_back(nt.ids[i]);
          if (gone) continue;
          StreamEvent ev;
          ev.kind = StreamEvent::Token;
          ev.token_id = nt.ids[i];
          ev.logprob = i < nt.logprobs.size() ? nt.logprobs[i] : 0.f;
          ev.text = i < nt.texts.size() ? nt.texts[i] : "";
          ev.special = i < nt.is_special.size() ? nt.is_special[i] : false;
          ev.skipped = i + 1 < nt.ids.size();
          if (i < nt.alternative_tokens.size()) ev.alternatives = nt.alternative_tokens[i];
          ev.queue_seconds = queue_s;
          e->sink->push(std::move(ev));
          if (metrics_ && i + 1 < nt.ids.size()) metrics_->inc("lorax_request_skipped_tokens");
        }
      }
      if (g.generated_text || gone) {
        if (g.generated_text && !gone) {
          StreamEvent ev;
          ev.kind = StreamEvent::End;
          ev.generated_text = g.generated_text;
          ev.queue_seconds = queue_s;
          ev.inference_seconds = std::chrono::duration<double>(Clock::now() - e->batch_time).count();
          e->sink->push(std::move(ev));
        }
        release(e);
        entries.erase(it);
      }
    }
    (void)step_start;
    std::vector<uint64_t> alive;
    for (auto& kv : entries) alive.push_back(kv.first);
    return alive;
  }

  // After a step: tell the shards which requests ended (FilterBatch) or drop the batch (ClearCache).
  std::optional<gen::CachedBatch> filter(std::optional<gen::CachedBatch> cached, EntryMap& entries) {
    if (!cached) return std::nullopt;
    std::vector<uint64_t> keep;
    for (uint64_t id : cached->request_ids) if (entries.count(id)) keep.push_back(id);
    if (keep.size() == cached->request_ids.size()) return cached;
    if (keep.empty()) { client_->clear_cache(cached->id); return std::nullopt; }
    return client_->filter_batch(cached->id, keep);
  }

  void batching_loop() {
    while (running_) {
      std::optional<NextBatch> nb;
      {
        std::unique_lock<std::mutex> g(mu_);
        cv_.wait_for(g, std::chrono::milliseconds(50), [&] { return !running_ || queues_.queued() > 0 || !chunking_.empty(); });
        if (!running_) break;
        nb = next_batch({}, std::nullopt, cfg_.max_batch_prefill_tokens, cfg_.max_batch_total_tokens);
      }
      if (!nb) continue;
      EntryMap entries;
      std::vector<gen::CachedBatch> batches;
      try {
        auto cached = run_prefill(*nb, entries);
        if (cached) batches.push_back(*cached);
        uint32_t waiting_tokens = 1;
        while (running_) {
          bool chunks_pending;
          { std::lock_guard<std::mutex> g(mu_); chunks_pending = !chunking_.empty(); }
          if (batches.empty() && !chunks_pending) break;
          uint32_t batch_size = 0, batch_max_tokens = 0;
          for (auto& b : batches) { batch_size += b.size; batch_max_tokens += b.max_tokens; }
          if (metrics_) { metrics_->set("lorax_batch_current_size", batch_size); metrics_->set("lorax_batch_current_max_tokens", batch_max_tokens); }
          std::optional<size_t> min_size;
          if (waiting_tokens < cfg_.max_waiting_tokens) min_size = (size_t)(batch_size * cfg_.waiting_served_ratio);
          if (cfg_.eager_prefill && min_size) min_size = std::min<size_t>(*min_size, 1);
          if (chunks_pending) min_size.reset();            // the rest of a started prompt does not wait
          uint32_t token_budget = cfg_.max_batch_total_tokens > batch_max_tokens ? cfg_.max_batch_total_tokens - batch_max_tokens : 0;
          std::optional<NextBatch> more;
          if (token_budget > 0) {
            std::set<uint32_t> in_use;
            for (auto& kv : entries) in_use.insert(kv.second->request.adapter.index);
            std::lock_guard<std::mutex> g(mu_);
            if (queues_.queued() > 0 || !chunking_.empty()) more = next_batch(in_use, min_size, cfg_.max_batch_prefill_tokens, token_budget);
          }
          if (more) {
            if (metrics_) metrics_->inc("lorax_batch_concat", {{"reason", min_size ? "backpressure" : "wait_exceeded"}});
            waiting_tokens = 1;
            if (fused_prefill_decode_ && !batches.empty()) {
              // one forward pass on the shards: the new prompts AND one decode step of everything that is running
              for (auto& e : more->entries) entries[e->id] = e;
              auto t0 = Clock::now();
              BatchSpan bs(this, "prefill_decode", entries);
              auto res = client_->prefill(more->batch, std::nullopt, batches);
              bs.finish(res.generations.size());
              if (metrics_) { metrics_->inc("lorax_batch_inference_count", {{"method", "prefill_decode"}}); metrics_->inc("lorax_batch_inference_success", {{"method", "prefill_decode"}}); metrics_->observe("lorax_batch_inference_duration", secs(t0), {{"method", "prefill_decode"}}); }
              deliver(res.generations, entries, t0);
              batches.clear();
              auto next = filter(res.batch, entries);
              if (next) batches.push_back(*next);
              waiting_tokens++;
              continue;
            }
            auto c2 = run_prefill(*more, entries);
            if (c2) batches.push_back(*c2);
          }
          waiting_tokens++;
          if (batches.empty()) continue;                     // only prompt chunks so far: nothing decodes yet
          auto t0 = Clock::now();
          BatchSpan bs(this, "decode", entries);
          auto res = client_->decode(batches);
          bs.finish(res.generations.size());
          if (metrics_) { metrics_->inc("lorax_batch_inference_count", {{"method", "decode"}}); metrics_->inc("lorax_batch_inference_success", {{"method", "decode"}}); metrics_->observe("lorax_batch_inference_duration", secs(t0), {{"method", "decode"}}); }
          deliver(res.generations, entries, t0);
          batches.clear();
          auto next = filter(res.batch, entries);
          if (next) batches.push_back(*next);
        }
        healthy_ = true;
      } catch (const std::exception& ex) {
        healthy_ = false;
        { std::lock_guard<std::mutex> g(mu_); chunking_.clear(); }
        if (metrics_) metrics_->inc("lorax_batch_inference_failure");
        fail_all(entries, std::string("Request failed during generation: ") + ex.what());
        try { client_->clear_cache(std::nullopt); } catch (...) {}
      }
    }
  }

  std::optional<gen::CachedBatch> run_prefill(NextBatch& nb, EntryMap& entries) {
    for (auto& e : nb.entries) entries[e->id] = e;
    auto t0 = Clock::now();
    BatchSpan bs(this, "prefill", entries);
    auto res = client_->prefill(nb.batch, std::nullopt);
    bs.finish(res.generations.size());
    if (metrics_) { metrics_->inc("lorax_batch_inference_count", {{"method", "prefill"}}); metrics_->inc("lorax_batch_inference_success", {{"method", "prefill"}}); metrics_->observe("lorax_batch_inference_duration", secs(t0), {{"method", "prefill"}}); }
    deliver(res.generations, entries, t0);
    return filter(res.batch, entries);
  }
  static double secs(Clock::time_point t0) { return std::chrono::duration<double>(Clock::now() - t0).count(); }

  // One span per shard call of the batching loop, in the loop's own trace, linked to the request spans of the entries in
  // the batch; its context goes to the shards in front of the message.  An exception between construction and `finish`
  // marks the span as failed.
  struct BatchSpan {
    Infer* self;
    telemetry::Span span;
    BatchSpan(Infer* s, const char* method, const EntryMap& entries) : self(s) {
      if (!s->tracer_ || !s->tracer_->enabled()) return;
      span = s->tracer_->start(method, s->loop_ctx_, 3);
      span.set("batch.size", json::Value((long long)entries.size()));
      for (auto& kv : entries) {
        if (span.links.size() >= 32) break;
        if (!kv.second->request.trace_id.empty()) span.links.push_back({kv.second->request.trace_id, kv.second->request.span_id});
      }
      s->client_->set_trace(telemetry::format_traceparent(span.ctx));
    }
    void finish(size_t generations) {
      if (!span.recording()) return;
      span.set("generations", json::Value((long long)generations));
      self->client_->set_trace("");
      self->tracer_->end(span);
      span.ctx = {};
    }
    ~BatchSpan() {
      if (!span.recording()) return;                      // finished (moved out) or tracing off
      span.error = true;
      span.error_message = "shard call failed";
      self->client_->set_trace("");
      self->tracer_->end(span);
    }
  };

  // ---------------------------------------------------------------- adapter loader thread
  struct LoaderCmd {
    enum Kind { Download, Load, Offload } kind;
    AdapterKey adapter;
  };
  void loader_loop() {
    while (running_) {
      LoaderCmd cmd;
      {
        std::unique_lock<std::mutex> g(mu_);
        loader_cv_.wait_for(g, std::chrono::milliseconds(100), [&] { return !running_ || !loader_queue_.empty(); });
        if (!running_) break;
        if (loader_queue_.empty()) continue;
        cmd = loader_queue_.front();
        loader_queue_.pop_front();
      }
      const AdapterKey& a = cmd.adapter;
      try {
        if (cmd.kind == LoaderCmd::Download) {
          gen::DownloadAdapterRequest r;
          r.adapter_parameters = a.params();
          r.adapter_source = a.source_enum();
          if (!a.api_token.empty()) r.api_token = a.api_token;
          auto resp = client_->download_adapter(r);
          std::lock_guard<std::mutex> g(mu_);
          queues_.set_downloaded(a.index, resp.memory_fraction);
        } else if (cmd.kind == LoaderCmd::Load) {
          gen::LoadAdapterRequest r;
          r.adapter_parameters = a.params();
          r.adapter_source = a.source_enum();
          r.adapter_index = a.index;
          if (!a.api_token.empty()) r.api_token = a.api_token;
          client_->load_adapter(r);
          std::lock_guard<std::mutex> g(mu_);
          queues_.set_ready(a.index);
        } else {
          gen::OffloadAdapterRequest r;
          r.adapter_parameters = a.params();
          r.adapter_source = a.source_enum();
          r.adapter_index = a.index;
          client_->offload_adapter(r);
        }
      } catch (const std::exception& ex) {
        std::vector<std::shared_ptr<Entry>> failed;
        {
          std::lock_guard<std::mutex> g(mu_);
          failed = queues_.set_errored(a.index, ex.what());
        }
        {
          std::lock_guard<std::mutex> g(index_mu_);
          adapter_index_.erase(a.identity());      // a later request may retry the download
        }
        for (auto& e : failed) {
          StreamEvent ev;
          ev.kind = StreamEvent::Error;
          ev.error = std::string("adapter '") + (a.ids.empty() ? "" : a.ids[0]) + "' could not be loaded: " + ex.what();
          ev.error_type = "generation";
          e->sink->push(ev);
        }
      }
      cv_.notify_one();
    }
  }

  std::shared_ptr<ShardedClient> client_;
  RouterConfig cfg_;
  Metrics* metrics_;
  std::deque<std::shared_ptr<Entry>> chunking_;      // entries whose prompt is only partly prefilled (guarded by mu_)
  telemetry::Tracer* tracer_ = nullptr;
  telemetry::SpanContext loop_ctx_;        // parent of every batch span: the "batching_task" span of this process
  std::mutex mu_;
  std::condition_variable cv_, loader_cv_;
  AdapterQueues queues_;
  std::unique_ptr<Allocator> allocator_;
  std::deque<LoaderCmd> loader_queue_;
  uint32_t block_size_;
  std::optional<uint32_t> window_;
  uint32_t speculate_;
  bool fused_prefill_decode_ = false;
  bool requires_padding_;
  std::mutex index_mu_;
  std::unordered_map<std::string, uint32_t> adapter_index_;
  uint32_t next_adapter_index_ = 1;
  uint64_t next_id_ = 1, next_batch_id_ = 1;
  std::atomic<bool> running_{false}, healthy_{true};
  std::atomic<size_t> in_flight_{0};
  std::thread batch_thread_, loader_thread_;
  // validation runs on the HTTP worker threads: one generator per thread (a shared one was a data race, found by the
  // ThreadSanitizer build of csrc/host/selftest)
  static uint64_t random_seed() {
    static thread_local std::mt19937_64 rng{std::random_device{}()};
    return rng();
  }
};

}  // namespace lx
