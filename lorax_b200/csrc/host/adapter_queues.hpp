// Per-adapter request queues and the adapter exchange policy.
//
// Behaviour follows router/src/queue.rs of the reference:
//   * every adapter has its own FIFO and a status  Downloading -> Downloaded -> Ready  (or Errored);
//   * `pending` adapters wait for a slot, `active` adapters are resident on the shards (or being loaded);
//   * update_adapters(): (1) evict active adapters that are idle -- empty queue and no request in the running
//     batch -- but only while other adapters are pending; (2) when the active adapter at the front has held its
//     slot longer than `max_active_time` and others are pending, rotate it out; (3) admit pending adapters while
//     fewer than `max_active_adapters` are active and the adapter's memory cost fits the remaining budget;
//   * next_entry(): among active + Ready adapters, serve the oldest waiting request, preferring adapters that are
//     still inside their time slice.
// The caller (scheduler) turns the returned load / offload lists into shard RPCs.
#pragma once
#include <chrono>
#include <condition_variable>
#include <deque>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <optional>
#include <set>
#include <string>
#include <unordered_map>
#include <vector>

#include "block_allocator.hpp"
#include "pb_gen.hpp"

namespace lx {

using Clock = std::chrono::steady_clock;

inline const char* kBaseModelAdapterId = "__base_model__";

struct AdapterKey {
  std::vector<std::string> ids;          // one id, or several for an on-the-fly merge
  std::vector<float> weights;
  int merge_strategy = 0;
  float density = 0.f;
  int majority_sign_method = 0;
  std::string source = "hub";
  std::string api_token;
  uint32_t index = 0;                    // 0 = base model

  bool is_base() const { return index == 0; }
  // identity: a single id is keyed by the id alone (router/src/lib.rs:127-165 of the reference)
  std::string identity() const {
    std::string k = source + "|";
    for (auto& s : ids) k += s + ",";
    if (ids.size() > 1) {
      k += "|" + std::to_string(merge_strategy) + "|" + std::to_string(density) + "|" + std::to_string(majority_sign_method);
      for (float w : weights) k += "," + std::to_string(w);
    }
    return k;
  }
  gen::AdapterParameters params() const {
    gen::AdapterParameters p;
    p.adapter_ids = ids;
    p.weights = weights;
    p.merge_strategy = merge_strategy;
    p.density = density;
    p.majority_sign_method = majority_sign_method;
    return p;
  }
  int source_enum() const { return source == "s3" ? 1 : source == "local" ? 2 : source == "pbase" ? 3 : 0; }
};

// What the HTTP side receives for one request.
struct StreamEvent {
  enum Kind { Prefill, Token, End, Error } kind = Token;
  gen::NextTokens prefill_tokens;
  uint32_t token_id = 0;
  float logprob = 0.f;
  std::string text;
  bool special = false;
  bool skipped = false;                  // token accepted from a speculation, not sampled in its own step
  std::optional<gen::AlternativeTokens> alternatives;
  std::optional<gen::GeneratedText> generated_text;
  double queue_seconds = 0, inference_seconds = 0;
  std::string error, error_type;
};

class ResponseSink {
 public:
  void push(StreamEvent ev) {
    { std::lock_guard<std::mutex> g(mu_); q_.push_back(std::move(ev)); }
    cv_.notify_one();
  }
  // false on timeout
  bool pop(StreamEvent& ev, int timeout_ms = -1) {
    std::unique_lock<std::mutex> g(mu_);
    if (timeout_ms < 0) cv_.wait(g, [&] { return !q_.empty(); });
    else if (!cv_.wait_for(g, std::chrono::milliseconds(timeout_ms), [&] { return !q_.empty(); })) return false;
    ev = std::move(q_.front());
    q_.pop_front();
    return true;
  }
  void close() { closed_ = true; }       // the client went away: the batching loop filters the request out
  bool closed() const { return closed_; }

 private:
  std::mutex mu_;
  std::condition_variable cv_;
  std::deque<StreamEvent> q_;
  std::atomic<bool> closed_{false};
};

struct ValidRequest {
  std::string inputs;
  std::vector<uint32_t> input_ids;
  uint32_t input_length = 0;
  uint32_t truncate = 0;
  bool decoder_input_details = false;
  gen::NextTokenChooserParameters parameters;
  gen::StoppingCriteriaParameters stopping;
  AdapterKey adapter;
  std::string trace_id, span_id;         // the request's span (empty when tracing is off): batch spans link to it
};

struct Entry {
  uint64_t id = 0;
  ValidRequest request;
  std::shared_ptr<ResponseSink> sink;
  Clock::time_point queue_time = Clock::now();
  Clock::time_point batch_time{};
  std::optional<BlockAllocation> allocation;
  std::vector<uint32_t> generated;       // for the radix trie on free
  uint32_t prefilled = 0;                // prompt tokens whose keys / values the shards hold (chunked prefill)
};

enum class AdapterStatus { Downloading, Downloaded, Ready, Errored };

struct QueueState {
  AdapterKey adapter;
  std::deque<std::shared_ptr<Entry>> entries;
  AdapterStatus status = AdapterStatus::Downloading;
  float cost = 0.f;                      // fraction of the adapter memory reservation
  std::optional<Clock::time_point> activation;
  std::string error;
};

struct AdapterUpdate {
  std::vector<AdapterKey> offload;
  std::vector<AdapterKey> load;
  std::vector<AdapterKey> download;      // adapters seen for the first time
};

class AdapterQueues {
 public:
  AdapterQueues(size_t max_active_adapters, double max_active_seconds, float memory_budget = 1.0f)
      : max_active_(max_active_adapters), max_active_time_(max_active_seconds), budget_(memory_budget) {
    // the base model is always resident and costs nothing
    QueueState base;
    base.adapter.ids = {kBaseModelAdapterId};
    base.status = AdapterStatus::Ready;
    base.activation = Clock::now();
    queues_[0] = std::move(base);
    active_.push_back(0);
  }

  // Returns true when the adapter is new and must be downloaded.
  bool append(const std::shared_ptr<Entry>& e) {
    uint32_t idx = e->request.adapter.index;
    auto it = queues_.find(idx);
    bool is_new = false;
    if (it == queues_.end()) {
      QueueState q;
      q.adapter = e->request.adapter;
      it = queues_.emplace(idx, std::move(q)).first;
      pending_.push_back(idx);
      is_new = true;
    } else if (std::find(active_.begin(), active_.end(), idx) == active_.end() &&
               std::find(pending_.begin(), pending_.end(), idx) == pending_.end()) {
      pending_.push_back(idx);
    }
    it->second.entries.push_back(e);
    return is_new;
  }

  void set_downloaded(uint32_t idx, float cost) {
    auto it = queues_.find(idx);
    if (it == queues_.end()) return;
    it->second.cost = cost;
    if (it->second.status == AdapterStatus::Downloading) it->second.status = AdapterStatus::Downloaded;
  }
  void set_ready(uint32_t idx) {
    auto it = queues_.find(idx);
    if (it != queues_.end()) it->second.status = AdapterStatus::Ready;
  }
  void set_offloaded(uint32_t idx) {
    auto it = queues_.find(idx);
    if (it != queues_.end() && it->second.status == AdapterStatus::Ready) it->second.status = AdapterStatus::Downloaded;
  }
  // Fails every queued request of the adapter and forgets it.  Returns the failed entries.
  std::vector<std::shared_ptr<Entry>> set_errored(uint32_t idx, const std::string& msg) {
    std::vector<std::shared_ptr<Entry>> failed;
    auto it = queues_.find(idx);
    if (it == queues_.end()) return failed;
    for (auto& e : it->second.entries) failed.push_back(e);
    if (std::find(active_.begin(), active_.end(), idx) != active_.end()) budget_ += it->second.cost;
    erase(active_, idx);
    erase(pending_, idx);
    queues_.erase(it);
    (void)msg;
    return failed;
  }

  AdapterUpdate update_adapters(const std::set<uint32_t>& adapters_in_use, Clock::time_point now = Clock::now()) {
    AdapterUpdate up;
    const bool others_waiting = !pending_.empty();
    if (others_waiting) {
      // (1) idle adapters give their slot back
      for (auto it = active_.begin(); it != active_.end();) {
        uint32_t idx = *it;
        QueueState& q = queues_[idx];
        if (idx != 0 && q.entries.empty() && !adapters_in_use.count(idx) && q.status != AdapterStatus::Downloading) {
          up.offload.push_back(q.adapter);
          budget_ += q.cost;
          q.activation.reset();
          set_offloaded(idx);
          it = active_.erase(it);
        } else {
          ++it;
        }
      }
      // (2) time slice of the oldest active adapter is over: rotate it to the back of the pending line
      for (size_t i = 0; i < active_.size(); ++i) {
        uint32_t idx = active_[i];
        if (idx == 0) continue;
        QueueState& q = queues_[idx];
        if (q.activation && std::chrono::duration<double>(now - *q.activation).count() > max_active_time_ &&
            !adapters_in_use.count(idx) && q.status == AdapterStatus::Ready) {
          up.offload.push_back(q.adapter);
          budget_ += q.cost;
          q.activation.reset();
          set_offloaded(idx);
          active_.erase(active_.begin() + i);
          if (!q.entries.empty()) pending_.push_back(idx);
        }
        break;      // only the front non-base adapter is considered per call
      }
    }
    // (3) admit
    for (auto it = pending_.begin(); it != pending_.end();) {
      if (active_.size() >= max_active_ + 1) break;          // +1: the base model does not count
      uint32_t idx = *it;
      QueueState& q = queues_[idx];
      if (q.status == AdapterStatus::Downloading) { ++it; continue; }
      if (q.cost > budget_) break;                              // FIFO admission: do not starve a big adapter
      budget_ -= q.cost;
      q.activation = now;
      active_.push_back(idx);
      up.load.push_back(q.adapter);
      it = pending_.erase(it);
    }
    return up;
  }

  // Oldest waiting request among active + Ready adapters; adapters inside their time slice are preferred.
  std::shared_ptr<Entry> next_entry(Clock::time_point now = Clock::now()) {
    QueueState* best = nullptr;
    bool best_in_slice = false;
    for (uint32_t idx : active_) {
      QueueState& q = queues_[idx];
      if (q.status != AdapterStatus::Ready) continue;
      // drop requests whose client disappeared while they were queued
      while (!q.entries.empty() && q.entries.front()->sink && q.entries.front()->sink->closed()) q.entries.pop_front();
      if (q.entries.empty()) continue;
      bool in_slice = idx == 0 || (q.activation && std::chrono::duration<double>(now - *q.activation).count() <= max_active_time_);
      if (best == nullptr || (in_slice && !best_in_slice) ||
          (in_slice == best_in_slice && q.entries.front()->queue_time < best->entries.front()->queue_time)) {
        best = &q;
        best_in_slice = in_slice;
      }
    }
    if (best == nullptr) return nullptr;
    auto e = best->entries.front();
    best->entries.pop_front();
    return e;
  }
  void push_front(const std::shared_ptr<Entry>& e) { queues_[e->request.adapter.index].entries.push_front(e); }

  size_t queued() const {
    size_t n = 0;
    for (auto& kv : queues_) n += kv.second.entries.size();
    return n;
  }
  size_t active_count() const { return active_.size() - 1; }
  size_t pending_count() const { return pending_.size(); }
  float budget_remaining() const { return budget_; }
  const QueueState* find(uint32_t idx) const { auto it = queues_.find(idx); return it == queues_.end() ? nullptr : &it->second; }
  bool is_active(uint32_t idx) const { return std::find(active_.begin(), active_.end(), idx) != active_.end(); }

 private:
  static void erase(std::deque<uint32_t>& d, uint32_t v) { d.erase(std::remove(d.begin(), d.end(), v), d.end()); }
  size_t max_active_;
  double max_active_time_;
  float budget_;
  std::map<uint32_t, QueueState> queues_;
  std::deque<uint32_t> pending_, active_;
};

}  // namespace lx
