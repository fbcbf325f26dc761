// Scheduler of the embedding / classification routes: inputs of concurrent HTTP calls wait in one queue and a batching thread
// sends them to the shards together, as the reference's batching task does for its Embed / Classify entries
// (router/src/infer.rs embed / classify / classify_batch -> adapter scheduler -> batching_task, router/src/batch.rs
// EmbedBatchEntries / ClassifyBatchEntries).  While one batch is on the shards the next one fills up, so the batch size follows
// the load without a linger time; a batch carries one kind of work, at most `max_batch_prefill_tokens` input tokens and at most
// `max_batch_requests` inputs, in arrival order.  Queue length, batch size, queue time and inference time are reported under the
// same metric names as the generation path.
#pragma once
#include <chrono>
#include <condition_variable>
#include <deque>
#include <future>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "metrics.hpp"
#include "shard_client.hpp"

namespace lx {

struct EncoderInputError : std::runtime_error { using std::runtime_error::runtime_error; };     // the input could not be tokenised

class EncoderBatcher {
 public:
  enum class Kind { Embed, Classify };
  struct Result {
    std::vector<float> embedding;                 // Kind::Embed
    gen::ClassifyPredictionList classes;          // Kind::Classify
  };
  struct Limits {
    uint32_t max_input_length = 1024;
    uint32_t max_batch_tokens = 4096;
    uint32_t max_batch_requests = 256;
    size_t max_queued = 4096;                     // beyond this a request is refused as "overloaded"
  };

  EncoderBatcher(std::shared_ptr<ShardedClient> client, Limits lim, Metrics* metrics)
      : client_(std::move(client)), lim_(lim), metrics_(metrics), thread_([this] { loop(); }) {}
  ~EncoderBatcher() {
    { std::lock_guard<std::mutex> g(mu_); stop_ = true; }
    cv_.notify_all();
    thread_.join();
  }

  // Tokenises in the calling thread (the tokenizer workers bound the parallelism) and queues the input.  The future carries the
  // result, or the exception the batch ended with.  Throws std::overflow_error when the queue is full.
  std::future<Result> submit(Kind kind, const std::string& text) {
    Item it;
    it.kind = kind;
    it.text = text;
    try {
      it.ids = client_->tokenize(text);
    } catch (const std::exception& e) {
      throw EncoderInputError(std::string("tokenizer error ") + e.what());
    }
    if (it.ids.size() > lim_.max_input_length) it.ids.resize(lim_.max_input_length);
    it.enqueued = Clock::now();
    auto fut = it.done.get_future();
    {
      std::lock_guard<std::mutex> g(mu_);
      if (queue_.size() >= lim_.max_queued) throw std::overflow_error("Model is overloaded");
      queue_.push_back(std::move(it));
      if (metrics_) metrics_->set("lorax_queue_length", (double)queue_.size(), {{"kind", "encoder"}});
    }
    cv_.notify_one();
    return fut;
  }
  uint64_t batches() const { return batches_.load(); }

 private:
  using Clock = std::chrono::steady_clock;
  struct Item {
    Kind kind;
    std::string text;
    std::vector<uint32_t> ids;
    Clock::time_point enqueued;
    std::promise<Result> done;
  };
  static double secs(Clock::time_point t0) { return std::chrono::duration<double>(Clock::now() - t0).count(); }

  void loop() {
    while (true) {
      std::vector<Item> batch;
      {
        std::unique_lock<std::mutex> g(mu_);
        cv_.wait(g, [&] { return stop_ || !queue_.empty(); });
        if (queue_.empty()) return;
        const Kind kind = queue_.front().kind;
        size_t tokens = 0;
        while (!queue_.empty() && queue_.front().kind == kind && batch.size() < lim_.max_batch_requests) {
          const size_t n = std::max<size_t>(1, queue_.front().ids.size());
          if (!batch.empty() && tokens + n > lim_.max_batch_tokens) break;
          tokens += n;
          batch.push_back(std::move(queue_.front()));
          queue_.pop_front();
        }
        if (metrics_) metrics_->set("lorax_queue_length", (double)queue_.size(), {{"kind", "encoder"}});
      }
      run(batch);
    }
  }

  void run(std::vector<Item>& items) {
    const Kind kind = items.front().kind;
    const char* method = kind == Kind::Embed ? "embed" : "classify";
    gen::Batch b;
    b.id = 1u << 31 | (uint32_t)(++batches_);
    for (size_t i = 0; i < items.size(); ++i) {
      gen::Request r;
      r.id = i;
      r.inputs = items[i].text;
      r.tokenized_inputs.emplace();
      r.tokenized_inputs->ids = items[i].ids;
      r.truncate = lim_.max_input_length;
      b.requests.push_back(std::move(r));
      if (metrics_) metrics_->observe("lorax_request_queue_duration", secs(items[i].enqueued));
    }
    b.size = (uint32_t)items.size();
    if (metrics_) {
      metrics_->observe("lorax_batch_next_size", (double)items.size());
      metrics_->inc("lorax_batch_inference_count", {{"method", method}});
    }
    const auto t0 = Clock::now();
    try {
      if (kind == Kind::Embed) {
        auto resp = client_->embed(b);
        if (!resp.errorMsg.empty()) throw std::runtime_error(resp.errorMsg);
        if (resp.embeddings.size() != items.size()) throw std::runtime_error("the shard answered " + std::to_string(resp.embeddings.size()) + " embeddings for " + std::to_string(items.size()) + " inputs");
        for (size_t i = 0; i < items.size(); ++i) {
          Result r;
          r.embedding = std::move(resp.embeddings[i].values);
          items[i].done.set_value(std::move(r));
        }
      } else {
        auto resp = client_->classify(b);
        if (!resp.errorMsg.empty()) throw std::runtime_error(resp.errorMsg);
        if (resp.classify_prediction_lists.size() != items.size()) throw std::runtime_error("the shard answered " + std::to_string(resp.classify_prediction_lists.size()) + " prediction lists for " + std::to_string(items.size()) + " inputs");
        for (size_t i = 0; i < items.size(); ++i) {
          Result r;
          r.classes = std::move(resp.classify_prediction_lists[i]);
          items[i].done.set_value(std::move(r));
        }
      }
      if (metrics_) {
        metrics_->inc("lorax_batch_inference_success", {{"method", method}});
        metrics_->observe("lorax_batch_inference_duration", secs(t0), {{"method", method}});
      }
    } catch (...) {
      if (metrics_) metrics_->inc("lorax_batch_inference_failure", {{"method", method}});
      for (auto& it : items) {
        try { it.done.set_exception(std::current_exception()); } catch (const std::future_error&) {}     // already answered
      }
    }
  }

  std::shared_ptr<ShardedClient> client_;
  Limits lim_;
  Metrics* metrics_;
  std::deque<Item> queue_;
  std::mutex mu_;
  std::condition_variable cv_;
  bool stop_ = false;
  std::atomic<uint64_t> batches_{0};
  std::thread thread_;
};

}  // namespace lx
