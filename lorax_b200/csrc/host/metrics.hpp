// Prometheus-style metrics registry (counters, gauges, histograms) with text exposition.
// Metric names and bucket layouts follow the reference router (router/src/server.rs:1505-1546 and the
// `metrics::` call sites): 35 geometric duration buckets starting at 0.15 ms, 100 linear buckets for token
// counts, powers of two up to 1024 for batch sizes.
#pragma once
#include <cmath>
#include <map>
#include <mutex>
#include <string>
#include <utility>
#include <vector>

namespace lx {

using Labels = std::vector<std::pair<std::string, std::string>>;

class Metrics {
 public:
  Metrics(uint32_t max_input_length = 1024, uint32_t max_total_tokens = 2048) {
    double v = 0.00015;
    for (int i = 0; i < 35; ++i) { duration_buckets_.push_back(v); v *= 1.5; }
    for (int i = 1; i <= 100; ++i) {
      input_buckets_.push_back((double)max_input_length * i / 100.0);
      total_buckets_.push_back((double)max_total_tokens * i / 100.0);
    }
    for (int b = 1; b <= 1024; b *= 2) batch_buckets_.push_back(b);
  }
  void inc(const std::string& name, const Labels& labels = {}, double by = 1.0) {
    std::lock_guard<std::mutex> g(mu_);
    counters_[key(name, labels)] += by;
  }
  void set(const std::string& name, double v, const Labels& labels = {}) {
    std::lock_guard<std::mutex> g(mu_);
    gauges_[key(name, labels)] = v;
  }
  void observe(const std::string& name, double v, const Labels& labels = {}) {
    std::lock_guard<std::mutex> g(mu_);
    auto& h = hists_[key(name, labels)];
    if (h.counts.empty()) {
      h.bounds = &buckets_for(name);
      h.counts.assign(h.bounds->size() + 1, 0);
    }
    size_t i = 0;
    while (i < h.bounds->size() && v > (*h.bounds)[i]) ++i;
    h.counts[i]++;
    h.sum += v;
    h.n++;
  }
  // Text exposition format.  Built with plain string appends: this code also runs inside a shared library loaded
  // into Python next to other C++ runtimes, where iostream locale state is not safe to rely on.
  std::string render() {
    std::lock_guard<std::mutex> g(mu_);
    std::string o, last;
    for (auto& kv : counters_) { type_line(o, last, base(kv.first), "counter"); o += kv.first + " " + fmt(kv.second) + "\n"; }
    for (auto& kv : gauges_) { type_line(o, last, base(kv.first), "gauge"); o += kv.first + " " + fmt(kv.second) + "\n"; }
    for (auto& kv : hists_) {
      const std::string b = base(kv.first);
      const std::string lbl = labels_of(kv.first);
      const std::string sep = lbl.empty() ? "" : ",";
      type_line(o, last, b, "histogram");
      uint64_t cum = 0;
      for (size_t i = 0; i < kv.second.bounds->size(); ++i) {
        cum += kv.second.counts[i];
        o += b + "_bucket{" + lbl + sep + "le=\"" + fmt((*kv.second.bounds)[i]) + "\"} " + std::to_string(cum) + "\n";
      }
      cum += kv.second.counts.back();
      o += b + "_bucket{" + lbl + sep + "le=\"+Inf\"} " + std::to_string(cum) + "\n";
      o += b + "_sum" + (lbl.empty() ? "" : "{" + lbl + "}") + " " + fmt(kv.second.sum) + "\n";
      o += b + "_count" + (lbl.empty() ? "" : "{" + lbl + "}") + " " + std::to_string(kv.second.n) + "\n";
    }
    return o;
  }

 private:
  struct Hist {
    const std::vector<double>* bounds = nullptr;
    std::vector<uint64_t> counts;
    double sum = 0;
    uint64_t n = 0;
  };
  const std::vector<double>& buckets_for(const std::string& name) const {
    if (name.find("duration") != std::string::npos) return duration_buckets_;
    if (name.find("input_length") != std::string::npos) return input_buckets_;
    if (name.find("batch") != std::string::npos) return batch_buckets_;
    return total_buckets_;
  }
  static std::string key(const std::string& name, const Labels& labels) {
    if (labels.empty()) return name;
    std::string k = name + "{";
    for (size_t i = 0; i < labels.size(); ++i) k += (i ? "," : "") + labels[i].first + "=\"" + labels[i].second + "\"";
    return k + "}";
  }
  static std::string base(const std::string& k) { return k.substr(0, k.find('{')); }
  static std::string labels_of(const std::string& k) {
    auto p = k.find('{');
    return p == std::string::npos ? "" : k.substr(p + 1, k.size() - p - 2);
  }
  static void type_line(std::string& o, std::string& last, const std::string& b, const char* t) {
    if (b != last) { o += "# TYPE " + b + " " + t + "\n"; last = b; }
  }
  static std::string fmt(double v) {
    char buf[32];
    if (v == std::floor(v) && std::fabs(v) < 1e15) snprintf(buf, sizeof buf, "%lld", (long long)v);
    else snprintf(buf, sizeof buf, "%.9g", v);
    return buf;
  }
  std::mutex mu_;
  std::map<std::string, double> counters_, gauges_;
  std::map<std::string, Hist> hists_;
  std::vector<double> duration_buckets_, input_buckets_, total_buckets_, batch_buckets_;
};

}  // namespace lx
