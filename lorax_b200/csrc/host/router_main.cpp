// lorax-router: REST / OpenAI-compatible front end + continuous batching scheduler.
//
// Public surface kept from the reference router (router/src/server.rs:1623-1647, router/src/lib.rs):
//   POST /  /generate  /generate_stream (SSE)  /v1/completions  /v1/chat/completions  /v1/embeddings  /embed
//        /classify  /classify_batch  /tokenize  /invocations
//   GET  /health  /ping  /startup  /info  /metrics  /docs
// with the same request / response JSON shapes, timing headers (x-compute-time, x-time-per-token, ...) and the
// error -> status map (422 validation, 429 overloaded, 424 generation, 500 incomplete generation).
#include <csignal>
#include <cstdio>
#include <cstdlib>
#include <iostream>

#include "openapi_gen.hpp"
#include "http.hpp"
#include "infer.hpp"
#include "chat_template.hpp"
#include "encoder_batcher.hpp"
#include "grpc_client.hpp"
#include "json.hpp"

using namespace lx;
using json::Value;

namespace {

// Reported by /info.  Tokenisation is delegated to shard 0 over its socket, one request at a time per handler thread, so the
// flag sizes nothing here; it is carried for clients that read it back.
int g_validation_workers = 2;

std::atomic<bool> g_stop{false};
void on_signal(int) { g_stop = true; }

struct Args {
  std::map<std::string, std::string> kv;
  std::string get(const std::string& k, const std::string& d = "") const {
    auto it = kv.find(k);
    if (it != kv.end()) return it->second;
    std::string env = k;
    for (auto& c : env) c = c == '-' ? '_' : (char)toupper(c);
    const char* e = getenv(env.c_str());
    return e ? std::string(e) : d;
  }
  long geti(const std::string& k, long d) const { std::string v = get(k); return v.empty() ? d : atol(v.c_str()); }
  double getd(const std::string& k, double d) const { std::string v = get(k); return v.empty() ? d : atof(v.c_str()); }
  bool getb(const std::string& k, bool d) const { std::string v = get(k); return v.empty() ? d : (v == "1" || v == "true" || v == "True"); }
};

Args parse_args(int argc, char** argv) {
  Args a;
  for (int i = 1; i < argc; ++i) {
    std::string s = argv[i];
    if (s.rfind("--", 0) != 0) continue;
    s = s.substr(2);
    size_t eq = s.find('=');
    if (eq != std::string::npos) a.kv[s.substr(0, eq)] = s.substr(eq + 1);
    else if (i + 1 < argc && std::string(argv[i + 1]).rfind("--", 0) != 0) a.kv[s] = argv[++i];
    else a.kv[s] = "true";
  }
  return a;
}

void log_json(const char* level, const std::string& msg) {
  Value v = Value::object();
  v.set("level", level);
  v.set("target", "lorax_router");
  v.set("message", msg);
  std::cerr << v.dump() << std::endl;
}

template <class T>
std::optional<T> opt_num(const Value& v) {
  if (v.is_number()) return (T)v.as_double();
  return std::nullopt;
}

GenerateParams params_from_json(const Value& p) {
  GenerateParams g;
  if (p["adapter_id"].is_string()) g.adapter_id = p["adapter_id"].as_string();
  if (p["adapter_source"].is_string()) g.adapter_source = p["adapter_source"].as_string();
  if (p["api_token"].is_string()) g.api_token = p["api_token"].as_string();
  const Value& m = p["merged_adapters"];
  if (m.is_object()) {
    for (auto& x : m["ids"].items()) g.merged_ids.push_back(x.as_string());
    for (auto& x : m["weights"].items()) g.merged_weights.push_back((float)x.as_double());
    if (m["merge_strategy"].is_string()) g.merge_strategy = m["merge_strategy"].as_string();
    g.density = (float)m["density"].as_double(0.0);
    if (m["majority_sign_method"].is_string()) g.majority_sign_method = m["majority_sign_method"].as_string();
  }
  g.best_of = opt_num<uint32_t>(p["best_of"]);
  g.temperature = opt_num<float>(p["temperature"]);
  g.repetition_penalty = opt_num<float>(p["repetition_penalty"]);
  g.frequency_penalty = opt_num<float>(p["frequency_penalty"]);
  g.presence_penalty = opt_num<float>(p["presence_penalty"]);
  g.top_k = opt_num<int32_t>(p["top_k"]);
  g.top_p = opt_num<float>(p["top_p"]);
  g.typical_p = opt_num<float>(p["typical_p"]);
  g.do_sample = p["do_sample"].as_bool(false);
  g.max_new_tokens = opt_num<uint32_t>(p["max_new_tokens"]);
  g.ignore_eos_token = p["ignore_eos_token"].as_bool(false);
  if (p["return_full_text"].is_bool()) g.return_full_text = p["return_full_text"].as_bool();
  for (auto& s : p["stop"].items()) g.stop.push_back(s.as_string());
  g.truncate = opt_num<uint32_t>(p["truncate"]);
  g.watermark = p["watermark"].as_bool(false);
  g.details = p["details"].as_bool(false);
  g.decoder_input_details = p["decoder_input_details"].as_bool(false);
  g.return_k_alternatives = opt_num<uint32_t>(p["return_k_alternatives"]);
  g.seed = opt_num<uint64_t>(p["seed"]);
  const Value& rf = p["response_format"];
  if (rf.is_object()) {
    std::string t = rf["type"].as_string();
    if (t == "json_object" && rf["schema"].is_object()) g.schema = rf["schema"].dump();
    else if (t == "json_schema") g.schema = (rf["json_schema"]["schema"].is_object() ? rf["json_schema"]["schema"] : rf["schema"]).dump();
    else if (t == "json_object") g.schema = "{\"type\":\"object\"}";
  }
  for (auto& t : p["input_ids"].items()) g.input_ids.push_back((uint32_t)t.as_int());
  return g;
}

const char* finish_reason_name(int r) { return r == 1 ? "eos_token" : r == 2 ? "stop_sequence" : "length"; }
const char* openai_finish_reason(int r) { return r == 0 ? "length" : "stop"; }

struct Collected {
  std::string text;
  int finish_reason = 0;
  uint32_t generated_tokens = 0, skipped_tokens = 0, prompt_tokens = 0;
  std::optional<uint64_t> seed;
  Value prefill = Value::array();
  Value tokens = Value::array();
  double queue_s = 0, inference_s = 0, ttft_s = 0, total_s = 0, validation_s = 0;
  double sum_logprob = 0;
};

Value token_json(const StreamEvent& ev) {
  Value t = Value::object();
  t.set("id", ev.token_id);
  t.set("text", ev.text);
  t.set("logprob", ev.logprob);
  t.set("special", ev.special);
  if (ev.alternatives) {
    Value alts = Value::array();
    for (size_t i = 0; i < ev.alternatives->ids.size(); ++i) {
      Value a = Value::object();
      a.set("id", ev.alternatives->ids[i]);
      a.set("text", i < ev.alternatives->texts.size() ? ev.alternatives->texts[i] : "");
      a.set("logprob", i < ev.alternatives->logprobs.size() ? ev.alternatives->logprobs[i] : 0.f);
      alts.push(a);
    }
    t.set("alternative_tokens", alts);
  }
  if (ev.skipped) t.set("skipped", true);
  return t;
}

class App {
 public:
  App(std::shared_ptr<ShardedClient> client, RouterConfig cfg, gen::InfoResponse info, uint32_t num_blocks,
      const std::string& otlp_endpoint = "", const std::string& request_logger_url = "")
      : client_(client), cfg_(cfg), info_(info), metrics_(cfg.max_input_length, cfg.max_total_tokens),
        infer_(client, cfg, info, num_blocks, &metrics_), tracer_(otlp_endpoint, "lorax.router"),
        request_logger_(telemetry::parse_url(request_logger_url), telemetry::parse_url(request_logger_url).path) {
    infer_.set_tracer(&tracer_);
    infer_.start();
    if (info_.supports_embeddings || info_.supports_classification) {
      EncoderBatcher::Limits lim;
      lim.max_input_length = cfg_.max_input_length;
      lim.max_batch_tokens = std::max(cfg_.max_batch_prefill_tokens, cfg_.max_input_length);
      lim.max_queued = cfg_.max_concurrent_requests ? cfg_.max_concurrent_requests * 4 : 4096;
      encoder_ = std::make_unique<EncoderBatcher>(client_, lim, &metrics_);
    }
  }
  void stop() {
    encoder_.reset();
    infer_.stop();
    tracer_.shutdown();
    request_logger_.stop();
  }
  bool tracing() const { return tracer_.enabled(); }
  // Chat templates rendered by the router itself (the shard's template, compiled at start-up); requests whose template needs
  // something the interpreter lacks still go to shard 0.
  void set_chat_renderer(std::shared_ptr<const jinja::ChatRenderer> r) { chat_renderer_ = std::move(r); }
  uint64_t chat_templates_rendered() const { return chat_rendered_.load(); }

  // Runs one request to completion; `on_event` sees every stream event (used by the SSE routes).
  Collected run(const std::string& inputs, const GenerateParams& p, const std::function<bool(const StreamEvent&)>& on_event = nullptr,
                http::ResponseWriter* w = nullptr) {
    // the request span: child of the caller's trace context when the request carried one
    telemetry::Span span = tracer_.start(on_event ? "generate_stream" : "generate", telemetry::parse_traceparent(p.traceparent), 2);
    try {
      Collected c;
      if (span.recording()) {
        GenerateParams traced = p;
        traced.trace_id = span.ctx.trace_id;
        traced.span_id = span.ctx.span_id;
        c = run_inner(inputs, traced, on_event, w);
      } else {
        c = run_inner(inputs, p, on_event, w);
      }
      if (span.recording()) {
        span.set("total_time_ms", Value(c.total_s * 1e3));
        span.set("queue_time_ms", Value(c.queue_s * 1e3));
        span.set("inference_time_ms", Value(c.inference_s * 1e3));
        span.set("time_to_first_token_ms", Value(c.ttft_s * 1e3));
        span.set("prompt_tokens", Value((long long)c.prompt_tokens));
        span.set("generated_tokens", Value((long long)c.generated_tokens));
        if (c.seed) span.set("seed", Value((unsigned long long)*c.seed));
        if (p.adapter_id) span.set("adapter_id", Value(*p.adapter_id));
        tracer_.end(span);
      }
      log_request(inputs, p, c);
      return c;
    } catch (const std::exception& e) {
      if (span.recording()) {
        span.error = true;
        span.error_message = e.what();
        tracer_.end(span);
      }
      throw;
    }
  }

  // REQUEST_LOGGER_URL: every finished request as one JSON document (reference: server.rs:1314-1349).
  void log_request(const std::string& inputs, const GenerateParams& p, const Collected& c) {
    if (!request_logger_.enabled()) return;
    Value v = Value::object();
    v.set("model_id", cfg_.model_id);
    v.set("adapter_id", p.adapter_id ? Value(*p.adapter_id) : Value());
    v.set("adapter_source", p.adapter_source ? Value(*p.adapter_source) : Value());
    v.set("input", inputs);
    v.set("output", c.text);
    v.set("prompt_tokens", (long long)c.prompt_tokens);
    v.set("generated_tokens", (long long)c.generated_tokens);
    v.set("finish_reason", finish_reason_name(c.finish_reason));
    v.set("total_time_ms", c.total_s * 1e3);
    request_logger_.post(v.dump());
  }

  Collected run_inner(const std::string& inputs, const GenerateParams& p, const std::function<bool(const StreamEvent&)>& on_event,
                      http::ResponseWriter* w) {
    auto t0 = Clock::now();
    ValidRequest valid;
    auto sink = infer_.generate_stream(inputs, p, &valid);
    metrics_.inc("lorax_request_count");
    Collected c;
    c.prompt_tokens = valid.input_length;
    c.validation_s = std::chrono::duration<double>(Clock::now() - t0).count();      // tokenisation and parameter checks
    metrics_.observe("lorax_request_validation_duration", c.validation_s);
    metrics_.observe("lorax_request_max_new_tokens", valid.stopping.max_new_tokens);
    struct Done { Infer& i; ~Done() { i.request_done(); } } done{infer_};
    bool first = true;
    while (true) {
      StreamEvent ev;
      if (!sink->pop(ev, 250)) {
        if (w && w->peer_closed()) { sink->close(); throw ApiError("client disconnected", "incomplete_generation", 499); }
        continue;
      }
      if (ev.kind == StreamEvent::Error) {
        metrics_.inc("lorax_request_failure", {{"err", ev.error_type}});
        throw ApiError(ev.error, ev.error_type, ev.error_type == "validation" ? 422 : 424);
      }
      if (ev.kind == StreamEvent::Prefill) {
        for (size_t i = 0; i < ev.prefill_tokens.ids.size(); ++i) {
          Value t = Value::object();
          t.set("id", ev.prefill_tokens.ids[i]);
          t.set("text", i < ev.prefill_tokens.texts.size() ? ev.prefill_tokens.texts[i] : "");
          if (i == 0) t.set("logprob", Value());
          else t.set("logprob", i < ev.prefill_tokens.logprobs.size() ? ev.prefill_tokens.logprobs[i] : 0.f);
          c.prefill.push(t);
        }
        continue;
      }
      if (ev.kind == StreamEvent::Token) {
        if (first) { c.ttft_s = std::chrono::duration<double>(Clock::now() - t0).count(); first = false; }
        c.tokens.push(token_json(ev));
        c.sum_logprob += ev.logprob;
        c.queue_s = ev.queue_seconds;
        if (on_event && !on_event(ev)) { sink->close(); throw ApiError("client disconnected", "incomplete_generation", 499); }
        continue;
      }
      // End
      c.text = ev.generated_text->text;
      c.finish_reason = ev.generated_text->finish_reason;
      c.generated_tokens = ev.generated_text->generated_tokens;
      c.skipped_tokens = ev.generated_text->skipped_tokens;
      c.seed = ev.generated_text->seed;
      c.queue_s = ev.queue_seconds;
      c.inference_s = ev.inference_seconds;
      c.total_s = std::chrono::duration<double>(Clock::now() - t0).count();
      if (on_event) on_event(ev);
      break;
    }
    metrics_.inc("lorax_request_success");
    metrics_.observe("lorax_request_duration", c.total_s);
    metrics_.observe("lorax_request_queue_duration", c.queue_s);
    metrics_.observe("lorax_request_inference_duration", c.inference_s);
    if (c.generated_tokens) metrics_.observe("lorax_request_mean_time_per_token_duration", c.inference_s / c.generated_tokens);
    metrics_.observe("lorax_request_generated_tokens", c.generated_tokens);
    metrics_.observe("lorax_request_input_length", c.prompt_tokens);
    return c;
  }

  Value details_json(const Collected& c, const GenerateParams& p) {
    Value d = Value::object();
    d.set("finish_reason", finish_reason_name(c.finish_reason));
    d.set("prompt_tokens", c.prompt_tokens);
    d.set("generated_tokens", c.generated_tokens);
    d.set("skipped_tokens", c.skipped_tokens);
    d.set("seed", c.seed ? Value((unsigned long long)*c.seed) : Value());
    d.set("prefill", p.decoder_input_details ? c.prefill : Value::array());
    d.set("tokens", c.tokens);
    return d;
  }
  http::ResponseWriter::Headers timing_headers(const Collected& c, const GenerateParams& p) {
    auto ms = [](double s) { return std::to_string((long long)(s * 1000.0)); };
    http::ResponseWriter::Headers h = {
        {"x-compute-type", info_.device_type.empty() ? "gpu+optimized" : info_.device_type + "+optimized"},
        {"x-compute-time", ms(c.total_s)},
        {"x-compute-characters", std::to_string(c.text.size())},
        {"x-total-time", ms(c.total_s)},
        {"x-validation-time", ms(c.validation_s)},
        {"x-queue-time", ms(c.queue_s)},
        {"x-inference-time", ms(c.inference_s)},
        {"x-time-per-token", ms(c.generated_tokens ? c.inference_s / c.generated_tokens : 0)},
        {"x-time-to-first-token", ms(c.ttft_s)},
        {"x-prompt-tokens", std::to_string(c.prompt_tokens)},
        {"x-generated-tokens", std::to_string(c.generated_tokens)},
        {"x-total-tokens", std::to_string(c.prompt_tokens + c.generated_tokens)},
        {"x-model-id", cfg_.model_id},
    };
    if (p.adapter_id) h.push_back({"x-adapter-id", *p.adapter_id});
    if (p.adapter_source) h.push_back({"x-adapter-source", *p.adapter_source});
    return h;
  }
  static void send_error(http::ResponseWriter& w, const ApiError& e) {
    Value v = Value::object();
    v.set("error", e.what());
    v.set("error_type", e.type);
    if (w.streaming()) w.event(v.dump());
    else if (!w.started()) w.send(e.status == 499 ? 500 : e.status, v.dump());
  }
  bool parse_body(const http::Request& req, http::ResponseWriter& w, Value& body) {
    std::string err;
    if (!json::parse(req.body, body, &err) || !body.is_object()) {
      send_error(w, ApiError("Failed to parse the request body as JSON: " + err, "validation", 422));
      return false;
    }
    return true;
  }
  void apply_auth(const http::Request& req, GenerateParams& p) {
    if (!p.api_token) {
      std::string a = req.header("authorization");
      if (a.rfind("Bearer ", 0) == 0) p.api_token = a.substr(7);
    }
  }

  // ---------------------------------------------------------------- native API
  void generate(const http::Request& req, http::ResponseWriter& w) {
    Value body;
    if (!parse_body(req, w, body)) return;
    GenerateParams p = params_from_json(body["parameters"]);
    p.traceparent = req.header("traceparent");
    apply_auth(req, p);
    if (body["stream"].as_bool(false)) return generate_stream_body(body, p, w);
    try {
      uint32_t n = p.best_of.value_or(1);
      std::vector<Collected> all;
      if (n > 1) {
        std::vector<std::future<Collected>> futs;
        for (uint32_t i = 0; i < n; ++i) {
          GenerateParams pi = p;
          pi.best_of.reset();
          pi.do_sample = true;
          futs.push_back(std::async(std::launch::async, [this, pi, &body] { return run(body["inputs"].as_string(), pi); }));
        }
        for (auto& f : futs) all.push_back(f.get());
        std::sort(all.begin(), all.end(), [](const Collected& a, const Collected& b) {
          return a.sum_logprob / std::max(1u, a.generated_tokens) > b.sum_logprob / std::max(1u, b.generated_tokens);
        });
      } else {
        all.push_back(run(body["inputs"].as_string(), p, nullptr, &w));
      }
      const Collected& c = all.front();
      Value out = Value::object();
      std::string text = c.text;
      if (p.return_full_text.value_or(false)) text = body["inputs"].as_string() + text;
      out.set("generated_text", text);
      if (p.details) {
        Value d = details_json(c, p);
        if (all.size() > 1) {
          Value seqs = Value::array();
          for (size_t i = 1; i < all.size(); ++i) {
            Value s = details_json(all[i], p);
            s.set("generated_text", all[i].text);
            seqs.push(s);
          }
          d.set("best_of_sequences", seqs);
        }
        out.set("details", d);
      }
      w.send(200, out.dump(), "application/json", timing_headers(c, p));
    } catch (const ApiError& e) {
      send_error(w, e);
    }
  }

  void generate_stream(const http::Request& req, http::ResponseWriter& w) {
    Value body;
    if (!parse_body(req, w, body)) return;
    GenerateParams p = params_from_json(body["parameters"]);
    p.traceparent = req.header("traceparent");
    apply_auth(req, p);
    generate_stream_body(body, p, w);
  }
  void generate_stream_body(const Value& body, const GenerateParams& p, http::ResponseWriter& w) {
    if (p.best_of.value_or(1) > 1) return send_error(w, ApiError("`best_of` != 1 is not supported when streaming tokens", "validation", 422));
    w.begin_stream(200, {{"x-accel-buffering", "no"}});
    try {
      // Each token event is held back until the next one arrives, so that the last token can be sent together
      // with the generated text and the details (the stream's final message carries all three).
      std::optional<Value> pending;
      uint32_t n_tokens = 0;
      run(body["inputs"].as_string(), p, [&](const StreamEvent& ev) {
        bool ok = true;
        if (ev.kind == StreamEvent::Token) {
          if (pending) ok = w.event(pending->dump());
          Value out = Value::object();
          out.set("token", token_json(ev));
          out.set("generated_text", Value());
          out.set("details", Value());
          pending = out;
          ++n_tokens;
        } else if (ev.kind == StreamEvent::End && pending) {
          pending->set("generated_text", ev.generated_text->text);
          if (p.details) {
            Value d = Value::object();
            d.set("finish_reason", finish_reason_name(ev.generated_text->finish_reason));
            d.set("generated_tokens", ev.generated_text->generated_tokens);
            d.set("skipped_tokens", ev.generated_text->skipped_tokens);
            d.set("seed", ev.generated_text->seed ? Value((unsigned long long)*ev.generated_text->seed) : Value());
            pending->set("details", d);
          }
          ok = w.event(pending->dump());
          pending.reset();
        }
        return ok;
      }, &w);
    } catch (const ApiError& e) {
      send_error(w, e);
    }
  }

  // ---------------------------------------------------------------- OpenAI compatible
  void completions(const http::Request& req, http::ResponseWriter& w) {
    Value body;
    if (!parse_body(req, w, body)) return;
    GenerateParams p = openai_params(body);
    p.traceparent = req.header("traceparent");
    apply_auth(req, p);
    std::string prompt = body["prompt"].is_array() ? body["prompt"].items().front().as_string() : body["prompt"].as_string();
    openai_run(body, prompt, p, w, false);
  }
  void chat_completions(const http::Request& req, http::ResponseWriter& w) {
    Value body;
    if (!parse_body(req, w, body)) return;
    GenerateParams p = openai_params(body);
    p.traceparent = req.header("traceparent");
    apply_auth(req, p);
    // tools -> JSON schema grammar: {"_name": const tool name, ...arguments} or the no_tool fallback
    if (body["tools"].is_array() && body["tools"].size() > 0 && !body["response_format"].is_object())
      p.schema = tool_schema(body["tools"], body["tool_choice"]);
    std::string prompt;
    try {
      Value treq = Value::object();
      treq.set("messages", body["messages"]);
      // a response_format takes precedence over tools: the template is then applied without them (server.rs:436-440 of the reference)
      if (body["tools"].is_array() && !body["response_format"].is_object()) treq.set("tools", body["tools"]);
      if (body["tool_prompt"].is_string()) treq.set("tool_prompt", body["tool_prompt"]);
      if (body["guideline"].is_string()) treq.set("guideline", body["guideline"]);
      treq.set("adapter_id", p.adapter_id ? Value(*p.adapter_id) : Value());
      bool rendered = false;
      if (chat_renderer_) {
        try {
          prompt = chat_renderer_->render(treq);
          rendered = true;
          ++chat_rendered_;
        } catch (const jinja::Unsupported&) {
          // this request needs a part of Jinja the router lacks: the shard renders it
        }
      }
      if (!rendered) prompt = client_->helper(102, treq.dump());
    } catch (const std::exception& e) {
      return send_error(w, ApiError(std::string("chat template error: ") + e.what(), "template_error", 422));
    }
    openai_run(body, prompt, p, w, true);
  }
  GenerateParams openai_params(const Value& b) {
    GenerateParams p;
    std::string model = b["model"].as_string();
    if (!model.empty() && model != cfg_.model_id) p.adapter_id = model;      // `model` names the adapter
    if (b["adapter_source"].is_string()) p.adapter_source = b["adapter_source"].as_string();
    if (b["api_token"].is_string()) p.api_token = b["api_token"].as_string();
    p.max_new_tokens = opt_num<uint32_t>(b["max_tokens"]);
    if (!p.max_new_tokens) p.max_new_tokens = opt_num<uint32_t>(b["max_completion_tokens"]);
    p.temperature = opt_num<float>(b["temperature"]);
    p.top_p = opt_num<float>(b["top_p"]);
    if (p.top_p && *p.top_p >= 1.0f) p.top_p.reset();
    p.frequency_penalty = opt_num<float>(b["frequency_penalty"]);
    p.presence_penalty = opt_num<float>(b["presence_penalty"]);
    p.repetition_penalty = opt_num<float>(b["repetition_penalty"]);
    p.top_k = opt_num<int32_t>(b["top_k"]);
    p.seed = opt_num<uint64_t>(b["seed"]);
    p.ignore_eos_token = b["ignore_eos_token"].as_bool(false);
    if (b["stop"].is_string()) p.stop.push_back(b["stop"].as_string());
    for (auto& s : b["stop"].items()) p.stop.push_back(s.as_string());
    p.do_sample = p.temperature && *p.temperature > 0.f;
    p.details = true;
    if (b["logprobs"].is_number()) p.return_k_alternatives = (uint32_t)b["logprobs"].as_int();
    if (b["top_logprobs"].is_number()) p.return_k_alternatives = (uint32_t)b["top_logprobs"].as_int();
    const Value& rf = b["response_format"];
    if (rf.is_object()) {
      Value wrap = Value::object();
      wrap.set("response_format", rf);
      p.schema = params_from_json(wrap).schema;
    }
    return p;
  }
  static std::string tool_schema(const Value& tools, const Value& choice) {
    Value any = Value::array();
    for (auto& t : tools.items()) {
      const Value& f = t["function"];
      if (choice.is_object() && choice["function"]["name"].as_string() != f["name"].as_string()) continue;
      Value props = Value::object();
      Value name = Value::object();
      name.set("type", "string");
      name.set("const", f["name"].as_string());
      props.set("_name", name);
      Value required = Value::array();
      required.push("_name");
      for (auto& kv : f["parameters"]["properties"].members()) props.set(kv.first, kv.second);
      for (auto& r : f["parameters"]["required"].items()) required.push(r);
      Value s = Value::object();
      s.set("type", "object");
      s.set("properties", props);
      s.set("required", required);
      any.push(s);
    }
    if (!choice.is_object() && choice.as_string() != "required") {
      Value props = Value::object();
      Value name = Value::object();
      name.set("type", "string");
      name.set("const", "no_tool");
      props.set("_name", name);
      Value content = Value::object();
      content.set("type", "string");
      props.set("content", content);
      Value req = Value::array();
      req.push("_name");
      req.push("content");
      Value s = Value::object();
      s.set("type", "object");
      s.set("properties", props);
      s.set("required", req);
      any.push(s);
    }
    Value schema = Value::object();
    schema.set("anyOf", any);
    return schema.dump();
  }
  void openai_run(const Value& body, const std::string& prompt, const GenerateParams& p, http::ResponseWriter& w, bool chat) {
    const bool stream = body["stream"].as_bool(false);
    const std::string id = (chat ? "chatcmpl-" : "cmpl-") + std::to_string(++openai_id_);
    const long long created = (long long)time(nullptr);
    const std::string model = body["model"].as_string().empty() ? cfg_.model_id : body["model"].as_string();
    auto envelope = [&](const char* object) {
      Value o = Value::object();
      o.set("id", id);
      o.set("object", object);
      o.set("created", created);
      o.set("model", model);
      return o;
    };
    try {
      if (stream) {
        w.begin_stream(200, {{"x-accel-buffering", "no"}});
        Collected c = run(prompt, p, [&](const StreamEvent& ev) {
          if (ev.kind != StreamEvent::Token && ev.kind != StreamEvent::End) return true;
          Value o = envelope(chat ? "chat.completion.chunk" : "text_completion");
          Value choice = Value::object();
          choice.set("index", 0);
          const std::string text = ev.kind == StreamEvent::Token ? ev.text : "";
          if (chat) {
            Value delta = Value::object();
            if (ev.kind == StreamEvent::Token) { delta.set("role", "assistant"); delta.set("content", text); }
            choice.set("delta", delta);
          } else {
            choice.set("text", text);
          }
          choice.set("finish_reason", ev.kind == StreamEvent::End ? Value(openai_finish_reason(ev.generated_text->finish_reason)) : Value());
          Value choices = Value::array();
          choices.push(choice);
          o.set("choices", choices);
          return w.event(o.dump());
        }, &w);
        (void)c;
        w.event("[DONE]");
        return;
      }
      Collected c = run(prompt, p, nullptr, &w);
      Value o = envelope(chat ? "chat.completion" : "text_completion");
      Value choice = Value::object();
      choice.set("index", 0);
      if (chat) {
        Value msg = Value::object();
        msg.set("role", "assistant");
        Value parsed;
        if (body["tools"].is_array() && body["tools"].size() > 0 && json::parse(c.text, parsed) && parsed.is_object() &&
            parsed["_name"].is_string() && parsed["_name"].as_string() != "no_tool") {
          Value args = Value::object();
          for (auto& kv : parsed.members()) if (kv.first != "_name") args.set(kv.first, kv.second);
          Value fn = Value::object();
          fn.set("name", parsed["_name"].as_string());
          fn.set("arguments", args.dump());
          Value call = Value::object();
          call.set("id", "call_" + std::to_string(openai_id_.load()));
          call.set("type", "function");
          call.set("function", fn);
          Value calls = Value::array();
          calls.push(call);
          msg.set("content", Value());
          msg.set("tool_calls", calls);
        } else if (parsed.is_object() && parsed["_name"].as_string() == "no_tool") {
          msg.set("content", parsed["content"].as_string());
        } else {
          msg.set("content", c.text);
        }
        choice.set("message", msg);
      } else {
        // `echo`: the completion is returned behind its prompt (return_full_text, server.rs:1272 of the reference)
        choice.set("text", body["echo"].is_bool() && body["echo"].as_bool() ? prompt + c.text : c.text);
      }
      choice.set("finish_reason", openai_finish_reason(c.finish_reason));
      Value choices = Value::array();
      choices.push(choice);
      o.set("choices", choices);
      Value usage = Value::object();
      usage.set("prompt_tokens", c.prompt_tokens);
      usage.set("completion_tokens", c.generated_tokens);
      usage.set("total_tokens", c.prompt_tokens + c.generated_tokens);
      o.set("usage", usage);
      w.send(200, o.dump(), "application/json", timing_headers(c, p));
    } catch (const ApiError& e) {
      send_error(w, e);
    }
  }

  // ---------------------------------------------------------------- embeddings / classification
  // Token classes -> entities, the "simple" aggregation of the reference (router/src/infer.rs:1765-1819): a B- tag, or a tag that
  // differs from the open entity's group, starts an entity at the token's character offsets; other tokens extend the open
  // entity (end offset, mean score); an untagged class counts as group "0", so a run of them after an entity becomes an
  // entity of that group, as it does there.  `word` is the lower-cased text span.  The class list carries one entry per token
  // of the input as the shard tokenised it, with the tokenizer's special tokens at both ends when it adds any.
  Value aggregate_entities(const std::string& input, const gen::ClassifyPredictionList& l) {
    Value q = Value::object();
    q.set("inputs", input);
    q.set("add_special_tokens", false);
    Value toks;
    std::string err;
    if (!json::parse(client_->helper(101, q.dump()), toks) || !toks.is_array()) toks = Value::array();
    const size_t n_tok = toks.size();
    const size_t skip = l.predictions.size() >= n_tok + 2 ? 1 : 0;          // [CLS] ... [SEP]
    struct Ent { std::string group; float score; size_t start, end; };
    std::vector<Ent> ents;
    bool open = false;
    Ent cur{};
    std::vector<float> scores;
    for (size_t i = 0; i < n_tok && i + skip < l.predictions.size(); ++i) {
      const std::string& cls = l.predictions[i + skip];
      const float score = i + skip < l.scores.size() ? l.scores[i + skip] : 0.f;
      std::string bi = "0", tag = "0";
      const size_t dash = cls.find('-');
      if (dash != std::string::npos && cls.find('-', dash + 1) == std::string::npos) { bi = cls.substr(0, dash); tag = cls.substr(dash + 1); }
      const size_t a = (size_t)toks.items()[i]["start"].as_int(0), b = (size_t)toks.items()[i]["stop"].as_int(0);
      if (bi == "B" || (open && tag != cur.group)) {
        if (open) { ents.push_back(cur); scores.clear(); scores.push_back(score); }
        cur = Ent{tag, score, a, b};
        open = true;
      } else if (open) {
        scores.push_back(score);
        float sum = 0.f;
        for (float f : scores) sum += f;
        cur.score = sum / (float)scores.size();
        cur.end = b;
      }
    }
    if (open) ents.push_back(cur);
    Value out = Value::array();
    for (auto& e : ents) {
      Value v = Value::object();
      v.set("entity_group", e.group);
      v.set("score", e.score);
      std::string word = (e.start <= e.end && e.end <= input.size()) ? input.substr(e.start, e.end - e.start) : "";
      for (auto& ch : word) ch = (char)std::tolower((unsigned char)ch);
      v.set("word", word);
      v.set("start", (unsigned long long)e.start);
      v.set("end", (unsigned long long)e.end);
      out.push(v);
    }
    return out;
  }
  gen::Batch one_shot_batch(const std::vector<std::string>& inputs) {
    gen::Batch b;
    b.id = 1u << 31 | (uint32_t)(++openai_id_);
    for (size_t i = 0; i < inputs.size(); ++i) {
      gen::Request r;
      r.id = i;
      r.inputs = inputs[i];
      r.tokenized_inputs.emplace();
      r.tokenized_inputs->ids = client_->tokenize(inputs[i]);
      r.truncate = cfg_.max_input_length;
      b.requests.push_back(r);
    }
    b.size = (uint32_t)inputs.size();
    return b;
  }
  void embed(const http::Request& req, http::ResponseWriter& w, bool openai) {
    Value body;
    if (!parse_body(req, w, body)) return;
    if (!info_.supports_embeddings) return send_error(w, ApiError("this model does not support embeddings", "validation", 422));
    std::vector<std::string> inputs;
    const Value& in = openai ? body["input"] : body["inputs"];
    if (in.is_array()) for (auto& s : in.items()) inputs.push_back(s.as_string());
    else inputs.push_back(in.as_string());
    try {
      // every input joins the encoder queue; inputs of concurrent calls share shard batches
      gen::EmbedResponse resp;
      {
        std::vector<std::future<EncoderBatcher::Result>> futs;
        for (auto& in_text : inputs) futs.push_back(encoder_->submit(EncoderBatcher::Kind::Embed, in_text));
        for (auto& f : futs) {
          gen::Embedding e;
          e.values = f.get().embedding;
          resp.embeddings.push_back(std::move(e));
        }
      }
      metrics_.observe("lorax_request_input_count", (double)inputs.size());
      Value out = Value::object();
      if (openai) {
        Value data = Value::array();
        for (size_t i = 0; i < resp.embeddings.size(); ++i) {
          Value e = Value::object();
          e.set("object", "embedding");
          e.set("index", (int)i);
          Value vals = Value::array();
          for (float f : resp.embeddings[i].values) vals.push(f);
          e.set("embedding", vals);
          data.push(e);
        }
        out.set("object", "list");
        out.set("data", data);
        out.set("model", cfg_.model_id);
      } else {
        Value vals = Value::array();
        if (!resp.embeddings.empty()) for (float f : resp.embeddings[0].values) vals.push(f);
        out.set("embeddings", vals);
      }
      w.send(200, out.dump());
    } catch (const ApiError& e) {
      send_error(w, e);
    } catch (const EncoderInputError& e) {
      send_error(w, ApiError(e.what(), "validation", 422));
    } catch (const std::overflow_error& e) {
      metrics_.inc("lorax_request_failure", {{"err", "overloaded"}});
      send_error(w, ApiError(e.what(), "overloaded", 429));
    } catch (const std::exception& e) {
      send_error(w, ApiError(e.what(), "generation", 424));
    }
  }
  void classify(const http::Request& req, http::ResponseWriter& w, bool batch) {
    Value body;
    if (!parse_body(req, w, body)) return;
    if (!info_.supports_classification) return send_error(w, ApiError("this model does not support classification", "validation", 422));
    std::vector<std::string> inputs;
    if (batch) for (auto& s : body["inputs"].items()) inputs.push_back(s.as_string());
    else inputs.push_back(body["inputs"].as_string());
    try {
      auto t0 = Clock::now();
      gen::ClassifyResponse resp;
      {
        std::vector<std::future<EncoderBatcher::Result>> futs;
        for (auto& in_text : inputs) futs.push_back(encoder_->submit(EncoderBatcher::Kind::Classify, in_text));
        for (auto& f : futs) resp.classify_prediction_lists.push_back(f.get().classes);
      }
      metrics_.observe("lorax_request_input_count", (double)inputs.size());
      metrics_.observe("lorax_request_inference_duration", std::chrono::duration<double>(Clock::now() - t0).count());
      size_t n_out = 0;
      for (auto& l : resp.classify_prediction_lists) n_out += l.predictions.size();
      metrics_.observe("lorax_request_classify_output_count", (double)n_out);
      Value all = Value::array();
      for (size_t li = 0; li < resp.classify_prediction_lists.size(); ++li) {
        auto& l = resp.classify_prediction_lists[li];
        bool bio = false;
        for (auto& pr : l.predictions) bio = bio || pr.find('-') != std::string::npos;
        if (bio && li < inputs.size()) {
          all.push(aggregate_entities(inputs[li], l));
          continue;
        }
        // labels without a B- / I- prefix: one entry per token
        Value ents = Value::array();
        for (size_t i = 0; i < l.predictions.size(); ++i) {
          Value e = Value::object();
          e.set("entity_group", l.predictions[i]);
          e.set("score", i < l.scores.size() ? l.scores[i] : 0.f);
          e.set("index", (int)i);
          ents.push(e);
        }
        all.push(ents);
      }
      w.send(200, batch ? all.dump() : (all.size() ? all.items()[0].dump() : "[]"));
    } catch (const ApiError& e) {
      send_error(w, e);
    } catch (const EncoderInputError& e) {
      send_error(w, ApiError(e.what(), "validation", 422));
    } catch (const std::overflow_error& e) {
      metrics_.inc("lorax_request_failure", {{"err", "overloaded"}});
      send_error(w, ApiError(e.what(), "overloaded", 429));
    } catch (const std::exception& e) {
      send_error(w, ApiError(e.what(), "generation", 424));
    }
  }

  // ---------------------------------------------------------------- misc routes
  void tokenize(const http::Request& req, http::ResponseWriter& w) {
    Value body;
    if (!parse_body(req, w, body)) return;
    try {
      std::string out = client_->helper(101, body.dump());     // shard 0 returns [{id,text,start,stop}]
      w.send(200, out);
    } catch (const std::exception& e) {
      send_error(w, ApiError(e.what(), "validation", 422));
    }
  }
  void health(http::ResponseWriter& w) {
    if (infer_.healthy()) return (void)w.send(200, "");
    try {
      client_->health();
      w.send(200, "");
    } catch (...) {
      w.send(503, "{\"error\":\"unhealthy\",\"error_type\":\"healthcheck\"}");
    }
  }
  // Startup probe: one real request through the whole stack, the kind the model serves (a one-token generation, an
  // embedding or a classification of "Hello"), as the reference's probe does (router/src/server.rs:488-588); a shard that
  // answers Health but cannot run a batch keeps the pod out of rotation.
  void startup(http::ResponseWriter& w) {
    try {
      if (info_.supports_embeddings) {
        auto resp = client_->embed(one_shot_batch({"Hello"}));
        if (!resp.errorMsg.empty()) throw std::runtime_error(resp.errorMsg);
      } else if (info_.supports_classification) {
        auto resp = client_->classify(one_shot_batch({"Hello"}));
        if (!resp.errorMsg.empty()) throw std::runtime_error(resp.errorMsg);
      } else {
        GenerateParams p;
        p.max_new_tokens = 1;
        (void)run("Hello", p);
      }
      w.send(200, "");
    } catch (const std::exception& e) {
      Value v = Value::object();
      v.set("error", std::string("unhealthy: ") + e.what());
      v.set("error_type", "healthcheck");
      w.send(503, v.dump());
    }
  }
  void info(http::ResponseWriter& w) {
    Value v = Value::object();
    v.set("model_id", cfg_.model_id);
    v.set("model_dtype", info_.dtype);
    v.set("model_device_type", info_.device_type);
    v.set("max_concurrent_requests", (unsigned long long)cfg_.max_concurrent_requests);
    v.set("max_best_of", cfg_.max_best_of);
    v.set("max_stop_sequences", cfg_.max_stop_sequences);
    v.set("max_input_length", cfg_.max_input_length);
    v.set("max_total_tokens", cfg_.max_total_tokens);
    v.set("waiting_served_ratio", cfg_.waiting_served_ratio);
    v.set("max_batch_total_tokens", cfg_.max_batch_total_tokens);
    v.set("max_waiting_tokens", cfg_.max_waiting_tokens);
    v.set("block_size", info_.block_size);
    v.set("window_size", info_.window_size ? Value(*info_.window_size) : Value());
    v.set("validation_workers", g_validation_workers);
    v.set("version", "0.1.0");
    v.set("docker_label", Value());
    v.set("request_logger_url", Value());
    v.set("eager_prefill", cfg_.eager_prefill);
    w.send(200, v.dump());
  }
  Metrics& metrics() { return metrics_; }

 private:
  std::shared_ptr<ShardedClient> client_;
  RouterConfig cfg_;
  gen::InfoResponse info_;
  Metrics metrics_;
  Infer infer_;
  telemetry::Tracer tracer_;
  telemetry::BackgroundPoster request_logger_;
  std::unique_ptr<EncoderBatcher> encoder_;       // queue + batching thread of /embed and /classify
  std::shared_ptr<const jinja::ChatRenderer> chat_renderer_;
  std::atomic<uint64_t> chat_rendered_{0};
  std::atomic<uint64_t> openai_id_{0};
};

// the OpenAPI document of docs/reference/openapi.json, embedded at build time
static std::string open_api_document() {
  std::string doc;
  for (const char* const* c = kOpenApiChunks; *c != nullptr; ++c) doc += *c;
  return doc;
}

}  // namespace

static lx::ShardedClient connect_grpc(const std::string& uds_path, int num_shards) {
  std::vector<std::shared_ptr<lx::ShardClient>> v;
  for (int r = 0; r < num_shards; ++r) {
    auto framed = std::make_shared<lx::FramedUdsClient>(uds_path + "-" + std::to_string(r) + ".lx");
    v.push_back(std::make_shared<lx::GrpcUdsClient>(uds_path + "-" + std::to_string(r), framed));
  }
  return lx::ShardedClient(std::move(v));
}

int main(int argc, char** argv) {
  Args a = parse_args(argc, argv);
  if (a.kv.count("help")) {
    std::cout << "lorax-router --port N --master-shard-uds-path PATH --num-shard N [--max-input-length ..] (flags also read from env)\n";
    return 0;
  }
  signal(SIGINT, on_signal);
  signal(SIGTERM, on_signal);
  signal(SIGPIPE, SIG_IGN);
  RouterConfig cfg;
  cfg.max_concurrent_requests = (size_t)a.geti("max-concurrent-requests", 1024);
  cfg.max_best_of = (uint32_t)a.geti("max-best-of", 2);
  cfg.max_stop_sequences = (uint32_t)a.geti("max-stop-sequences", 4);
  cfg.max_input_length = (uint32_t)a.geti("max-input-length", 1024);
  cfg.max_total_tokens = (uint32_t)a.geti("max-total-tokens", 2048);
  cfg.max_batch_prefill_tokens = (uint32_t)a.geti("max-batch-prefill-tokens", 4096);
  cfg.max_batch_total_tokens = (uint32_t)a.geti("max-batch-total-tokens", 0);
  cfg.waiting_served_ratio = (float)a.getd("waiting-served-ratio", 0.3);
  cfg.max_waiting_tokens = (uint32_t)a.geti("max-waiting-tokens", 20);
  cfg.max_active_adapters = (size_t)a.geti("max-active-adapters", 128);
  cfg.adapter_cycle_time_s = a.getd("adapter-cycle-time-s", 2.0);
  cfg.eager_prefill = a.getb("eager-prefill", true);
  cfg.prefix_caching = a.getb("prefix-caching", false);
  cfg.chunked_prefill = a.getb("chunked-prefill", false);
  cfg.default_adapter_source = a.get("adapter-source", "hub");
  cfg.model_id = a.get("model-id", "");
  const std::string uds = a.get("master-shard-uds-path", "/tmp/lorax-server");
  const int num_shard = (int)a.geti("num-shard", 1);
  const int port = (int)a.geti("port", 3000);
  const std::string host = a.get("hostname", "0.0.0.0");
  if (cfg.max_input_length >= cfg.max_total_tokens) { log_json("ERROR", "`max_input_length` must be < `max_total_tokens`"); return 2; }

  // framed socket (default) or the original gRPC contract on unix://{uds}-{rank}; the tokenizer helpers always use the framed one
  const std::string transport = a.get("shard-transport", "framed");
  if (transport != "framed" && transport != "grpc") {
    std::cerr << "--shard-transport must be framed or grpc\n";
    return 2;
  }
  auto client = std::make_shared<ShardedClient>(transport == "grpc" ? connect_grpc(uds, num_shard) : ShardedClient::connect_uds(uds, num_shard));
  gen::InfoResponse info;
  uint32_t num_blocks = 0;
  try {
    client->clear_cache(std::nullopt);          // a restarted router starts from empty shard caches
    info = client->info();
    gen::WarmupRequest wr;
    wr.max_input_length = cfg.max_input_length;
    wr.max_prefill_tokens = cfg.max_batch_prefill_tokens;
    wr.max_new_tokens = cfg.max_total_tokens - cfg.max_input_length;
    auto supported = client->warmup(wr);
    if (supported) {
      if (cfg.max_batch_total_tokens == 0 || cfg.max_batch_total_tokens > *supported) cfg.max_batch_total_tokens = *supported;
    } else if (cfg.max_batch_total_tokens == 0) {
      cfg.max_batch_total_tokens = std::max(16000u, cfg.max_batch_prefill_tokens);
    }
    if (cfg.max_batch_total_tokens < cfg.max_total_tokens) {
      log_json("ERROR", "`max_total_tokens` must be <= `max_batch_total_tokens`");
      return 2;
    }
    num_blocks = cfg.max_batch_total_tokens / std::max(1u, info.block_size) + 1;
  } catch (const std::exception& e) {
    log_json("ERROR", std::string("could not connect to the shards: ") + e.what());
    return 1;
  }
  log_json("INFO", "connected to " + std::to_string(num_shard) + " shard(s); max_batch_total_tokens=" + std::to_string(cfg.max_batch_total_tokens));

  g_validation_workers = (int)a.geti("validation-workers", 2);
  // Tokenisation inside the router, on `validation_workers` threads, from the tokenizer file of shard 0 (or --tokenizer-name: a
  // tokenizer.json or a directory with one).  `--router-tokenizer off`, a runtime whose prompts need more than the tokenizer
  // (image placeholders) or a file with a component the router does not implement leave tokenisation with shard 0.
  if (a.get("router-tokenizer", "on") != "off") {
    try {
      std::shared_ptr<const tok::Tokenizer> t;
      bool images_to_shard = false;
      img::ImagePolicy image_policy;
      const std::string named = a.get("tokenizer-name", "");
      if (!named.empty()) {
        t = tok::Tokenizer::load(named);
      } else {
        std::string file = client->helper(103, "");
        json::Value root;
        std::string perr;
        if (file.empty()) throw tok::Unsupported("the shard has no tokenizer file");
        if (file.rfind("#images", 0) == 0) {               // "#images {policy json}\n" in front of the tokenizer file
          const size_t nl = file.find('\n');
          if (nl == std::string::npos) throw std::runtime_error("tokenizer file: bad header");
          images_to_shard = true;
          json::Value pol;
          if (nl > 8 && json::parse(file.substr(8, nl - 8), pol, &perr)) image_policy = img::ImagePolicy::from_json(pol);
          file.erase(0, nl + 1);
        }
        if (!json::parse(file, root, &perr)) throw std::runtime_error("tokenizer file: " + perr);
        t = tok::Tokenizer::from_json(root);
      }
      client->set_local_tokenizer(std::make_shared<tok::TokenizerPool>(t, g_validation_workers), images_to_shard, image_policy);
      log_json("INFO", "tokenising in the router on " + std::to_string(g_validation_workers) + " worker(s)" +
                           (!images_to_shard ? "" : image_policy.kind != img::ImagePolicy::None ? "; inline images are counted here, image URLs go to shard 0"
                                                                                                : "; prompts with images go to shard 0"));
    } catch (const std::exception& e) {
      log_json("INFO", std::string("shard 0 tokenises (router tokenizer not used: ") + e.what() + ")");
    }
  }
  const std::string otlp = a.get("otlp-endpoint", "");
  const char* logger_env = std::getenv("REQUEST_LOGGER_URL");
  App app(client, cfg, info, num_blocks, otlp, logger_env ? logger_env : "");
  if (a.get("router-chat-template", "on") != "off") {
    try {
      json::Value setup;
      std::string perr;
      if (!json::parse(client->helper(104, ""), setup, &perr)) throw std::runtime_error(perr);
      if (setup["chat_template"].is_string()) {
        auto r = std::make_shared<jinja::ChatRenderer>();
        r->tmpl = jinja::Template::compile(setup["chat_template"].as_string());
        r->bos_token = setup["bos_token"].as_string();
        r->eos_token = setup["eos_token"].as_string();
        app.set_chat_renderer(r);
        log_json("INFO", "rendering chat templates in the router");
      }
    } catch (const std::exception& e) {
      log_json("INFO", std::string("shard 0 renders chat templates (") + e.what() + ")");
    }
  }
  if (!otlp.empty()) log_json(app.tracing() ? "INFO" : "WARN", app.tracing() ? "tracing to " + otlp + (lx::telemetry::parse_url(otlp).grpc ? " (OTLP/gRPC)" : " (OTLP/HTTP JSON)")
                                                                              : "otlp endpoint must be an http:// or grpc:// URL; tracing is off");
  http::Server server;
  std::vector<std::string> cors;
  std::string cors_arg = a.get("cors-allow-origin", "");
  if (!cors_arg.empty()) cors.push_back(cors_arg);
  server.set_cors(cors);
  server.set_cors_options(a.get("cors-allow-method", ""), a.get("cors-allow-header", ""), a.get("cors-expose-header", ""),
                          a.getb("cors-allow-credentials", false));
  auto R = [&](const char* m, const char* p, http::Handler h) { server.route(m, p, std::move(h)); };
  R("POST", "/", [&](auto& q, auto& w) { app.generate(q, w); });
  R("POST", "/generate", [&](auto& q, auto& w) { app.generate(q, w); });
  R("POST", "/invocations", [&](auto& q, auto& w) { app.generate(q, w); });
  R("POST", "/generate_stream", [&](auto& q, auto& w) { app.generate_stream(q, w); });
  R("POST", "/v1/completions", [&](auto& q, auto& w) { app.completions(q, w); });
  R("POST", "/v1/chat/completions", [&](auto& q, auto& w) { app.chat_completions(q, w); });
  R("POST", "/v1/embeddings", [&](auto& q, auto& w) { app.embed(q, w, true); });
  R("POST", "/embed", [&](auto& q, auto& w) { app.embed(q, w, false); });
  R("POST", "/classify", [&](auto& q, auto& w) { app.classify(q, w, false); });
  R("POST", "/classify_batch", [&](auto& q, auto& w) { app.classify(q, w, true); });
  R("POST", "/tokenize", [&](auto& q, auto& w) { app.tokenize(q, w); });
  R("GET", "/health", [&](auto&, auto& w) { app.health(w); });
  R("GET", "/ping", [&](auto&, auto& w) { app.health(w); });
  R("GET", "/startup", [&](auto&, auto& w) { app.startup(w); });
  R("GET", "/info", [&](auto&, auto& w) { app.info(w); });
  R("GET", "/", [&](auto&, auto& w) { app.health(w); });
  // Prometheus text by default; JSON with ?format=json or "Accept: application/json" (reference router/src/server.rs:1200-1290):
  // {family: {"type": counter|gauge|histogram, "data": [{"key": labelled series name | "sum" | "count" | "", "value": v}]}}
  R("GET", "/metrics", [&](auto& req, auto& w) {
    std::string text = app.metrics().render();
    if (client->tokenizes_locally())
      text += "# TYPE lorax_router_tokenizations counter\nlorax_router_tokenizations " + std::to_string(client->local_tokenizations()) + "\n";
    text += "# TYPE lorax_router_chat_templates counter\nlorax_router_chat_templates " + std::to_string(app.chat_templates_rendered()) + "\n";
    std::string fmt = req.query_param("format");
    for (auto& ch : fmt) ch = (char)std::tolower((unsigned char)ch);
    const bool want_json = fmt.empty() ? req.header("accept").find("application/json") != std::string::npos : fmt == "json";
    if (!want_json) return (void)w.send(200, text, "text/plain; version=0.0.4");
    Value out = Value::object();
    std::string current;
    std::map<std::string, std::pair<std::string, Value>> fams;
    size_t pos = 0;
    while (pos < text.size()) {
      size_t nl = text.find('\n', pos);
      std::string line = text.substr(pos, nl == std::string::npos ? std::string::npos : nl - pos);
      pos = nl == std::string::npos ? text.size() : nl + 1;
      if (line.empty()) continue;
      if (line.rfind("# TYPE ", 0) == 0) {
        const size_t sp = line.find(' ', 7);
        if (sp != std::string::npos) {
          current = line.substr(7, sp - 7);
          fams[current] = {line.substr(sp + 1), Value::array()};
        }
        continue;
      }
      auto it = fams.find(current);
      const size_t sp = line.rfind(' ');
      if (it == fams.end() || sp == std::string::npos) continue;
      const std::string name = line.substr(0, sp);
      Value dp = Value::object();
      std::string key;
      if (name.find('{') != std::string::npos) key = name;
      else if (name.size() > 4 && name.compare(name.size() - 4, 4, "_sum") == 0) key = "sum";
      else if (name.size() > 6 && name.compare(name.size() - 6, 6, "_count") == 0) key = "count";
      dp.set("key", key);
      dp.set("value", std::strtod(line.c_str() + sp + 1, nullptr));
      it->second.second.push(dp);
    }
    for (auto& kv : fams) {
      Value fam = Value::object();
      fam.set("type", kv.second.first);
      fam.set("data", kv.second.second);
      out.set(kv.first, fam);
    }
    w.send(200, out.dump());
  });
  const std::string open_api = open_api_document();
  R("GET", "/docs", [&](auto&, auto& w) { w.send(200, open_api); });
  R("GET", "/api-doc/openapi.json", [&](auto&, auto& w) { w.send(200, open_api); });
  int bound = server.listen_and_serve(host, port);
  if (!bound) { log_json("ERROR", "cannot bind port " + std::to_string(port)); return 1; }
  log_json("INFO", "Connected; listening on " + host + ":" + std::to_string(bound));
  while (!g_stop) std::this_thread::sleep_for(std::chrono::milliseconds(100));
  log_json("INFO", "signal received, starting graceful shutdown");
  server.stop();
  app.stop();
  return 0;
}
