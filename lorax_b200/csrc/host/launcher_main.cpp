// lorax-launcher: starts one shard process per GPU and the router, and supervises them.
//
// Behaviour kept from the reference launcher (launcher/src/main.rs:664-1021, 1114-1152, 1316-1647, 1649-1875):
//   * flags are also read from the environment (MODEL_ID, NUM_SHARD, PORT, ...);
//   * the number of shards comes from --num-shard, else from CUDA_VISIBLE_DEVICES / NVIDIA_VISIBLE_DEVICES, else 1;
//   * every shard gets RANK / WORLD_SIZE / LOCAL_RANK / MASTER_ADDR / MASTER_PORT and is "ready" once its unix
//     socket exists; then the router is started;
//   * a shard that exits takes the deployment down; a router exit shuts the shards down; SIGTERM / SIGINT are
//     forwarded and children get a grace period (90 s) before SIGKILL;
//   * JSON log lines of the children are re-emitted at their own level.
#include <fcntl.h>
#include <poll.h>
#include <signal.h>
#include <spawn.h>
#include <sys/stat.h>
#include <sys/wait.h>
#include <unistd.h>

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <iostream>
#include <map>
#include <sstream>
#include <string>
#include <thread>
#include <vector>

#include "json.hpp"

extern char** environ;

namespace {

volatile sig_atomic_t g_signal = 0;
void on_signal(int s) { g_signal = s; }

struct Flag { const char* name; const char* env; const char* def; const char* help; };
// Public flag names follow the reference launcher.
const Flag kFlags[] = {
    {"model-id", "MODEL_ID", "", "model directory or hub id"},
    {"adapter-id", "ADAPTER_ID", "", "adapter applied to every request by default"},
    {"source", "SOURCE", "hub", "hub | s3 | local"},
    {"adapter-source", "ADAPTER_SOURCE", "hub", "default adapter source"},
    {"revision", "REVISION", "", "model revision"},
    {"num-shard", "NUM_SHARD", "", "number of tensor-parallel shards"},
    {"quantize", "QUANTIZE", "", "fp8 | gptq | awq | eetq | bitsandbytes ..."},
    {"dtype", "DTYPE", "", "float16 | bfloat16"},
    {"compile", "COMPILE", "true", "capture decode steps in CUDA graphs"},
    {"skip-download", "SKIP_DOWNLOAD", "false", "do not run the download-weights step before the shards start"},
    {"merge-adapter-weights", "MERGE_ADAPTER_WEIGHTS", "false", "fold --adapter-id into the base weights at load time"},
    {"speculative-tokens", "SPECULATIVE_TOKENS", "", "tokens proposed per step"},
    {"preloaded-adapter-ids", "PRELOADED_ADAPTER_IDS", "", "comma separated"},
    {"max-concurrent-requests", "MAX_CONCURRENT_REQUESTS", "1024", ""},
    {"max-best-of", "MAX_BEST_OF", "2", ""},
    {"max-stop-sequences", "MAX_STOP_SEQUENCES", "4", ""},
    {"max-input-length", "MAX_INPUT_LENGTH", "", "default: min(max positions, 4096) - 1"},
    {"max-total-tokens", "MAX_TOTAL_TOKENS", "", "default: min(max positions, 4096)"},
    {"max-batch-prefill-tokens", "MAX_BATCH_PREFILL_TOKENS", "", "default: max_input_length + 50"},
    {"max-batch-total-tokens", "MAX_BATCH_TOTAL_TOKENS", "", "default: from warmup"},
    {"waiting-served-ratio", "WAITING_SERVED_RATIO", "1.2", ""},
    {"max-waiting-tokens", "MAX_WAITING_TOKENS", "20", ""},
    {"max-active-adapters", "MAX_ACTIVE_ADAPTERS", "1024", ""},
    {"adapter-cycle-time-s", "ADAPTER_CYCLE_TIME_S", "2", ""},
    {"adapter-memory-fraction", "ADAPTER_MEMORY_FRACTION", "0.1", ""},
    {"eager-prefill", "EAGER_PREFILL", "true", ""},
    {"prefix-caching", "PREFIX_CACHING", "false", ""},
    {"chunked-prefill", "CHUNKED_PREFILL", "false", ""},
    {"hostname", "HOSTNAME", "0.0.0.0", ""},
    {"port", "PORT", "3000", ""},
    {"shard-uds-path", "SHARD_UDS_PATH", "/tmp/lorax-server", ""},
    {"master-addr", "MASTER_ADDR", "127.0.0.1", ""},
    {"master-port", "MASTER_PORT", "29500", ""},
    {"cuda-memory-fraction", "CUDA_MEMORY_FRACTION", "1.0", ""},
    {"otlp-endpoint", "OTLP_ENDPOINT", "", ""},
    {"cors-allow-origin", "CORS_ALLOW_ORIGIN", "", ""},
    {"json-output", "JSON_OUTPUT", "false", ""},
    {"sharded", "SHARDED", "", "false: one shard whatever devices are visible; true: one shard per visible device"},
    {"eager", "EAGER", "false", "no CUDA graphs (same as --compile false)"},
    {"compile-max-batch-size", "COMPILE_MAX_BATCH_SIZE", "", "largest decode batch captured in a CUDA graph"},
    {"compile-max-rank", "COMPILE_MAX_RANK", "", "largest LoRA rank captured in a CUDA graph"},
    {"compile-batch-size", "COMPILE_BATCH_SIZE", "", "step between captured batch sizes"},
    {"speculation-max-batch-size", "SPECULATION_MAX_BATCH_SIZE", "", "no speculation above this many decode rows"},
    {"memory-wiggle-room", "MEMORY_WIGGLE_ROOM", "", "fraction of the free HBM the KV cache may take after warm-up"},
    {"watermark-gamma", "WATERMARK_GAMMA", "", ""},
    {"watermark-delta", "WATERMARK_DELTA", "", ""},
    {"huggingface-hub-cache", "HUGGINGFACE_HUB_CACHE", "", "where hub downloads are kept"},
    {"weights-cache-override", "WEIGHTS_CACHE_OVERRIDE", "", "read weights from this directory instead of the hub cache"},
    {"predibase-api-token", "PREDIBASE_API_TOKEN", "", "token for adapters of source pbase"},
    {"preloaded-adapter-source", "PRELOADED_ADAPTER_SOURCE", "", "source of --preloaded-adapter-ids (default: --adapter-source)"},
    {"default-adapter-source", "DEFAULT_ADAPTER_SOURCE", "", "source the router assumes for requests that name none"},
    {"download-only", "DOWNLOAD_ONLY", "false", "fetch the weights and exit"},
    {"validation-workers", "VALIDATION_WORKERS", "2", "tokenisation workers of the router"},
    {"tokenizer-config-path", "TOKENIZER_CONFIG_PATH", "", "tokenizer_config.json to take the chat template from"},
    {"tokenizer-name", "TOKENIZER_NAME", "", "tokenizer.json (or its directory) for the router; default: the file shard 0 loaded"},
    {"router-tokenizer", "ROUTER_TOKENIZER", "", "`off` leaves tokenisation of requests to shard 0"},
    {"router-chat-template", "ROUTER_CHAT_TEMPLATE", "", "`off` leaves the rendering of chat templates to shard 0"},
    {"cors-allow-method", "CORS_ALLOW_METHOD", "", ""},
    {"cors-allow-header", "CORS_ALLOW_HEADER", "", ""},
    {"cors-expose-header", "CORS_EXPOSE_HEADER", "", ""},
    {"cors-allow-credentials", "CORS_ALLOW_CREDENTIALS", "", ""},
    // accepted so that command lines written for the reference launcher keep working; they select between code paths that do not
    // exist here (one attention backend, one LoRA kernel family, no remote code, no tunnel)
    {"backend", "BACKEND", "", "accepted, no effect: there is one attention backend"},
    {"disable-custom-kernels", "DISABLE_CUSTOM_KERNELS", "false", "accepted, no effect: the CUDA kernels are the only path"},
    {"disable-sgmv", "DISABLE_SGMV", "false", "accepted, no effect: one segmented LoRA kernel family serves prefill and decode"},
    {"trust-remote-code", "TRUST_REMOTE_CODE", "false", "accepted, no effect: no code from a model repository is ever run"},
    {"embedding-dim", "EMBEDDING_DIM", "", "accepted, no effect: encoders report their own width"},
    {"ngrok", "NGROK", "false", "refused: no tunnel client is built in"},
    {"ngrok-authtoken", "NGROK_AUTHTOKEN", "", ""},
    {"ngrok-edge", "NGROK_EDGE", "", ""},
    {"python", "LORAX_PYTHON", "python", "interpreter that runs the shards"},
    {"router-bin", "LORAX_ROUTER_BIN", "", "path of lorax-router (default: next to this binary)"},
};

struct Config {
  std::map<std::string, std::string> v;
  bool env_only = false;
  std::string get(const std::string& k) const { auto it = v.find(k); return it == v.end() ? "" : it->second; }
  bool truthy(const std::string& k) const { std::string s = get(k); return s == "1" || s == "true" || s == "True"; }
};

Config parse(int argc, char** argv) {
  Config c;
  for (auto& f : kFlags) {
    const char* e = getenv(f.env);
    c.v[f.name] = e ? e : f.def;
  }
  for (int i = 1; i < argc; ++i) {
    std::string s = argv[i];
    if (s == "--env") { c.env_only = true; continue; }
    if (s == "--help" || s == "-h") {
      std::cout << "lorax-launcher [flags]\n";
      for (auto& f : kFlags) std::cout << "  --" << f.name << " (env " << f.env << ", default '" << f.def << "') " << f.help << "\n";
      exit(0);
    }
    if (s.rfind("--", 0) != 0) continue;
    s = s.substr(2);
    size_t eq = s.find('=');
    if (eq != std::string::npos) c.v[s.substr(0, eq)] = s.substr(eq + 1);
    else if (i + 1 < argc && std::string(argv[i + 1]).rfind("--", 0) != 0) c.v[s] = argv[++i];
    else c.v[s] = "true";
  }
  return c;
}

bool g_json = false;
void emit(const std::string& level, const std::string& target, const std::string& msg) {
  if (g_json) {
    json::Value v = json::Value::object();
    v.set("level", level);
    v.set("target", target);
    v.set("message", msg);
    std::cout << v.dump() << std::endl;
  } else {
    std::cout << level << " " << target << ": " << msg << std::endl;
  }
}

// Flags that reach the shards (and the download step) as environment variables, under the names the shard reads.
std::vector<std::string> shard_env(const Config& c) {
  static const std::pair<const char*, const char*> kMap[] = {
      {"compile-max-batch-size", "LORAX_COMPILE_MAX_BATCH_SIZE"}, {"compile-max-rank", "LORAX_COMPILE_MAX_RANK"},
      {"compile-batch-size", "LORAX_COMPILE_BATCH_SIZE"}, {"speculation-max-batch-size", "LORAX_SPECULATION_MAX_BATCH_SIZE"},
      {"memory-wiggle-room", "MEMORY_WIGGLE_ROOM"}, {"watermark-gamma", "WATERMARK_GAMMA"}, {"watermark-delta", "WATERMARK_DELTA"},
      {"huggingface-hub-cache", "HUGGINGFACE_HUB_CACHE"}, {"weights-cache-override", "WEIGHTS_CACHE_OVERRIDE"},
      {"predibase-api-token", "PREDIBASE_API_TOKEN"}, {"tokenizer-config-path", "TOKENIZER_CONFIG_PATH"}};
  std::vector<std::string> env;
  for (auto& m : kMap)
    if (!c.get(m.first).empty()) env.push_back(std::string(m.second) + "=" + c.get(m.first));
  return env;
}

// Shard count: explicit flag, else the visible-devices list, else 1.
int find_num_shards(const Config& c) {
  if (c.get("sharded") == "false") return 1;
  if (!c.get("num-shard").empty()) return std::max(1, atoi(c.get("num-shard").c_str()));
  for (const char* name : {"CUDA_VISIBLE_DEVICES", "NVIDIA_VISIBLE_DEVICES"}) {
    const char* e = getenv(name);
    if (e && *e && std::string(e) != "all" && std::string(e) != "void") {
      int n = 1;
      for (const char* p = e; *p; ++p) if (*p == ',') ++n;
      return n;
    }
  }
  return 1;
}

// max_position_embeddings from config.json of a local model directory (0 if unknown).
long max_positions(const std::string& model_id) {
  std::string path = model_id + "/config.json";
  FILE* f = fopen(path.c_str(), "rb");
  if (!f) return 0;
  std::string s;
  char buf[4096];
  size_t n;
  while ((n = fread(buf, 1, sizeof buf, f)) > 0) s.append(buf, n);
  fclose(f);
  json::Value v;
  if (!json::parse(s, v)) return 0;
  for (const char* k : {"max_position_embeddings", "n_positions", "max_seq_len"})
    if (v[k].is_number()) return v[k].as_int();
  return 0;
}

struct Child {
  pid_t pid = -1;
  int out_fd = -1;
  std::string name;
  std::string buf;
};

Child spawn(const std::string& name, const std::vector<std::string>& argv, const std::vector<std::string>& extra_env) {
  int pipefd[2];
  if (pipe(pipefd) != 0) { perror("pipe"); exit(1); }
  posix_spawn_file_actions_t fa;
  posix_spawn_file_actions_init(&fa);
  posix_spawn_file_actions_adddup2(&fa, pipefd[1], 1);
  posix_spawn_file_actions_adddup2(&fa, pipefd[1], 2);
  posix_spawn_file_actions_addclose(&fa, pipefd[0]);
  std::vector<std::string> env_s;
  for (char** e = environ; *e; ++e) {
    std::string kv = *e;
    bool overridden = false;
    for (auto& x : extra_env) if (kv.compare(0, kv.find('=') + 1, x, 0, x.find('=') + 1) == 0) overridden = true;
    if (!overridden) env_s.push_back(kv);
  }
  for (auto& x : extra_env) env_s.push_back(x);
  std::vector<char*> envp, args;
  for (auto& s : env_s) envp.push_back(const_cast<char*>(s.c_str()));
  envp.push_back(nullptr);
  for (auto& s : argv) args.push_back(const_cast<char*>(s.c_str()));
  args.push_back(nullptr);
  Child c;
  c.name = name;
  // own process group per child, so signals can be delivered to the child and everything it starts
  posix_spawnattr_t attr;
  posix_spawnattr_init(&attr);
  posix_spawnattr_setflags(&attr, POSIX_SPAWN_SETPGROUP);
  posix_spawnattr_setpgroup(&attr, 0);
  int rc = posix_spawnp(&c.pid, args[0], &fa, &attr, args.data(), envp.data());
  posix_spawn_file_actions_destroy(&fa);
  posix_spawnattr_destroy(&attr);
  close(pipefd[1]);
  if (rc != 0) {
    emit("ERROR", "lorax_launcher", "cannot start " + name + ": " + strerror(rc));
    close(pipefd[0]);
    c.pid = -1;
    return c;
  }
  c.out_fd = pipefd[0];
  fcntl(c.out_fd, F_SETFL, fcntl(c.out_fd, F_GETFL) | O_NONBLOCK);
  return c;
}

// Forward the child's output; JSON lines keep their level.
void pump(Child& c) {
  if (c.out_fd < 0) return;
  char tmp[4096];
  while (true) {
    ssize_t r = read(c.out_fd, tmp, sizeof tmp);
    if (r > 0) { c.buf.append(tmp, (size_t)r); continue; }
    if (r == 0) { close(c.out_fd); c.out_fd = -1; }
    break;
  }
  size_t nl;
  while ((nl = c.buf.find('\n')) != std::string::npos) {
    std::string line = c.buf.substr(0, nl);
    c.buf.erase(0, nl + 1);
    if (line.empty()) continue;
    json::Value v;
    if (line[0] == '{' && json::parse(line, v) && v.is_object()) {
      std::string level = v["level"].as_string().empty() ? "INFO" : v["level"].as_string();
      std::string msg = v["message"].is_string() ? v["message"].as_string() : (v["text"].is_string() ? v["text"].as_string() : line);
      emit(level, c.name, msg);
    } else {
      emit("INFO", c.name, line);
    }
  }
}

bool exited(Child& c, int* status) {
  if (c.pid <= 0) return true;
  int st = 0;
  pid_t r = waitpid(c.pid, &st, WNOHANG);
  if (r == c.pid) { *status = st; c.pid = -1; return true; }
  return false;
}

void terminate_all(std::vector<Child*> kids, int grace_s) {
  for (auto* k : kids) if (k->pid > 0) kill(-k->pid, SIGTERM);
  auto deadline = std::chrono::steady_clock::now() + std::chrono::seconds(grace_s);
  while (std::chrono::steady_clock::now() < deadline) {
    bool any = false;
    for (auto* k : kids) {
      pump(*k);
      int st;
      if (!exited(*k, &st)) any = true;
    }
    if (!any) return;
    std::this_thread::sleep_for(std::chrono::milliseconds(100));
  }
  for (auto* k : kids) if (k->pid > 0) { kill(-k->pid, SIGKILL); int st; waitpid(k->pid, &st, 0); k->pid = -1; }
}

std::string self_dir(const char* argv0) {
  char buf[4096];
  ssize_t n = readlink("/proc/self/exe", buf, sizeof buf - 1);
  std::string p = n > 0 ? std::string(buf, (size_t)n) : std::string(argv0);
  size_t slash = p.rfind('/');
  return slash == std::string::npos ? "." : p.substr(0, slash);
}

}  // namespace

int main(int argc, char** argv) {
  Config c = parse(argc, argv);
  g_json = c.truthy("json-output");
  if (c.env_only) {
    emit("INFO", "lorax_launcher", "version 0.1.0; printing the runtime environment");
    int rc = system("nvidia-smi --query-gpu=name,driver_version,memory.total --format=csv 2>&1");
    (void)rc;
    return 0;
  }
  if (c.get("model-id").empty()) { emit("ERROR", "lorax_launcher", "--model-id (or MODEL_ID) is required"); return 2; }
  signal(SIGINT, on_signal);
  signal(SIGTERM, on_signal);
  signal(SIGPIPE, SIG_IGN);

  // ---- derived token limits
  long pos = max_positions(c.get("model-id"));
  long cap = pos > 0 ? std::min<long>(pos, 4096) : 4096;
  if (c.get("max-total-tokens").empty()) c.v["max-total-tokens"] = std::to_string(cap);
  if (c.get("max-input-length").empty()) c.v["max-input-length"] = std::to_string(std::min<long>(cap, atol(c.get("max-total-tokens").c_str())) - 1);
  if (c.get("max-batch-prefill-tokens").empty()) c.v["max-batch-prefill-tokens"] = std::to_string(atol(c.get("max-input-length").c_str()) + 50);
  if (atol(c.get("max-input-length").c_str()) >= atol(c.get("max-total-tokens").c_str())) {
    emit("ERROR", "lorax_launcher", "`max_input_length` must be < `max_total_tokens`");
    return 2;
  }
  if (c.truthy("ngrok")) { emit("ERROR", "lorax_launcher", "--ngrok: no tunnel client is built into this launcher"); return 2; }
  if (atol(c.get("validation-workers").c_str()) <= 0) { emit("ERROR", "lorax_launcher", "`validation_workers` must be > 0"); return 2; }
  for (const char* opt : {"backend", "embedding-dim"})
    if (!c.get(opt).empty()) emit("WARN", "lorax_launcher", std::string("--") + opt + " is accepted for compatibility and has no effect");
  for (const char* opt : {"disable-custom-kernels", "disable-sgmv", "trust-remote-code"})
    if (c.truthy(opt)) emit("WARN", "lorax_launcher", std::string("--") + opt + " is accepted for compatibility and has no effect");
  const int num_shard = find_num_shards(c);
  if (c.get("sharded") == "true" && num_shard <= 1) {
    emit("ERROR", "lorax_launcher", "`sharded` is true but only one device is visible (or `num_shard` is 1)");
    return 2;
  }
  emit("INFO", "lorax_launcher", "starting " + std::to_string(num_shard) + " shard(s) for " + c.get("model-id"));

  // ---- weights: one download / conversion step before any shard starts (the reference runs `lorax-server download-weights`
  // the same way, launcher/src/main.rs:1166-1313); a local model directory needs none
  struct stat model_sb;
  const bool local_dir = stat(c.get("model-id").c_str(), &model_sb) == 0 && S_ISDIR(model_sb.st_mode);
  if (!local_dir && !c.truthy("skip-download")) {
    std::vector<std::string> dargs = {c.get("python"), "-m", "lorax_b200.server.cli", "download-weights", c.get("model-id"),
                                      "--source", c.get("source"), "--json-output"};
    if (!c.get("revision").empty()) { dargs.push_back("--revision"); dargs.push_back(c.get("revision")); }
    if (!c.get("adapter-id").empty()) {
      dargs.insert(dargs.end(), {"--adapter-id", c.get("adapter-id"), "--adapter-source", c.get("adapter-source")});
    }
    emit("INFO", "lorax_launcher", "Starting download process.");
    Child dl = spawn("download", dargs, shard_env(c));
    if (dl.pid <= 0) return 1;
    int st = 0;
    while (!exited(dl, &st)) {
      pump(dl);
      if (g_signal) { terminate_all({&dl}, 10); return 0; }
      std::this_thread::sleep_for(std::chrono::milliseconds(100));
    }
    pump(dl);
    if (!WIFEXITED(st) || WEXITSTATUS(st) != 0) {
      emit("ERROR", "lorax_launcher", "download of " + c.get("model-id") + " failed (status " + std::to_string(st) + ")");
      return 1;
    }
    emit("INFO", "lorax_launcher", "Successfully downloaded weights.");
  }
  if (c.truthy("download-only")) {
    emit("INFO", "lorax_launcher", "weights are in place; --download-only: not starting shards");
    return 0;
  }

  // ---- shards
  const std::string uds = c.get("shard-uds-path");
  std::vector<Child> shards((size_t)num_shard);
  for (int r = 0; r < num_shard; ++r) {
    std::string sock = uds + "-" + std::to_string(r) + ".lx";
    unlink(sock.c_str());
    std::vector<std::string> args = {c.get("python"), "-m", "lorax_b200.server.cli", "serve", c.get("model-id"),
                                     "--uds-path", uds, "--source", c.get("source"), "--adapter-source", c.get("adapter-source"),
                                     "--max-input-length", c.get("max-input-length"), "--max-total-tokens", c.get("max-total-tokens"),
                                     "--max-batch-prefill-tokens", c.get("max-batch-prefill-tokens"),
                                     "--adapter-memory-fraction", c.get("adapter-memory-fraction"), "--json-output"};
    if (num_shard > 1) args.push_back("--sharded");
    for (const char* opt : {"revision", "quantize", "dtype", "adapter-id", "speculative-tokens", "preloaded-adapter-ids", "otlp-endpoint",
                            "preloaded-adapter-source"})
      if (!c.get(opt).empty()) { args.push_back(std::string("--") + opt); args.push_back(c.get(opt)); }
    if (!c.truthy("compile") || c.truthy("eager")) args.push_back("--no-compile");
    if (c.truthy("prefix-caching")) args.push_back("--prefix-caching");
    if (c.truthy("merge-adapter-weights")) args.push_back("--merge-adapter-weights");
    if (c.truthy("chunked-prefill")) args.push_back("--chunked-prefill");
    std::vector<std::string> env = {"RANK=" + std::to_string(r), "LOCAL_RANK=" + std::to_string(r), "WORLD_SIZE=" + std::to_string(num_shard),
                                    "MASTER_ADDR=" + c.get("master-addr"), "MASTER_PORT=" + c.get("master-port"),
                                    "NCCL_ASYNC_ERROR_HANDLING=1", "CUDA_MEMORY_FRACTION=" + c.get("cuda-memory-fraction"),
                                    "ADAPTER_MEMORY_FRACTION=" + c.get("adapter-memory-fraction")};
    for (auto& kv : shard_env(c)) env.push_back(kv);
    shards[(size_t)r] = spawn("shard-" + std::to_string(r), args, env);
    if (shards[(size_t)r].pid <= 0) return 1;
  }
  std::vector<Child*> all;
  for (auto& s : shards) all.push_back(&s);

  // ---- wait until every shard listens
  std::vector<bool> ready((size_t)num_shard, false);
  while (true) {
    if (g_signal) { terminate_all(all, 90); return 0; }
    bool all_ready = true;
    for (int r = 0; r < num_shard; ++r) {
      pump(shards[(size_t)r]);
      int st;
      if (exited(shards[(size_t)r], &st)) {
        pump(shards[(size_t)r]);
        emit("ERROR", "lorax_launcher", "shard " + std::to_string(r) + " failed to start (status " + std::to_string(st) + ")");
        terminate_all(all, 10);
        return 1;
      }
      struct stat sb;
      std::string sock = uds + "-" + std::to_string(r) + ".lx";
      if (!ready[(size_t)r] && stat(sock.c_str(), &sb) == 0) {
        ready[(size_t)r] = true;
        emit("INFO", "lorax_launcher", "shard " + std::to_string(r) + " ready");
      }
      all_ready = all_ready && ready[(size_t)r];
    }
    if (all_ready) break;
    std::this_thread::sleep_for(std::chrono::milliseconds(100));
  }

  // ---- router
  std::string router_bin = c.get("router-bin").empty() ? self_dir(argv[0]) + "/lorax-router" : c.get("router-bin");
  std::vector<std::string> rargs = {router_bin, "--master-shard-uds-path", uds, "--num-shard", std::to_string(num_shard),
                                    "--model-id", c.get("model-id")};
  for (const char* opt : {"max-concurrent-requests", "max-best-of", "max-stop-sequences", "max-input-length", "max-total-tokens",
                          "max-batch-prefill-tokens", "max-batch-total-tokens", "waiting-served-ratio", "max-waiting-tokens",
                          "max-active-adapters", "adapter-cycle-time-s", "eager-prefill", "prefix-caching", "chunked-prefill", "hostname",
                          "port", "adapter-source", "cors-allow-origin", "otlp-endpoint", "validation-workers", "tokenizer-name", "router-tokenizer", "router-chat-template", "cors-allow-method",
                          "cors-allow-header", "cors-expose-header", "cors-allow-credentials"})
    if (!c.get(opt).empty()) { rargs.push_back(std::string("--") + opt); rargs.push_back(c.get(opt)); }
  if (!c.get("default-adapter-source").empty()) {          // overrides --adapter-source for the router, as in the reference
    rargs.push_back("--adapter-source");
    rargs.push_back(c.get("default-adapter-source"));
  }
  Child router = spawn("router", rargs, {});
  if (router.pid <= 0) { terminate_all(all, 10); return 1; }
  all.push_back(&router);

  // ---- supervise
  int exit_code = 0;
  while (true) {
    for (auto* k : all) pump(*k);
    if (g_signal) { emit("INFO", "lorax_launcher", "signal received, shutting down"); break; }
    int st;
    bool stop = false;
    for (int r = 0; r < num_shard; ++r) {
      if (exited(shards[(size_t)r], &st)) {
        emit("ERROR", "lorax_launcher", "shard " + std::to_string(r) + " exited (status " + std::to_string(st) + "); stopping the deployment");
        exit_code = 1;
        stop = true;
      }
    }
    if (!stop && exited(router, &st)) {
      emit(st == 0 ? "INFO" : "ERROR", "lorax_launcher", "router exited (status " + std::to_string(st) + ")");
      exit_code = st == 0 ? 0 : 1;
      stop = true;
    }
    if (stop) break;
    std::this_thread::sleep_for(std::chrono::milliseconds(100));
  }
  // router first (stops accepting, drains), then the shards
  terminate_all({&router}, 30);
  terminate_all(all, 90);
  for (auto* k : all) pump(*k);
  return exit_code;
}
