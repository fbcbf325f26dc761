// Host-side self test meant to be built with -fsanitize=address,undefined and with -fsanitize=thread: it drives the
// allocator, the JSON codec, the adapter queues and the whole batching loop (many concurrent requests over several adapters
// against the in-process fake shard, with and without injected shard failures) through the same C API the Python tests use.
// The reference has no sanitizer target (only `cargo fmt --check` and ruff in CI); this is the race / memory check of the C++
// router code.  Exit status 0 and the word OK on stdout mean every scenario finished with the expected outcome; sanitizer
// findings make the process exit non-zero on their own.
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <string>
#include <thread>
#include <unistd.h>

#include "flag_protocols.hpp"
#include <vector>

extern "C" {
void* lx_alloc_new(uint32_t num_blocks, uint32_t block_size, int window, int prefix_caching);
void lx_alloc_delete(void* a);
uint64_t lx_alloc_free_blocks(void* a);
void* lx_alloc_allocate(void* a, uint32_t adapter, uint32_t tokens, const uint32_t* prompt, uint32_t prompt_len);
uint32_t lx_allocation_num_blocks(void* h);
uint32_t lx_allocation_prefix_len(void* h);
void lx_alloc_free(void* a, void* h, uint32_t adapter, const uint32_t* all_tokens, uint32_t n);
const char* lx_json_roundtrip(const char* s);
const char* lx_infer_fake_run(const char* requests_json, int max_active_adapters, int fail_decode_after, uint32_t num_blocks,
                              int prefix_caching);
void* lx_tokenizer_load(const char* path, int workers, char* err, int err_cap);
void lx_tokenizer_free(void* h);
long lx_tokenizer_encode(void* h, const char* text, size_t len, int add_special, uint32_t* out, size_t cap);
const char* lx_encoder_batcher_fake_run(int threads, int each);
const char* lx_chat_render(const char* request_json);
}

// A byte-level BPE tokenizer file over printable ASCII: normaliser, regex split, merges, a special token and a template, so
// that the router's tokenizer pipeline and its worker pool run under the sanitizers.
static std::string tiny_tokenizer_json() {
  std::string vocab = "\"<s>\":0";
  int id = 1;
  for (int c = '!'; c <= '~'; ++c) {
    std::string key(1, (char)c);
    if (c == '"' || c == '\\') key = std::string("\\") + (char)c;
    vocab += ",\"" + key + "\":" + std::to_string(id++);
  }
  vocab += ",\"\u0120\":" + std::to_string(id++);
  for (const char* m : {"th", "the", "\u0120t", "er", "in"}) vocab += std::string(",\"") + m + "\":" + std::to_string(id++);
  return std::string("{\"added_tokens\":[{\"id\":0,\"content\":\"<s>\",\"single_word\":false,\"lstrip\":false,\"rstrip\":false,"
                     "\"normalized\":false,\"special\":true}],"
                     "\"normalizer\":{\"type\":\"Sequence\",\"normalizers\":[{\"type\":\"NFKC\"},{\"type\":\"Lowercase\"}]},"
                     "\"pre_tokenizer\":{\"type\":\"Sequence\",\"pretokenizers\":[{\"type\":\"Split\",\"pattern\":{\"Regex\":"
                     "\"'s|'t| ?\\\\p{L}+| ?\\\\p{N}+| ?[^\\\\s\\\\p{L}\\\\p{N}]+|\\\\s+(?!\\\\S)|\\\\s+\"},\"behavior\":\"Isolated\",\"invert\":false},"
                     "{\"type\":\"ByteLevel\",\"add_prefix_space\":false,\"use_regex\":false}]},"
                     "\"post_processor\":{\"type\":\"TemplateProcessing\",\"single\":[{\"SpecialToken\":{\"id\":\"<s>\",\"type_id\":0}},"
                     "{\"Sequence\":{\"id\":\"A\",\"type_id\":0}}],\"special_tokens\":{\"<s>\":{\"id\":\"<s>\",\"ids\":[0],\"tokens\":[\"<s>\"]}}},"
                     "\"model\":{\"type\":\"BPE\",\"unk_token\":null,\"vocab\":{") +
         vocab + "},\"merges\":[\"t h\",\"th e\",\"\u0120 t\",\"e r\",\"i n\"]}}";
}

static int fail(const char* what, const std::string& detail = "") {
  std::printf("FAILED: %s %s\n", what, detail.c_str());
  return 1;
}

static size_t count(const std::string& hay, const std::string& needle) {
  size_t n = 0, pos = 0;
  while ((pos = hay.find(needle, pos)) != std::string::npos) { ++n; pos += needle.size(); }
  return n;
}

int main() {
  // allocator with the radix prefix cache: a second request with the same prompt reuses the first one's blocks
  for (int prefix = 0; prefix < 2; ++prefix) {
    void* a = lx_alloc_new(64, 16, 0, prefix);
    const uint64_t free0 = lx_alloc_free_blocks(a);
    std::vector<uint32_t> prompt(40);
    for (size_t i = 0; i < prompt.size(); ++i) prompt[i] = (uint32_t)(i * 7 + 3);
    void* h1 = lx_alloc_allocate(a, 1, 60, prompt.data(), (uint32_t)prompt.size());
    if (!h1 || lx_allocation_num_blocks(h1) != 4) return fail("allocate");
    std::vector<uint32_t> all = prompt;
    for (uint32_t t = 0; t < 20; ++t) all.push_back(1000 + t);
    lx_alloc_free(a, h1, 1, all.data(), (uint32_t)all.size());
    void* h2 = lx_alloc_allocate(a, 1, 60, prompt.data(), (uint32_t)prompt.size());
    if (!h2) return fail("allocate again");
    if (prefix && lx_allocation_prefix_len(h2) == 0) return fail("prefix reuse");
    void* h3 = lx_alloc_allocate(a, 2, 60, prompt.data(), (uint32_t)prompt.size());      // another adapter: no sharing
    if (!h3 || lx_allocation_prefix_len(h3) != 0) return fail("adapter isolation");
    lx_alloc_free(a, h2, 1, all.data(), (uint32_t)all.size());
    lx_alloc_free(a, h3, 2, all.data(), (uint32_t)all.size());
    if (!prefix && lx_alloc_free_blocks(a) != free0) return fail("blocks leaked");
    lx_alloc_delete(a);
  }
  // JSON
  const char* doc = "{\"a\":[1,2.5,\"x\\n\",null,true],\"b\":{\"c\":-3}}";
  if (std::string(lx_json_roundtrip(doc)) != doc) return fail("json", lx_json_roundtrip(doc));
  // batching loop: 36 concurrent requests over 6 adapters with 2 adapter slots, prefix caching on
  std::string reqs = "[";
  for (int i = 0; i < 36; ++i) {
    if (i) reqs += ",";
    reqs += "{\"inputs\":\"w" + std::to_string(i % 5) + " w7 w9 w" + std::to_string(i) + "\",\"max_new_tokens\":" + std::to_string(3 + i % 6);
    if (i % 7) reqs += ",\"adapter_id\":\"adapter-" + std::to_string(i % 6) + "\"";
    reqs += "}";
  }
  reqs += "]";
  std::string out = lx_infer_fake_run(reqs.c_str(), 2, -1, 512, 1);
  if (count(out, "\"ok\":true") != 36) return fail("concurrent run", out.substr(0, 400));
  // the same with a shard that starts failing: every request ends (with an error or a result), nothing hangs or leaks
  out = lx_infer_fake_run(reqs.c_str(), 3, 4, 512, 0);
  if (count(out, "\"ok\":true") + count(out, "\"ok\":false") != 36) return fail("failing shard", out.substr(0, 400));
  if (count(out, "\"ok\":false") == 0) return fail("failure was not injected");
  // CPU-thread models of the device-side flag protocols (races would be reported by ThreadSanitizer, wrong sums here)
  if (!lx_model::model_all_reduce(4, 3, 257, 6)) return fail("two-shot all-reduce protocol model");
  if (!lx_model::model_all_reduce(2, 5, 64, 10)) return fail("two-shot all-reduce protocol model (2 ranks)");
  if (!lx_model::model_lora_sync(6, 17, 2, 5)) return fail("LoRA-in-GEMM protocol model");
  if (!lx_model::model_lora_sync(4, 9, 1, 5)) return fail("LoRA-in-GEMM protocol model (no K split)");
  {
    // tokenizer: four request threads share a pool of two workers; every thread must see the ids a lone call produced
    char path[] = "/tmp/lx_selftest_tok_XXXXXX";
    const int fd = mkstemp(path);
    if (fd < 0) return fail("mkstemp");
    const std::string js = tiny_tokenizer_json();
    if (write(fd, js.data(), js.size()) != (ssize_t)js.size()) return fail("write tokenizer file");
    close(fd);
    char err[256] = {0};
    void* h = lx_tokenizer_load(path, 2, err, sizeof err);
    unlink(path);
    if (!h) return fail("tokenizer load", err);
    const std::string text = "The other thing<s>in THE winter, isn't it?  42 times\n\n  there";
    std::vector<uint32_t> want(256);
    const long n = lx_tokenizer_encode(h, text.data(), text.size(), 1, want.data(), want.size());
    if (n < 8 || want[0] != 0) return fail("tokenizer encode");
    want.resize((size_t)n);
    int bad = 0;
    std::vector<std::thread> threads;
    std::vector<int> bads(4, 0);
    for (int t = 0; t < 4; ++t)
      threads.emplace_back([&, t] {
        for (int k = 0; k < 100; ++k) {
          std::vector<uint32_t> got(256);
          const long m = lx_tokenizer_encode(h, text.data(), text.size(), 1, got.data(), got.size());
          got.resize(m < 0 ? 0 : (size_t)m);
          if (got != want) ++bads[(size_t)t];
        }
      });
    for (auto& th : threads) th.join();
    for (int b : bads) bad += b;
    lx_tokenizer_free(h);
    if (bad) return fail("tokenizer pool", std::to_string(bad));
  }
  if (const char* files = std::getenv("LX_SELFTEST_TOKENIZERS")) {
    // tokenizer files and a text file from the caller (the Python tests write real pipelines: byte-level BPE, SentencePiece-style
    // BPE, Unigram behind a compiled character map, WordPiece): every line through every tokenizer, for the sanitizers' eyes
    const char* text_path = std::getenv("LX_SELFTEST_TEXT");
    std::vector<std::string> lines;
    if (text_path) {
      if (FILE* f = std::fopen(text_path, "rb")) {
        std::string cur;
        for (int ch; (ch = std::fgetc(f)) != EOF;) { if (ch == '\x1e') { lines.push_back(cur); cur.clear(); } else cur.push_back((char)ch); }
        lines.push_back(cur);
        std::fclose(f);
      }
    }
    std::string list = files;
    size_t at = 0, total = 0;
    while (at <= list.size()) {
      const size_t colon = list.find(':', at);
      const std::string path = list.substr(at, colon == std::string::npos ? std::string::npos : colon - at);
      at = colon == std::string::npos ? list.size() + 1 : colon + 1;
      if (path.empty()) continue;
      char err[256] = {0};
      void* h = lx_tokenizer_load(path.c_str(), 2, err, sizeof err);
      if (!h) return fail("tokenizer load", path + ": " + err);
      std::vector<uint32_t> ids(1 << 16);
      for (auto& line : lines) {
        const long n = lx_tokenizer_encode(h, line.data(), line.size(), 1, ids.data(), ids.size());
        if (n > 0) total += (size_t)n;
      }
      lx_tokenizer_free(h);
    }
    std::printf("tokenizer files: %zu ids\n", total);
  }
  if (const char* chat_path = std::getenv("LX_SELFTEST_CHAT")) {
    // chat requests from the caller (the templates of the chat template tests with their conversations), one JSON document per record
    size_t rendered = 0, records = 0;
    if (FILE* f = std::fopen(chat_path, "rb")) {
      std::string cur;
      auto run = [&]() {
        if (cur.empty()) return;
        ++records;
        if (std::string(lx_chat_render(cur.c_str())).find("\"text\"") != std::string::npos) ++rendered;
        cur.clear();
      };
      for (int ch; (ch = std::fgetc(f)) != EOF;) { if (ch == '\x1e') run(); else cur.push_back((char)ch); }
      run();
      std::fclose(f);
    }
    std::printf("chat requests: %zu of %zu rendered\n", rendered, records);
  }
  {
    // embed / classify batcher: eight caller threads, shared batches, a failing batch now and then
    const std::string out = lx_encoder_batcher_fake_run(8, 30);
    if (out.find("\"wrong\":0") == std::string::npos) return fail("encoder batcher answers", out.substr(0, 200));
    if (out.find("\"ok\":0,") != std::string::npos) return fail("encoder batcher: nothing succeeded");
  }
  {
    // chat template interpreter: loops, namespace, filters, slices, white-space control; four threads render the same request
    const std::string req =
        "{\"template\":\"{%- set ns = namespace(n=0) -%}{% for m in messages if m.role != 'system' %}{% set ns.n = ns.n + 1 %}"
        "<{{ m.role | upper }}>{{ m.content | trim }}{{ m.content[:2] ~ loop.index }}{% endfor %}|{{ ns.n }}|{{ tools | tojson }}"
        "{% if add_generation_prompt %}<A>{% endif %}\",\"bos_token\":\"<s>\",\"eos_token\":\"</s>\",\"messages\":["
        "{\"role\":\"system\",\"content\":\"sys\"},{\"role\":\"user\",\"content\":\"  hello  \"},{\"role\":\"assistant\",\"content\":\"hi\"}]}";
    const std::string want = lx_chat_render(req.c_str());
    if (want.find("\"text\":\"<USER>hello  1<ASSISTANT>hihi2|2|null<A>\"") == std::string::npos) return fail("chat template", want);
    std::vector<std::thread> threads;
    std::vector<int> bads(4, 0);
    for (int t = 0; t < 4; ++t)
      threads.emplace_back([&, t] { for (int k = 0; k < 50; ++k) if (std::string(lx_chat_render(req.c_str())) != want) ++bads[(size_t)t]; });
    for (auto& th : threads) th.join();
    for (int b : bads) if (b) return fail("chat template under threads");
  }
  std::printf("OK\n");
  return 0;
}
