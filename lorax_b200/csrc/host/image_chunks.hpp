// Image chunks of vision-language prompts in the router: `![](uri)` markdown is cut out of the prompt, the image's size is read from
// its header, and the number of feature tokens it becomes is computed from the model's vision configuration, so that prompts with
// inline images are tokenised and validated without a call to a shard.  The reference router does this in
// router/src/validation.rs:498-638 (fetch_image, image_tokens, prepare_input) with the feature counts of router/src/config.rs:6-140.
// Handled here: `data:` URIs (PNG, JPEG, GIF, WebP, BMP) for LLaVA-NeXT style models (any-resolution grid) and for models that spend
// one token per image (Mllama).  Everything else (http(s) URLs, which need TLS, an image format not listed, another model kind)
// reports "not handled" and the router asks shard 0, which fetches and decodes the image anyway.
#pragma once
#include <cmath>
#include <cstdint>
#include <string>
#include <utility>
#include <vector>

#include "json.hpp"

namespace lx {
namespace img {

inline std::string base64_decode(const std::string& in) {
  std::string out;
  uint32_t acc = 0;
  int bits = 0;
  for (unsigned char c : in) {
    int v;
    if (c >= 'A' && c <= 'Z') v = c - 'A';
    else if (c >= 'a' && c <= 'z') v = c - 'a' + 26;
    else if (c >= '0' && c <= '9') v = c - '0' + 52;
    else if (c == '+' || c == '-') v = 62;
    else if (c == '/' || c == '_') v = 63;
    else continue;
    acc = (acc << 6) | (uint32_t)v;
    bits += 6;
    if (bits >= 8) { bits -= 8; out.push_back((char)((acc >> bits) & 0xFF)); }
  }
  return out;
}

// Width and height from the header of an encoded image.  False for formats not listed or a truncated header.
inline bool probe_image_size(const std::string& d, long* w, long* h) {
  auto u8 = [&](size_t i) { return (unsigned long)(unsigned char)d[i]; };
  auto be16 = [&](size_t i) { return (u8(i) << 8) | u8(i + 1); };
  auto be32 = [&](size_t i) { return (u8(i) << 24) | (u8(i + 1) << 16) | (u8(i + 2) << 8) | u8(i + 3); };
  auto le16 = [&](size_t i) { return u8(i) | (u8(i + 1) << 8); };
  auto le24 = [&](size_t i) { return u8(i) | (u8(i + 1) << 8) | (u8(i + 2) << 16); };
  auto le32 = [&](size_t i) { return u8(i) | (u8(i + 1) << 8) | (u8(i + 2) << 16) | (u8(i + 3) << 24); };
  const size_t n = d.size();
  if (n >= 24 && d.compare(0, 8, "\x89PNG\r\n\x1a\n") == 0 && d.compare(12, 4, "IHDR") == 0) { *w = (long)be32(16); *h = (long)be32(20); return *w > 0 && *h > 0; }
  if (n >= 10 && (d.compare(0, 6, "GIF87a") == 0 || d.compare(0, 6, "GIF89a") == 0)) { *w = (long)le16(6); *h = (long)le16(8); return *w > 0 && *h > 0; }
  if (n >= 26 && d[0] == 'B' && d[1] == 'M') {
    const long bw = (long)(int32_t)le32(18), bh = (long)(int32_t)le32(22);
    *w = bw; *h = bh < 0 ? -bh : bh;
    return *w > 0 && *h > 0;
  }
  if (n >= 30 && d.compare(0, 4, "RIFF") == 0 && d.compare(8, 4, "WEBP") == 0) {
    if (d.compare(12, 4, "VP8 ") == 0 && u8(23) == 0x9D && u8(24) == 0x01 && u8(25) == 0x2A) { *w = (long)(le16(26) & 0x3FFF); *h = (long)(le16(28) & 0x3FFF); return *w > 0 && *h > 0; }
    if (d.compare(12, 4, "VP8L") == 0 && u8(20) == 0x2F) {
      const unsigned long b = le32(21);
      *w = (long)(b & 0x3FFF) + 1; *h = (long)((b >> 14) & 0x3FFF) + 1;
      return true;
    }
    if (d.compare(12, 4, "VP8X") == 0) { *w = (long)le24(24) + 1; *h = (long)le24(27) + 1; return true; }
    return false;
  }
  if (n >= 4 && u8(0) == 0xFF && u8(1) == 0xD8) {            // JPEG: walk the segments up to the frame header
    size_t i = 2;
    while (i + 9 < n) {
      if (u8(i) != 0xFF) { ++i; continue; }
      const unsigned long m = u8(i + 1);
      if (m == 0xFF) { ++i; continue; }
      if (m == 0xD8 || m == 0x01 || (m >= 0xD0 && m <= 0xD7)) { i += 2; continue; }
      if (m >= 0xC0 && m <= 0xCF && m != 0xC4 && m != 0xC8 && m != 0xCC) { *h = (long)be16(i + 5); *w = (long)be16(i + 7); return *w > 0 && *h > 0; }
      if (m == 0xD9 || m == 0xDA) return false;
      i += 2 + be16(i + 2);
    }
    return false;
  }
  return false;
}

// "a ![](uri) b" -> ("text", "a "), ("image", uri), ("text", " b")
inline std::vector<std::pair<bool, std::string>> split_prompt(const std::string& text) {
  std::vector<std::pair<bool, std::string>> out;          // (is image, text or uri)
  size_t pos = 0, scan = 0;
  while (true) {
    const size_t at = text.find("![](", scan);
    if (at == std::string::npos) break;
    const size_t close = text.find(')', at + 4);
    if (close == std::string::npos) break;                 // no closing parenthesis anywhere behind: nothing more can match
    if (close == at + 4) { scan = at + 1; continue; }      // "![]()": an empty reference is no image
    if (at > pos) out.emplace_back(false, text.substr(pos, at - pos));
    out.emplace_back(true, text.substr(at + 4, close - at - 4));
    pos = scan = close + 1;
  }
  if (pos < text.size()) out.emplace_back(false, text.substr(pos));
  return out;
}

// How many feature tokens an image becomes, from the vision configuration shard 0 hands over.
struct ImagePolicy {
  enum Kind { None, OnePerImage, LlavaNext } kind = None;
  uint32_t image_token = 0;
  long image_size = 336, patch_size = 14, extra_tokens = 1;
  bool drop_class_token = true;                     // vision_feature_select_strategy "default"
  std::vector<std::pair<long, long>> pinpoints;     // (height, width) of the any-resolution canvases

  static ImagePolicy from_json(const json::Value& v) {
    ImagePolicy p;
    const std::string& kind = v["kind"].as_string();
    p.image_token = (uint32_t)v["image_token"].as_int();
    if (kind == "one_per_image") p.kind = OnePerImage;
    else if (kind == "llava_next") {
      p.kind = LlavaNext;
      p.image_size = (long)v["image_size"].as_int(336);
      p.patch_size = (long)v["patch_size"].as_int(14);
      p.extra_tokens = (long)v["extra_tokens"].as_int(1);
      p.drop_class_token = v["strategy"].as_string() != "full";
      for (auto& pp : v["pinpoints"].items()) if (pp.size() == 2) p.pinpoints.emplace_back((long)pp.items()[0].as_int(), (long)pp.items()[1].as_int());
      if (p.pinpoints.empty() || p.image_size <= 0 || p.patch_size <= 0) p.kind = None;
    }
    return p;
  }

  // Feature tokens of an image of `h` x `w` pixels (LLaVA-NeXT: the base tile plus the unpadded any-resolution grid with one
  // newline feature per row; config.rs:87-110 of the reference router).
  long features(long h, long w) const {
    if (kind == OnePerImage) return 1;
    const long side = image_size / patch_size;
    const long base = side * side + extra_tokens - (drop_class_token ? 1 : 0);
    long bh = 0, bw = 0, best_eff = -1;
    double best_waste = 1e300;
    for (auto& c : pinpoints) {
      const double scale = std::min((double)c.second / (double)w, (double)c.first / (double)h);
      const long eff = std::min((long)((double)w * scale) * (long)((double)h * scale), w * h);
      const double waste = (double)c.first * (double)c.second - (double)eff;
      if (eff > best_eff || (eff == best_eff && waste < best_waste)) { bh = c.first; bw = c.second; best_eff = eff; best_waste = waste; }
    }
    const long gh = bh / image_size * side, gw = bw / image_size * side;
    long rows, cols;
    auto round7 = [](double x) { return (long)(std::nearbyint(x * 1e7) / 1e7); };
    if ((double)w / (double)h > (double)gw / (double)gh) {
      const long new_h = round7((double)h * ((double)gw / (double)w));
      const long pad = (gh - new_h) / 2;
      rows = gh - 2 * pad; cols = gw;
    } else {
      const long new_w = round7((double)w * ((double)gh / (double)h));
      const long pad = (gw - new_w) / 2;
      rows = gh; cols = gw - 2 * pad;
    }
    return base + rows * (cols + 1);
  }

  // Number of image tokens for `uri`, or -1 when this image has to go to the shard.
  long count(const std::string& uri) const {
    if (kind == None) return -1;
    if (uri.compare(0, 5, "data:") != 0) return -1;
    const size_t comma = uri.find(',');
    if (comma == std::string::npos || comma < 7 || uri.compare(comma - 7, 7, ";base64") != 0) return -1;
    const std::string bytes = base64_decode(uri.substr(comma + 1));
    long w = 0, h = 0;
    if (!probe_image_size(bytes, &w, &h) || w > 65535 || h > 65535) return -1;
    return features(h, w);
  }
};

}  // namespace img
}  // namespace lx
