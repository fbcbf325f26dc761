// Minimal protobuf wire-format reader / writer (varint, fixed32/64, length-delimited) used by the generated
// message structs in pb_gen.hpp.  No reflection, no arena: messages are plain structs.
#pragma once
#include <cstdint>
#include <cstring>
#include <string>

namespace pb {

struct Writer {
  std::string buf;
  void varint(uint64_t v) {
    while (v >= 0x80) { buf.push_back((char)(v | 0x80)); v >>= 7; }
    buf.push_back((char)v);
  }
  void tag(uint32_t field, uint32_t wire_type) { varint(((uint64_t)field << 3) | wire_type); }
  void f32(float f) { char b[4]; std::memcpy(b, &f, 4); buf.append(b, 4); }
  void f64(double f) { char b[8]; std::memcpy(b, &f, 8); buf.append(b, 8); }
  void bytes(const std::string& s) { varint(s.size()); buf.append(s); }
};

struct Reader {
  const uint8_t* p = nullptr;
  const uint8_t* end = nullptr;
  Reader() = default;
  explicit Reader(const std::string& s) : p((const uint8_t*)s.data()), end((const uint8_t*)s.data() + s.size()) {}
  Reader(const uint8_t* b, const uint8_t* e) : p(b), end(e) {}
  bool done() const { return p >= end; }
  bool varint(uint64_t& v) {
    v = 0;
    for (int shift = 0; shift < 64 && p < end; shift += 7) {
      uint8_t b = *p++;
      v |= (uint64_t)(b & 0x7f) << shift;
      if (!(b & 0x80)) return true;
    }
    return false;
  }
  bool tag(uint32_t& field, uint32_t& wt) {
    uint64_t v;
    if (!varint(v)) return false;
    field = (uint32_t)(v >> 3);
    wt = (uint32_t)(v & 7);
    return field != 0;
  }
  bool f32(float& f) { if (end - p < 4) return false; std::memcpy(&f, p, 4); p += 4; return true; }
  bool f64(double& f) { if (end - p < 8) return false; std::memcpy(&f, p, 8); p += 8; return true; }
  bool bytes(std::string& s) {
    uint64_t n;
    if (!varint(n) || (uint64_t)(end - p) < n) return false;
    s.assign((const char*)p, (size_t)n);
    p += n;
    return true;
  }
  bool sub(Reader& r) {
    uint64_t n;
    if (!varint(n) || (uint64_t)(end - p) < n) return false;
    r = Reader(p, p + n);
    p += n;
    return true;
  }
  bool skip(uint32_t wt) {
    uint64_t v;
    switch (wt) {
      case 0: return varint(v);
      case 1: if (end - p < 8) return false; p += 8; return true;
      case 2: if (!varint(v) || (uint64_t)(end - p) < v) return false; p += v; return true;
      case 5: if (end - p < 4) return false; p += 4; return true;
      default: return false;
    }
  }
};

}  // namespace pb
