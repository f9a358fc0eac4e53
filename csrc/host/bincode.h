// Minimal bincode-2 "standard configuration" codec (little-endian, variable-length integers),
// the wire format ToRSh's `oxicode::config::standard()` produces for TRSH tensor metadata, model
// state files and TCP-store messages.
//   unsigned: v < 251 -> 1 byte; 251 + u16; 252 + u32; 253 + u64
//   signed:   zig-zag, then as unsigned
//   bool: 1 byte; Option: tag byte 0/1 + value; String / Vec / Map: length (as u64 varint) + items
//   enum: variant index as u32 varint + fields; f32 / f64: raw little-endian
#pragma once
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

namespace tsh {

struct Writer {
  std::vector<uint8_t> buf;
  void u8(uint8_t v) { buf.push_back(v); }
  void raw(const void* p, size_t n) {
    const uint8_t* b = static_cast<const uint8_t*>(p);
    buf.insert(buf.end(), b, b + n);
  }
  void varu(uint64_t v) {
    if (v < 251) {
      u8((uint8_t)v);
    } else if (v <= 0xFFFF) {
      u8(251);
      uint16_t x = (uint16_t)v;
      raw(&x, 2);
    } else if (v <= 0xFFFFFFFFull) {
      u8(252);
      uint32_t x = (uint32_t)v;
      raw(&x, 4);
    } else {
      u8(253);
      raw(&v, 8);
    }
  }
  void vari(int64_t v) { varu(((uint64_t)v << 1) ^ (uint64_t)(v >> 63)); }
  void boolean(bool b) { u8(b ? 1 : 0); }
  void str(const std::string& s) {
    varu(s.size());
    raw(s.data(), s.size());
  }
  void bytes(const void* p, size_t n) {
    varu(n);
    raw(p, n);
  }
  void f32(float v) { raw(&v, 4); }
  void f64(double v) { raw(&v, 8); }
};

struct Reader {
  const uint8_t* p;
  const uint8_t* end;
  Reader(const void* data, size_t n) : p(static_cast<const uint8_t*>(data)), end(p + n) {}
  void need(size_t n) const {
    if ((size_t)(end - p) < n) throw std::runtime_error("bincode: unexpected end of input");
  }
  uint8_t u8() {
    need(1);
    return *p++;
  }
  template <typename T> T fixed() {
    need(sizeof(T));
    T v;
    std::memcpy(&v, p, sizeof(T));
    p += sizeof(T);
    return v;
  }
  uint64_t varu() {
    uint8_t t = u8();
    if (t < 251) return t;
    if (t == 251) return fixed<uint16_t>();
    if (t == 252) return fixed<uint32_t>();
    if (t == 253) return fixed<uint64_t>();
    throw std::runtime_error("bincode: 128-bit integers are not supported");
  }
  int64_t vari() {
    uint64_t z = varu();
    return (int64_t)(z >> 1) ^ -(int64_t)(z & 1);
  }
  bool boolean() {
    uint8_t b = u8();
    if (b > 1) throw std::runtime_error("bincode: invalid bool");
    return b == 1;
  }
  std::string str() {
    uint64_t n = varu();
    need(n);
    std::string s(reinterpret_cast<const char*>(p), n);
    p += n;
    return s;
  }
  std::vector<uint8_t> bytes() {
    uint64_t n = varu();
    need(n);
    std::vector<uint8_t> v(p, p + n);
    p += n;
    return v;
  }
  float f32() { return fixed<float>(); }
  double f64() { return fixed<double>(); }
  size_t remaining() const { return (size_t)(end - p); }
};

}  // namespace tsh
