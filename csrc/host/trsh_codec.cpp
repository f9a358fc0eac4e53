// TRSH tensor file codec (the reference's `.trsh` / `.bin` tensor format,
// crates/torsh-tensor/src/serialize/binary.rs:12-16,84-95,249-344,356-458):
//   28-byte little-endian header: "TRSH" | version u32 = 1 | metadata_size u64 | data_size u64 | crc32 u32
//   metadata = bincode-standard(TensorMetadata) with fields in declaration order
//     shape{dims: Vec<usize>}, device: DeviceType{Cpu, Cuda(i), Metal(i), Wgpu(i)}, requires_grad: bool,
//     dtype_name: String, version: String, timestamp: u64, custom_metadata: Map<String,String>,
//     format: String ("Binary"), data_size: usize, compressed: bool, checksum: Option<String>
//     (crates/torsh-tensor/src/serialize/common.rs:315-383; written with checksum = None)
//   data = raw little-endian elements, zstd-compressed when compression_level > 0
//   crc32 (poly 0xEDB88320, init 0xFFFFFFFF, final NOT) over metadata || data as stored
// zstd comes from the system libzstd.so.1 through dlopen; without it only level 0 is available.
#include <dlfcn.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <map>

#include "bincode.h"
#include "host_api.h"

namespace tsh {

static uint32_t crc_table[256];
static bool crc_ready = false;
static void crc_init() {
  for (uint32_t i = 0; i < 256; ++i) {
    uint32_t c = i;
    for (int k = 0; k < 8; ++k) c = (c & 1) ? (0xEDB88320u ^ (c >> 1)) : (c >> 1);
    crc_table[i] = c;
  }
  crc_ready = true;
}
uint32_t crc32_update(uint32_t crc, const uint8_t* p, size_t n) {
  if (!crc_ready) crc_init();
  for (size_t i = 0; i < n; ++i) crc = crc_table[(crc ^ p[i]) & 0xFF] ^ (crc >> 8);
  return crc;
}

struct Zstd {
  void* h = nullptr;
  size_t (*compressBound)(size_t) = nullptr;
  size_t (*compress)(void*, size_t, const void*, size_t, int) = nullptr;
  size_t (*decompress)(void*, size_t, const void*, size_t) = nullptr;
  unsigned long long (*frameContentSize)(const void*, size_t) = nullptr;
  unsigned (*isError)(size_t) = nullptr;
  bool ok() const { return h && compressBound && compress && decompress && frameContentSize && isError; }
};
static Zstd& zstd() {
  static Zstd z;
  static bool tried = false;
  if (!tried) {
    tried = true;
    z.h = dlopen("libzstd.so.1", RTLD_NOW | RTLD_LOCAL);
    if (z.h) {
      z.compressBound = (size_t(*)(size_t))dlsym(z.h, "ZSTD_compressBound");
      z.compress = (size_t(*)(void*, size_t, const void*, size_t, int))dlsym(z.h, "ZSTD_compress");
      z.decompress = (size_t(*)(void*, size_t, const void*, size_t))dlsym(z.h, "ZSTD_decompress");
      z.frameContentSize = (unsigned long long (*)(const void*, size_t))dlsym(z.h, "ZSTD_getFrameContentSize");
      z.isError = (unsigned (*)(size_t))dlsym(z.h, "ZSTD_isError");
    }
  }
  return z;
}

static std::string json_escape(const std::string& s) {
  std::string o;
  for (char c : s) {
    if (c == '"' || c == '\\') { o += '\\'; o += c; }
    else if (c == '\n') o += "\\n";
    else if ((unsigned char)c < 0x20) { char b[8]; snprintf(b, 8, "\\u%04x", c); o += b; }
    else o += c;
  }
  return o;
}


}  // namespace tsh
using namespace tsh;

TSH_EXPORT const char* tsh_last_error() { return g_err.c_str(); }
TSH_EXPORT void tsh_free(void* p) { free(p); }
TSH_EXPORT uint32_t tsh_crc32(const void* data, uint64_t n) {
  return ~crc32_update(0xFFFFFFFFu, static_cast<const uint8_t*>(data), n);
}
TSH_EXPORT int tsh_zstd_available() { return zstd().ok() ? 1 : 0; }

// device_kind: 0 cpu, 1 cuda, 2 metal, 3 wgpu. meta_kv: nmeta pairs (key, value) as C strings.
TSH_EXPORT int tsh_trsh_encode(const int64_t* dims, int ndim, int device_kind, int64_t device_index,
                               int requires_grad, const char* dtype_name, const char* version, uint64_t timestamp,
                               const char** meta_kv, int nmeta, const void* data, uint64_t data_bytes,
                               int compression_level, uint8_t** out, uint64_t* out_len) {
  try {
    std::vector<uint8_t> stored;
    bool compressed = false;
    if (compression_level > 0) {
      Zstd& z = zstd();
      if (!z.ok()) throw std::runtime_error("zstd compression requested but libzstd.so.1 is not loadable");
      int level = std::min(std::max(compression_level, 1), 22);
      stored.resize(z.compressBound(data_bytes));
      size_t n = z.compress(stored.data(), stored.size(), data, data_bytes, level);
      if (z.isError(n)) throw std::runtime_error("zstd compression failed");
      stored.resize(n);
      compressed = true;
    } else {
      stored.assign(static_cast<const uint8_t*>(data), static_cast<const uint8_t*>(data) + data_bytes);
    }
    Writer w;
    w.varu((uint64_t)ndim);
    for (int i = 0; i < ndim; ++i) w.varu((uint64_t)dims[i]);
    w.varu((uint64_t)device_kind);
    if (device_kind != 0) w.varu((uint64_t)device_index);
    w.boolean(requires_grad != 0);
    w.str(dtype_name);
    w.str(version);
    w.varu(timestamp);
    std::map<std::string, std::string> meta;
    for (int i = 0; i < nmeta; ++i) meta[meta_kv[2 * i]] = meta_kv[2 * i + 1];
    w.varu(meta.size());
    for (auto& kv : meta) { w.str(kv.first); w.str(kv.second); }
    w.str("Binary");
    w.varu(stored.size());
    w.boolean(compressed);
    w.u8(0);  // checksum: None
    uint32_t crc = crc32_update(0xFFFFFFFFu, w.buf.data(), w.buf.size());
    crc = ~crc32_update(crc, stored.data(), stored.size());
    uint64_t total = 28 + w.buf.size() + stored.size();
    uint8_t* o = static_cast<uint8_t*>(malloc(total));
    if (!o) throw std::runtime_error("out of memory");
    memcpy(o, "TRSH", 4);
    uint32_t ver = 1;
    uint64_t ms = w.buf.size(), ds = stored.size();
    memcpy(o + 4, &ver, 4);
    memcpy(o + 8, &ms, 8);
    memcpy(o + 16, &ds, 8);
    memcpy(o + 24, &crc, 4);
    memcpy(o + 28, w.buf.data(), ms);
    memcpy(o + 28 + ms, stored.data(), ds);
    *out = o;
    *out_len = total;
    return 0;
  } catch (const std::exception& e) {
    g_err = e.what();
    return -1;
  }
}

// Decodes a TRSH buffer. *meta_json receives a malloc'd JSON object with every metadata field;
// *data receives the malloc'd (decompressed) element bytes.
TSH_EXPORT int tsh_trsh_decode(const uint8_t* buf, uint64_t len, char** meta_json, uint8_t** data, uint64_t* data_len) {
  try {
    if (len < 28 || memcmp(buf, "TRSH", 4) != 0) throw std::runtime_error("not a TRSH file (bad magic)");
    uint32_t ver, crc;
    uint64_t ms, ds;
    memcpy(&ver, buf + 4, 4);
    memcpy(&ms, buf + 8, 8);
    memcpy(&ds, buf + 16, 8);
    memcpy(&crc, buf + 24, 4);
    if (ver != 1) throw std::runtime_error("unsupported TRSH version " + std::to_string(ver));
    if (ms == 0 || ds == 0) throw std::runtime_error("TRSH header has a zero section size");
    if (28 + ms + ds > len) throw std::runtime_error("TRSH file is truncated");
    uint32_t got = ~crc32_update(0xFFFFFFFFu, buf + 28, ms + ds);
    if (got != crc) {
      char m[96];
      snprintf(m, 96, "TRSH checksum mismatch: header 0x%08X, computed 0x%08X", crc, got);
      throw std::runtime_error(m);
    }
    Reader r(buf + 28, ms);
    struct J { std::string s; J& operator<<(const char* c) { s += c; return *this; } J& operator<<(const std::string& c) { s += c; return *this; } J& operator<<(uint64_t v) { s += std::to_string(v); return *this; } std::string str() const { return s; } } js;
    js << "{\"shape\":[";
    uint64_t nd = r.varu();
    for (uint64_t i = 0; i < nd; ++i) js << (i ? "," : "") << r.varu();
    js << "]";
    uint64_t dk = r.varu();
    uint64_t di = dk != 0 ? r.varu() : 0;
    static const char* kinds[] = {"cpu", "cuda", "metal", "wgpu"};
    if (dk > 3) throw std::runtime_error("unknown device variant");
    js << ",\"device\":\"" << kinds[dk] << "\",\"device_index\":" << di;
    js << ",\"requires_grad\":" << (r.boolean() ? "true" : "false");
    js << ",\"dtype_name\":\"" << json_escape(r.str()) << "\"";
    js << ",\"version\":\"" << json_escape(r.str()) << "\"";
    js << ",\"timestamp\":" << r.varu();
    uint64_t nm = r.varu();
    js << ",\"custom_metadata\":{";
    for (uint64_t i = 0; i < nm; ++i) {
      std::string k = r.str(), v = r.str();
      js << (i ? "," : "") << "\"" << json_escape(k) << "\":\"" << json_escape(v) << "\"";
    }
    js << "}";
    js << ",\"format\":\"" << json_escape(r.str()) << "\"";
    js << ",\"data_size\":" << r.varu();
    bool compressed = r.boolean();
    js << ",\"compressed\":" << (compressed ? "true" : "false");
    if (r.u8() == 1) js << ",\"checksum\":\"" << json_escape(r.str()) << "\""; else js << ",\"checksum\":null";
    js << "}";
    const uint8_t* payload = buf + 28 + ms;
    uint8_t* o;
    uint64_t on;
    if (compressed) {
      Zstd& z = zstd();
      if (!z.ok()) throw std::runtime_error("file is zstd-compressed but libzstd.so.1 is not loadable");
      unsigned long long n = z.frameContentSize(payload, ds);
      if (n == (unsigned long long)-1 || n == (unsigned long long)-2) throw std::runtime_error("zstd frame has no content size");
      o = static_cast<uint8_t*>(malloc(n ? n : 1));
      size_t k = z.decompress(o, n, payload, ds);
      if (z.isError(k) || k != n) { free(o); throw std::runtime_error("zstd decompression failed"); }
      on = n;
    } else {
      o = static_cast<uint8_t*>(malloc(ds));
      memcpy(o, payload, ds);
      on = ds;
    }
    std::string s = js.str();
    char* mj = static_cast<char*>(malloc(s.size() + 1));
    memcpy(mj, s.c_str(), s.size() + 1);
    *meta_json = mj;
    *data = o;
    *data_len = on;
    return 0;
  } catch (const std::exception& e) {
    g_err = e.what();
    return -1;
  }
}
