// Shared declarations of the host runtime library (libtorsh_b200_host.so).
#pragma once
#include <cstdint>
#include <string>

#define TSH_EXPORT extern "C" __attribute__((visibility("default")))

namespace tsh {
// Last error message of the calling thread (function-local TLS: safe across translation units).
inline std::string& err_slot() {
  static thread_local std::string e;
  return e;
}
#define g_err (::tsh::err_slot())
uint32_t crc32_update(uint32_t crc, const uint8_t* p, size_t n);
}  // namespace tsh
