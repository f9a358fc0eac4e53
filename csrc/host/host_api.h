// Shared declarations of the host runtime library (libtorsh_b200_host.so).
#pragma once
#include <cstdint>
#include <string>

#define TSH_EXPORT extern "C" __attribute__((visibility("default")))

namespace tsh {
extern thread_local std::string g_err;
uint32_t crc32_update(uint32_t crc, const uint8_t* p, size_t n);
}  // namespace tsh
