// Symmetric heap over the CUDA virtual-memory API: every rank of one NVSwitch domain allocates a block of the same
// size, exports it as a POSIX file descriptor, receives its peers' descriptors over abstract-namespace Unix datagram
// sockets (SCM_RIGHTS) and maps every peer's block into its own address space; optionally the blocks are bound to one
// multicast object so that `multimem.*` instructions reach all copies through the switch.
//
// All driver entry points are looked up at run time (cudaGetDriverEntryPoint): the library does not link libcuda.
// Every step that can fail undoes what the call has mapped so far, in reverse order, before it returns: a block is
// either fully usable on return or leaves no mapping, reservation or handle behind.
//
// The calls are COLLECTIVE: every rank of the job calls tb_symm_alloc / tb_symm_free in the same order. Ranks find
// each other by the job string (unique per job and per group; the caller derives it from its rendezvous) and their
// rank index; the caller must make sure (a barrier on its process group) that every rank has returned from
// tb_symm_init before any rank calls tb_symm_alloc.
//
// The reference's device-memory layer has pools and unified buffers for one process
// (crates/torsh-backend/src/cuda/memory/allocation.rs) and no cross-process mapping.
#include <errno.h>
#include <poll.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <mutex>
#include <string>
#include <vector>

#include "host_util.h"

namespace tb {
namespace {

constexpr int SYMM_MAX_RANKS = 8;
constexpr int SYMM_TIMEOUT_MS = 30000;

template <typename Fn>
bool entry(const char* name, Fn* out) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || !p)
    return false;
  *out = (Fn)p;
  return true;
}

struct Driver {
  CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
  CUresult (*MemRelease)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*MemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
  CUresult (*MemExportToShareableHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long) = nullptr;
  CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType) = nullptr;
  CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
  CUresult (*MemAddressFree)(CUdeviceptr, size_t) = nullptr;
  CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
  CUresult (*MemUnmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  CUresult (*MulticastCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*) = nullptr;
  CUresult (*MulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice) = nullptr;
  CUresult (*MulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long) = nullptr;
  CUresult (*MulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t) = nullptr;
  CUresult (*MulticastGetGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags) = nullptr;
  CUresult (*DeviceGet)(CUdevice*, int) = nullptr;
  CUresult (*DeviceGetAttribute)(int*, CUdevice_attribute, CUdevice) = nullptr;
  bool ok = false, multicast = false;
};

Driver& driver() {
  static Driver d;
  static std::once_flag once;
  std::call_once(once, [] {
    d.ok = entry("cuMemCreate", &d.MemCreate) && entry("cuMemRelease", &d.MemRelease) &&
           entry("cuMemGetAllocationGranularity", &d.MemGetAllocationGranularity) &&
           entry("cuMemExportToShareableHandle", &d.MemExportToShareableHandle) &&
           entry("cuMemImportFromShareableHandle", &d.MemImportFromShareableHandle) &&
           entry("cuMemAddressReserve", &d.MemAddressReserve) && entry("cuMemAddressFree", &d.MemAddressFree) &&
           entry("cuMemMap", &d.MemMap) && entry("cuMemUnmap", &d.MemUnmap) && entry("cuMemSetAccess", &d.MemSetAccess) &&
           entry("cuDeviceGet", &d.DeviceGet) && entry("cuDeviceGetAttribute", &d.DeviceGetAttribute);
    d.multicast = d.ok && entry("cuMulticastCreate", &d.MulticastCreate) && entry("cuMulticastAddDevice", &d.MulticastAddDevice) &&
                  entry("cuMulticastBindMem", &d.MulticastBindMem) && entry("cuMulticastUnbind", &d.MulticastUnbind) &&
                  entry("cuMulticastGetGranularity", &d.MulticastGetGranularity);
  });
  return d;
}

// ---- rendezvous over abstract Unix datagram sockets ---------------------------------------------------------------
struct Msg {
  uint32_t magic, src, seq, phase;  // seq = allocation number, phase = step inside the allocation
};
constexpr uint32_t MSG_MAGIC = 0x7b5e11a9u;

struct Heap {
  std::string job;
  int rank = -1, world = 0, device = 0, sock = -1;
  uint32_t seq = 0;
  std::vector<std::pair<Msg, int>> pending;  // messages that arrived early, with the descriptor they carried (-1: none)
  std::mutex mu;
};
constexpr int SYMM_MAX_HEAPS = 16;  // one per process group that owns symmetric buffers
Heap g_heaps[SYMM_MAX_HEAPS];
std::mutex g_heaps_mu;

sockaddr_un peer_addr(const std::string& job, int rank, socklen_t* len) {
  sockaddr_un a;
  memset(&a, 0, sizeof(a));
  a.sun_family = AF_UNIX;
  std::string name = "tb_symm_" + job + "_" + std::to_string(rank);
  if (name.size() > sizeof(a.sun_path) - 2) name.resize(sizeof(a.sun_path) - 2);
  memcpy(a.sun_path + 1, name.data(), name.size());  // sun_path[0] == 0: abstract namespace, vanishes with the socket
  *len = (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + name.size());
  return a;
}

int send_msg(Heap& h, int dst, uint32_t phase, int fd) {
  Msg m{MSG_MAGIC, (uint32_t)h.rank, h.seq, phase};
  socklen_t alen;
  sockaddr_un addr = peer_addr(h.job, dst, &alen);
  iovec iov{&m, sizeof(m)};
  msghdr mh;
  memset(&mh, 0, sizeof(mh));
  mh.msg_name = &addr;
  mh.msg_namelen = alen;
  mh.msg_iov = &iov;
  mh.msg_iovlen = 1;
  alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
  if (fd >= 0) {
    memset(ctrl, 0, sizeof(ctrl));
    mh.msg_control = ctrl;
    mh.msg_controllen = sizeof(ctrl);
    cmsghdr* c = CMSG_FIRSTHDR(&mh);
    c->cmsg_level = SOL_SOCKET;
    c->cmsg_type = SCM_RIGHTS;
    c->cmsg_len = CMSG_LEN(sizeof(int));
    memcpy(CMSG_DATA(c), &fd, sizeof(int));
  }
  for (int attempt = 0; attempt < 300; ++attempt) {
    if (sendmsg(h.sock, &mh, 0) == (ssize_t)sizeof(m)) return 0;
    if (errno != ECONNREFUSED && errno != ENOENT && errno != EAGAIN && errno != ENOBUFS) break;
    usleep(100000);  // the peer's socket is not bound yet (or its queue is full): bounded retry
  }
  TB_FAIL(TB_E_CUDA, "symmetric heap: sendmsg to rank %d failed: %s", dst, strerror(errno));
}

// Receives the message (src, seq, phase); *fd gets the descriptor it carried (-1 if none). Bounded by SYMM_TIMEOUT_MS.
int recv_msg(Heap& h, int src, uint32_t phase, int* fd) {
  for (size_t i = 0; i < h.pending.size(); ++i) {
    const Msg& m = h.pending[i].first;
    if ((int)m.src == src && m.seq == h.seq && m.phase == phase) {
      *fd = h.pending[i].second;
      h.pending.erase(h.pending.begin() + i);
      return 0;
    }
  }
  int waited = 0;
  while (waited < SYMM_TIMEOUT_MS) {
    pollfd p{h.sock, POLLIN, 0};
    int r = poll(&p, 1, 200);
    if (r < 0 && errno != EINTR) TB_FAIL(TB_E_CUDA, "symmetric heap: poll failed: %s", strerror(errno));
    if (r <= 0) {
      waited += 200;
      continue;
    }
    Msg m;
    iovec iov{&m, sizeof(m)};
    msghdr mh;
    memset(&mh, 0, sizeof(mh));
    mh.msg_iov = &iov;
    mh.msg_iovlen = 1;
    alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
    mh.msg_control = ctrl;
    mh.msg_controllen = sizeof(ctrl);
    ssize_t n = recvmsg(h.sock, &mh, 0);
    if (n != (ssize_t)sizeof(m) || m.magic != MSG_MAGIC) continue;
    int got = -1;
    for (cmsghdr* c = CMSG_FIRSTHDR(&mh); c; c = CMSG_NXTHDR(&mh, c))
      if (c->cmsg_level == SOL_SOCKET && c->cmsg_type == SCM_RIGHTS) memcpy(&got, CMSG_DATA(c), sizeof(int));
    if ((int)m.src == src && m.seq == h.seq && m.phase == phase) {
      *fd = got;
      return 0;
    }
    h.pending.emplace_back(m, got);
  }
  TB_FAIL(TB_E_CUDA, "symmetric heap: rank %d did not answer within %d ms (allocation %u, phase %u)", src,
          SYMM_TIMEOUT_MS, h.seq, phase);
}

int barrier(Heap& h, uint32_t phase) {
  for (int q = 0; q < h.world; ++q)
    if (q != h.rank)
      if (int r = send_msg(h, q, phase, -1)) return r;
  for (int q = 0; q < h.world; ++q)
    if (q != h.rank) {
      int fd = -1;
      if (int r = recv_msg(h, q, phase, &fd)) return r;
      if (fd >= 0) close(fd);
    }
  return 0;
}

}  // namespace

struct SymmBlock {
  size_t size = 0;                              // mapped bytes (the request rounded up to the granularity)
  CUmemGenericAllocationHandle mem[SYMM_MAX_RANKS] = {};
  CUdeviceptr va[SYMM_MAX_RANKS] = {};
  bool have_mem[SYMM_MAX_RANKS] = {}, mapped[SYMM_MAX_RANKS] = {};
  CUmemGenericAllocationHandle mc = 0;
  CUdeviceptr mc_va = 0;
  bool have_mc = false, mc_bound = false, mc_mapped = false;
  int rank = 0, world = 0, device = 0, heap = 0;
};

namespace {
void destroy(SymmBlock* b) {
  Driver& d = driver();
  if (!b) return;
  if (b->mc_mapped) d.MemUnmap(b->mc_va, b->size);
  if (b->mc_va) d.MemAddressFree(b->mc_va, b->size);
  if (b->mc_bound) {
    CUdevice dev;
    if (d.DeviceGet(&dev, b->device) == CUDA_SUCCESS) d.MulticastUnbind(b->mc, dev, 0, b->size);
  }
  if (b->have_mc) d.MemRelease(b->mc);
  for (int q = 0; q < b->world; ++q) {
    if (b->mapped[q]) d.MemUnmap(b->va[q], b->size);
    if (b->va[q]) d.MemAddressFree(b->va[q], b->size);
    if (b->have_mem[q]) d.MemRelease(b->mem[q]);
  }
  delete b;
}
}  // namespace
}  // namespace tb
using namespace tb;

#define TB_DRV(expr, blk)                                                                             \
  do {                                                                                                \
    CUresult _r = (expr);                                                                             \
    if (_r != CUDA_SUCCESS) {                                                                         \
      destroy(blk);                                                                                   \
      TB_FAIL(TB_E_CUDA, "%s failed with CUresult %d (%s:%d)", #expr, (int)_r, __FILE__, __LINE__);   \
    }                                                                                                 \
  } while (0)

// Opens a heap for one group of ranks and binds this rank's rendezvous socket; returns the heap index (>= 0) or a
// negative error code. `job` must be the same string on every rank of the group and unique on the host.
TB_EXPORT int tb_symm_init(const char* job, int rank, int world, int device) {
  TB_ENSURE_DEVICE();
  if (!job || world < 1 || world > SYMM_MAX_RANKS || rank < 0 || rank >= world)
    TB_FAIL(TB_E_ARG, "symmetric heap: bad job / rank / world");
  if (!driver().ok) TB_FAIL(TB_E_CUDA, "symmetric heap: the virtual-memory driver entry points are not available");
  if (device != g_device().load())
    TB_FAIL(TB_E_ARG, "symmetric heap: device %d is not the library's current device (%d): call tb_set_device first", device,
            g_device().load());
  std::lock_guard<std::mutex> all(g_heaps_mu);
  int idx = -1;
  for (int i = 0; i < SYMM_MAX_HEAPS && idx < 0; ++i)
    if (g_heaps[i].sock < 0) idx = i;
  if (idx < 0) TB_FAIL(TB_E_TOO_LARGE, "symmetric heap: more than %d heaps open", SYMM_MAX_HEAPS);
  Heap& h = g_heaps[idx];
  std::lock_guard<std::mutex> lk(h.mu);
  h.sock = socket(AF_UNIX, SOCK_DGRAM | SOCK_CLOEXEC, 0);
  if (h.sock < 0) TB_FAIL(TB_E_CUDA, "symmetric heap: socket() failed: %s", strerror(errno));
  h.job = job;
  h.rank = rank;
  h.world = world;
  h.device = device;
  h.seq = 0;
  h.pending.clear();
  socklen_t alen;
  sockaddr_un addr = peer_addr(h.job, rank, &alen);
  if (bind(h.sock, (sockaddr*)&addr, alen) != 0) {
    const int e = errno;
    close(h.sock);
    h.sock = -1;
    TB_FAIL(TB_E_CUDA, "symmetric heap: bind failed: %s", strerror(e));
  }
  return idx;
}

// 1 when the device and driver can create multicast objects (NVSwitch in-switch reduction), else 0.
TB_EXPORT int tb_symm_multicast_supported(int device) {
  if (tb::ensure_device()) return 0;
  Driver& d = driver();
  if (!d.multicast) return 0;
  CUdevice dev;
  int v = 0;
  if (d.DeviceGet(&dev, device) != CUDA_SUCCESS) return 0;
  if (d.DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) != CUDA_SUCCESS) return 0;
  return v;
}

// Collective allocation of `bytes` per rank. On success *handle identifies the block, peer_ptrs[q] is rank q's block
// as mapped into THIS process (peer_ptrs[rank] is the local one), *mc_ptr the multicast address (0 when
// want_multicast == 0 or multicast is not supported) and *mapped_bytes the size that was mapped.
TB_EXPORT int tb_symm_alloc(int heap, size_t bytes, int want_multicast, void** handle, void** peer_ptrs, void** mc_ptr,
                            size_t* mapped_bytes) {
  TB_ENSURE_DEVICE();
  Driver& d = driver();
  if (heap < 0 || heap >= SYMM_MAX_HEAPS) TB_FAIL(TB_E_ARG, "symmetric heap: bad heap index %d", heap);
  Heap& h = g_heaps[heap];
  std::lock_guard<std::mutex> lk(h.mu);
  if (h.sock < 0) TB_FAIL(TB_E_ARG, "symmetric heap: tb_symm_init has not been called");
  if (!handle || !peer_ptrs || bytes == 0) TB_FAIL(TB_E_ARG, "symmetric heap: bad arguments");
  h.seq += 1;
  const bool use_mc = want_multicast && h.world > 1 && tb_symm_multicast_supported(h.device);
  CUmemAllocationProp prop;
  memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = h.device;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  size_t gran = 0;
  SymmBlock* b = new SymmBlock();
  b->rank = h.rank;
  b->world = h.world;
  b->device = h.device;
  b->heap = heap;
  TB_DRV(d.MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED), b);
  CUmulticastObjectProp mprop;
  memset(&mprop, 0, sizeof(mprop));
  if (use_mc) {
    mprop.numDevices = (unsigned)h.world;
    mprop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    mprop.size = bytes;
    size_t mgran = 0;
    TB_DRV(d.MulticastGetGranularity(&mgran, &mprop, CU_MULTICAST_GRANULARITY_RECOMMENDED), b);
    if (mgran > gran) gran = mgran;
  }
  b->size = (bytes + gran - 1) / gran * gran;
  mprop.size = b->size;

  // 1. local physical block, exported and sent to every peer
  TB_DRV(d.MemCreate(&b->mem[h.rank], b->size, &prop, 0), b);
  b->have_mem[h.rank] = true;
  int my_fd = -1;
  TB_DRV(d.MemExportToShareableHandle(&my_fd, b->mem[h.rank], CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0), b);
  int rc = 0;
  for (int q = 0; q < h.world && !rc; ++q)
    if (q != h.rank) rc = send_msg(h, q, 1, my_fd);
  close(my_fd);
  // 2. peers' blocks imported
  for (int q = 0; q < h.world && !rc; ++q) {
    if (q == h.rank) continue;
    int fd = -1;
    rc = recv_msg(h, q, 1, &fd);
    if (rc) break;
    if (fd < 0) {
      rc = TB_E_CUDA;
      snprintf(tb::last_error_buf(), 512, "symmetric heap: rank %d sent no descriptor", q);
      break;
    }
    CUresult r = d.MemImportFromShareableHandle(&b->mem[q], (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
    close(fd);
    if (r != CUDA_SUCCESS) {
      rc = TB_E_CUDA;
      snprintf(tb::last_error_buf(), 512, "symmetric heap: import of rank %d's block failed with CUresult %d", q, (int)r);
      break;
    }
    b->have_mem[q] = true;
  }
  if (rc) {
    destroy(b);
    return rc;
  }
  // 3. every block mapped read / write for this device
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = h.device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  for (int q = 0; q < h.world; ++q) {
    TB_DRV(d.MemAddressReserve(&b->va[q], b->size, gran, 0, 0), b);
    TB_DRV(d.MemMap(b->va[q], b->size, 0, b->mem[q], 0), b);
    b->mapped[q] = true;
    TB_DRV(d.MemSetAccess(b->va[q], b->size, &acc, 1), b);
  }
  // 4. multicast object: created by rank 0, every device added, then every rank binds its block and maps the object
  if (use_mc) {
    CUdevice dev;
    TB_DRV(d.DeviceGet(&dev, h.device), b);
    if (h.rank == 0) {
      TB_DRV(d.MulticastCreate(&b->mc, &mprop), b);
      b->have_mc = true;
      int mfd = -1;
      TB_DRV(d.MemExportToShareableHandle(&mfd, b->mc, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0), b);
      for (int q = 1; q < h.world && !rc; ++q) rc = send_msg(h, q, 2, mfd);
      close(mfd);
    } else {
      int mfd = -1;
      rc = recv_msg(h, 0, 2, &mfd);
      if (!rc && mfd < 0) rc = TB_E_CUDA;
      if (!rc) {
        CUresult r = d.MemImportFromShareableHandle(&b->mc, (void*)(uintptr_t)mfd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
        close(mfd);
        if (r != CUDA_SUCCESS) {
          rc = TB_E_CUDA;
          snprintf(tb::last_error_buf(), 512, "symmetric heap: import of the multicast object failed with CUresult %d", (int)r);
        } else {
          b->have_mc = true;
        }
      }
    }
    if (rc) {
      destroy(b);
      return rc;
    }
    TB_DRV(d.MulticastAddDevice(b->mc, dev), b);
    if ((rc = barrier(h, 3))) {  // memory may be bound only after every device has been added
      destroy(b);
      return rc;
    }
    TB_DRV(d.MulticastBindMem(b->mc, 0, b->mem[h.rank], 0, b->size, 0), b);
    b->mc_bound = true;
    TB_DRV(d.MemAddressReserve(&b->mc_va, b->size, gran, 0, 0), b);
    TB_DRV(d.MemMap(b->mc_va, b->size, 0, b->mc, 0), b);
    b->mc_mapped = true;
    TB_DRV(d.MemSetAccess(b->mc_va, b->size, &acc, 1), b);
  }
  // 5. nobody touches a peer's block before everyone has mapped (and bound) theirs
  if ((rc = barrier(h, 4))) {
    destroy(b);
    return rc;
  }
  TB_CUDA_CHECK(cudaMemset((void*)b->va[h.rank], 0, b->size));
  TB_CUDA_CHECK(cudaDeviceSynchronize());
  if ((rc = barrier(h, 5))) {
    destroy(b);
    return rc;
  }
  for (int q = 0; q < h.world; ++q) peer_ptrs[q] = (void*)b->va[q];
  if (mc_ptr) *mc_ptr = (void*)b->mc_va;
  if (mapped_bytes) *mapped_bytes = b->size;
  *handle = b;
  return 0;
}

// Collective release: every rank waits for the others to stop using the block (barrier), then unmaps, unbinds and
// releases its handles.
TB_EXPORT int tb_symm_free(void* handle) {
  TB_ENSURE_DEVICE();
  if (!handle) return 0;
  Heap& h = g_heaps[((SymmBlock*)handle)->heap];
  std::lock_guard<std::mutex> lk(h.mu);
  TB_CUDA_CHECK(cudaDeviceSynchronize());
  h.seq += 1;
  int rc = h.sock >= 0 ? barrier(h, 9) : 0;
  destroy((SymmBlock*)handle);
  return rc;
}

// Closes a heap's socket (blocks that are still allocated stay mapped until tb_symm_free; free then skips its barrier).
TB_EXPORT int tb_symm_shutdown(int heap) {
  if (heap < 0 || heap >= SYMM_MAX_HEAPS) return 0;
  std::lock_guard<std::mutex> all(g_heaps_mu);
  Heap& h = g_heaps[heap];
  std::lock_guard<std::mutex> lk(h.mu);
  if (h.sock >= 0) close(h.sock);
  h.sock = -1;
  for (auto& p : h.pending)
    if (p.second >= 0) close(p.second);
  h.pending.clear();
  return 0;
}
