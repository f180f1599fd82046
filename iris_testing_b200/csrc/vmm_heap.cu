// Symmetric heap on the CUDA virtual-memory-management API.
//
// Every rank reserves ONE virtual-address window of world * slot_bytes and maps into slot r
// the physical memory of rank r: its own chunks directly, the peers' chunks after importing
// the POSIX file descriptors the peers exported.  Kernels then reach rank r's copy of a
// symmetric buffer at window + r * slot_bytes + offset with plain loads and stores over
// NVLink.  A heap can GROW: every rank adds a chunk at the same offset (a collective call),
// and the window was reserved for the final size up front, so addresses never move.
//
// The descriptors travel between the processes of one node over Unix datagram sockets in
// the abstract namespace (SCM_RIGHTS), one socket per rank, no helper thread: a grow sends
// this rank's descriptor to every peer and then receives one from every peer.  Receives have
// a time limit, so a missing peer yields an error code, not a hang.
//
// Plays the role the external `iris` library plays for the reference project
// (benchmark.py:38-42, utils.py:48-80: a fixed-size heap, identical offsets on all ranks, a
// table of per-rank heap bases); the CUDA-IPC heap of symm_heap.cu is the fallback where
// this API or descriptor export is not available.
//
// Driver entry points are resolved at run time (cudaGetDriverEntryPoint), so the library
// links against the runtime only and loads on machines without a driver.
#include <cuda.h>
#include <cuda_runtime.h>
#include <errno.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/time.h>
#include <sys/un.h>
#include <unistd.h>

#include <string>
#include <vector>

#include "moe_args.h"

namespace {

struct Driver {
  CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
  CUresult (*MemRelease)(CUmemGenericAllocationHandle);
  CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
  CUresult (*MemAddressFree)(CUdeviceptr, size_t);
  CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
  CUresult (*MemUnmap)(CUdeviceptr, size_t);
  CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
  CUresult (*MemExport)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long);
  CUresult (*MemImport)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType);
  CUresult (*MemGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
  CUresult (*DeviceGetAttribute)(int*, CUdevice_attribute, CUdevice);
  bool ok;
};

template <typename F>
bool resolve(const char* name, F& fn) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess || p == nullptr) {
    (void)cudaGetLastError();
    return false;
  }
  fn = reinterpret_cast<F>(p);
  return true;
}

Driver& driver() {
  static Driver d = [] {
    Driver x;
    memset(&x, 0, sizeof(x));
    x.ok = resolve("cuMemCreate", x.MemCreate) && resolve("cuMemRelease", x.MemRelease) &&
           resolve("cuMemAddressReserve", x.MemAddressReserve) &&
           resolve("cuMemAddressFree", x.MemAddressFree) && resolve("cuMemMap", x.MemMap) &&
           resolve("cuMemUnmap", x.MemUnmap) && resolve("cuMemSetAccess", x.MemSetAccess) &&
           resolve("cuMemExportToShareableHandle", x.MemExport) &&
           resolve("cuMemImportFromShareableHandle", x.MemImport) &&
           resolve("cuMemGetAllocationGranularity", x.MemGranularity) &&
           resolve("cuDeviceGetAttribute", x.DeviceGetAttribute);
    return x;
  }();
  return d;
}

struct Chunk {
  CUmemGenericAllocationHandle handle;
  size_t offset;   // inside the rank's slot
  size_t bytes;
};

struct VmmHeap {
  int device, world, rank;
  size_t slot_bytes, gran, mapped;   // `mapped`: bytes mapped in every slot (same on all ranks)
  CUdeviceptr window;
  std::vector<std::vector<Chunk>> chunks;   // [rank]
  int sock;
  std::string prefix;
  unsigned generation;
};

// error codes (negative; positive values are CUresult / errno as documented per call)
enum { E_NO_DRIVER = -30, E_UNSUPPORTED = -31, E_ARG = -32, E_SOCKET = -33, E_TIMEOUT = -34,
       E_PROTOCOL = -35, E_FULL = -36 };

struct Message {
  uint32_t magic, generation;
  int32_t rank;
  uint64_t bytes;
};
constexpr uint32_t MAGIC = 0xB2005EA9u;

CUmemAllocationProp alloc_prop(int device) {
  CUmemAllocationProp p;
  memset(&p, 0, sizeof(p));
  p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  p.location.id = device;
  p.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return p;
}

void fill_addr(sockaddr_un& a, socklen_t& len, const std::string& prefix, int rank) {
  memset(&a, 0, sizeof(a));
  a.sun_family = AF_UNIX;
  const std::string name = prefix + "." + std::to_string(rank);
  // abstract namespace: leading NUL byte, no file is created
  const size_t n = name.size() < sizeof(a.sun_path) - 1 ? name.size() : sizeof(a.sun_path) - 1;
  memcpy(a.sun_path + 1, name.data(), n);
  len = static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + 1 + n);
}

int send_fd(int sock, const std::string& prefix, int my_rank, unsigned generation, int peer, int fd,
            uint64_t bytes) {
  sockaddr_un a;
  socklen_t alen;
  fill_addr(a, alen, prefix, peer);
  Message m = {MAGIC, generation, my_rank, bytes};
  iovec iov = {&m, sizeof(m)};
  alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
  memset(ctrl, 0, sizeof(ctrl));
  msghdr msg;
  memset(&msg, 0, sizeof(msg));
  msg.msg_name = &a;
  msg.msg_namelen = alen;
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  cmsghdr* c = CMSG_FIRSTHDR(&msg);
  c->cmsg_level = SOL_SOCKET;
  c->cmsg_type = SCM_RIGHTS;
  c->cmsg_len = CMSG_LEN(sizeof(int));
  memcpy(CMSG_DATA(c), &fd, sizeof(int));
  for (int attempt = 0; attempt < 200; ++attempt) {
    if (sendmsg(sock, &msg, 0) == static_cast<ssize_t>(sizeof(m))) return 0;
    // the peer's socket may not be bound yet, or its queue is full: retry for a while
    if (errno != ECONNREFUSED && errno != ENOENT && errno != EAGAIN && errno != ENOBUFS) break;
    usleep(50 * 1000);
  }
  return E_SOCKET;
}

int recv_fd(int sock, Message* m, int* fd) {
  iovec iov = {m, sizeof(*m)};
  alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
  msghdr msg;
  memset(&msg, 0, sizeof(msg));
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  const ssize_t n = recvmsg(sock, &msg, 0);
  if (n < 0) return (errno == EAGAIN || errno == EWOULDBLOCK) ? E_TIMEOUT : E_SOCKET;
  if (n != static_cast<ssize_t>(sizeof(*m)) || m->magic != MAGIC) return E_PROTOCOL;
  *fd = -1;
  for (cmsghdr* c = CMSG_FIRSTHDR(&msg); c != nullptr; c = CMSG_NXTHDR(&msg, c))
    if (c->cmsg_level == SOL_SOCKET && c->cmsg_type == SCM_RIGHTS) memcpy(fd, CMSG_DATA(c), sizeof(int));
  return *fd >= 0 ? 0 : E_PROTOCOL;
}

int open_socket(const std::string& prefix, int rank, int recv_timeout_ms) {
  const int sock = socket(AF_UNIX, SOCK_DGRAM | SOCK_CLOEXEC, 0);
  if (sock < 0) return -1;
  sockaddr_un a;
  socklen_t alen;
  fill_addr(a, alen, prefix, rank);
  timeval tv = {recv_timeout_ms / 1000, (recv_timeout_ms % 1000) * 1000};
  if (bind(sock, reinterpret_cast<sockaddr*>(&a), alen) != 0 ||
      setsockopt(sock, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv)) != 0) {
    close(sock);
    return -1;
  }
  return sock;
}

int map_chunk(VmmHeap* h, int slot, CUmemGenericAllocationHandle handle, size_t offset, size_t bytes) {
  Driver& d = driver();
  const CUdeviceptr at = h->window + static_cast<size_t>(slot) * h->slot_bytes + offset;
  CUresult r = d.MemMap(at, bytes, 0, handle, 0);
  if (r != CUDA_SUCCESS) return static_cast<int>(r);
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = h->device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  r = d.MemSetAccess(at, bytes, &acc, 1);
  if (r != CUDA_SUCCESS) {
    d.MemUnmap(at, bytes);
    return static_cast<int>(r);
  }
  h->chunks[slot].push_back(Chunk{handle, offset, bytes});
  return 0;
}

}  // namespace

extern "C" {

// out[0]: virtual memory management supported, out[1]: POSIX descriptor export supported,
// out[2]: NVLink multicast objects (NVLS, multimem.*) supported, out[3]: allocation
// granularity in bytes.  Queries only; changes nothing.
int b200_vmm_probe(int device, long long* out) {
  out[0] = out[1] = out[2] = out[3] = 0;
  if (cudaSetDevice(device) != cudaSuccess || cudaFree(nullptr) != cudaSuccess) {
    (void)cudaGetLastError();
    return E_UNSUPPORTED;
  }
  Driver& d = driver();
  if (!d.ok) return E_NO_DRIVER;
  int v = 0;
  if (d.DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_VIRTUAL_MEMORY_MANAGEMENT_SUPPORTED, device) == CUDA_SUCCESS)
    out[0] = v;
  if (d.DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, device) == CUDA_SUCCESS)
    out[1] = v;
  if (d.DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, device) == CUDA_SUCCESS)
    out[2] = v;
  CUmemAllocationProp p = alloc_prop(device);
  size_t g = 0;
  if (d.MemGranularity(&g, &p, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS)
    out[3] = static_cast<long long>(g);
  return 0;
}

// Reserves the window (world * slot_bytes of address space, no memory yet) and binds this
// rank's socket "<prefix>.<rank>".  slot_bytes is rounded up to the granularity.
int b200_vmm_create(int device, int world, int rank, unsigned long long slot_bytes, const char* prefix,
                    int recv_timeout_ms, void** out) {
  if (world < 1 || world > B200_MAX_WORLD || rank < 0 || rank >= world || slot_bytes == 0 ||
      out == nullptr || prefix == nullptr)
    return E_ARG;
  long long caps[4];
  int r = b200_vmm_probe(device, caps);
  if (r != 0) return r;
  if (!caps[0] || (world > 1 && !caps[1]) || caps[3] <= 0) return E_UNSUPPORTED;
  VmmHeap* h = new VmmHeap();
  h->device = device;
  h->world = world;
  h->rank = rank;
  h->gran = static_cast<size_t>(caps[3]);
  h->slot_bytes = (static_cast<size_t>(slot_bytes) + h->gran - 1) / h->gran * h->gran;
  h->mapped = 0;
  h->window = 0;
  h->chunks.resize(world);
  h->sock = -1;
  h->prefix = prefix;
  h->generation = 0;
  CUresult cr = driver().MemAddressReserve(&h->window, h->slot_bytes * world, h->gran, 0, 0);
  if (cr != CUDA_SUCCESS) {
    delete h;
    return static_cast<int>(cr);
  }
  if (world > 1) {
    h->sock = open_socket(h->prefix, rank, recv_timeout_ms);
    if (h->sock < 0) {
      driver().MemAddressFree(h->window, h->slot_bytes * world);
      delete h;
      return E_SOCKET;
    }
  }
  *out = h;
  return 0;
}

// Collective: every rank adds `bytes` (rounded up to the granularity; returned through
// bytes_out) of zero-filled memory at the end of its slot and maps every peer's new chunk.
// All ranks must have created their heap (sockets bound) before the first call, and must
// make the same sequence of calls.
int b200_vmm_grow(void* heap, unsigned long long bytes, unsigned long long* bytes_out) {
  VmmHeap* h = static_cast<VmmHeap*>(heap);
  if (h == nullptr || bytes == 0) return E_ARG;
  Driver& d = driver();
  if (cudaSetDevice(h->device) != cudaSuccess) return E_UNSUPPORTED;
  const size_t sz = (static_cast<size_t>(bytes) + h->gran - 1) / h->gran * h->gran;
  if (h->mapped + sz > h->slot_bytes) return E_FULL;
  CUmemAllocationProp p = alloc_prop(h->device);
  CUmemGenericAllocationHandle mine;
  CUresult cr = d.MemCreate(&mine, sz, &p, 0);
  if (cr != CUDA_SUCCESS) return static_cast<int>(cr);
  int r = map_chunk(h, h->rank, mine, h->mapped, sz);
  if (r != 0) {
    d.MemRelease(mine);
    return r;
  }
  void* local = reinterpret_cast<void*>(h->window + static_cast<size_t>(h->rank) * h->slot_bytes + h->mapped);
  if (cudaMemset(local, 0, sz) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) return E_UNSUPPORTED;
  ++h->generation;
  if (h->world > 1) {
    int fd = -1;
    cr = d.MemExport(&fd, mine, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
    if (cr != CUDA_SUCCESS) return static_cast<int>(cr);
    for (int s = 1; s < h->world; ++s) {
      r = send_fd(h->sock, h->prefix, h->rank, h->generation, (h->rank + s) % h->world, fd, sz);
      if (r != 0) {
        close(fd);
        return r;
      }
    }
    close(fd);
    std::vector<char> seen(h->world, 0);
    for (int got = 0; got < h->world - 1; ++got) {
      Message m;
      int pfd = -1;
      r = recv_fd(h->sock, &m, &pfd);
      if (r != 0) return r;
      const bool fine = m.generation == h->generation && m.rank >= 0 && m.rank < h->world &&
                        m.rank != h->rank && !seen[m.rank] && m.bytes == sz;
      if (!fine) {
        close(pfd);
        return E_PROTOCOL;
      }
      seen[m.rank] = 1;
      CUmemGenericAllocationHandle ph;
      cr = d.MemImport(&ph, reinterpret_cast<void*>(static_cast<intptr_t>(pfd)),
                       CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
      close(pfd);
      if (cr != CUDA_SUCCESS) return static_cast<int>(cr);
      r = map_chunk(h, m.rank, ph, h->mapped, sz);
      if (r != 0) {
        d.MemRelease(ph);
        return r;
      }
    }
  }
  h->mapped += sz;
  if (bytes_out != nullptr) *bytes_out = sz;
  return 0;
}

unsigned long long b200_vmm_base(void* heap, int rank) {
  VmmHeap* h = static_cast<VmmHeap*>(heap);
  if (h == nullptr || rank < 0 || rank >= h->world) return 0;
  return static_cast<unsigned long long>(h->window) + static_cast<unsigned long long>(rank) * h->slot_bytes;
}

unsigned long long b200_vmm_mapped_bytes(void* heap) {
  return heap ? static_cast<unsigned long long>(static_cast<VmmHeap*>(heap)->mapped) : 0ull;
}

unsigned long long b200_vmm_slot_bytes(void* heap) {
  return heap ? static_cast<unsigned long long>(static_cast<VmmHeap*>(heap)->slot_bytes) : 0ull;
}

// Unmaps every chunk, releases the handles (the owning rank's release frees the memory once
// every importer has released too), frees the window and closes the socket.
int b200_vmm_destroy(void* heap) {
  VmmHeap* h = static_cast<VmmHeap*>(heap);
  if (h == nullptr) return E_ARG;
  Driver& d = driver();
  cudaSetDevice(h->device);
  cudaDeviceSynchronize();
  int first_err = 0;
  for (int r = 0; r < h->world; ++r) {
    for (const Chunk& c : h->chunks[r]) {
      const CUdeviceptr at = h->window + static_cast<size_t>(r) * h->slot_bytes + c.offset;
      CUresult e1 = d.MemUnmap(at, c.bytes);
      CUresult e2 = d.MemRelease(c.handle);
      if (first_err == 0 && e1 != CUDA_SUCCESS) first_err = static_cast<int>(e1);
      if (first_err == 0 && e2 != CUDA_SUCCESS) first_err = static_cast<int>(e2);
    }
  }
  CUresult e3 = d.MemAddressFree(h->window, h->slot_bytes * h->world);
  if (first_err == 0 && e3 != CUDA_SUCCESS) first_err = static_cast<int>(e3);
  if (h->sock >= 0) close(h->sock);
  delete h;
  return first_err;
}

// ---------------------------------------------------------------------------
// The descriptor channel on its own (what b200_vmm_grow uses), exported so that it can be
// exercised between CPU processes with any file descriptor.
// ---------------------------------------------------------------------------
struct FdChannel {
  int sock, rank;
  std::string prefix;
};

int b200_fdchan_open(const char* prefix, int rank, int recv_timeout_ms, void** out) {
  if (prefix == nullptr || out == nullptr || rank < 0) return E_ARG;
  const int sock = open_socket(prefix, rank, recv_timeout_ms);
  if (sock < 0) return E_SOCKET;
  *out = new FdChannel{sock, rank, prefix};
  return 0;
}

int b200_fdchan_send(void* chan, int peer, int fd, unsigned generation, unsigned long long bytes) {
  FdChannel* c = static_cast<FdChannel*>(chan);
  if (c == nullptr || fd < 0) return E_ARG;
  return send_fd(c->sock, c->prefix, c->rank, generation, peer, fd, bytes);
}

// Receives one descriptor (owned by the caller afterwards).  E_TIMEOUT (-34) when nothing
// arrived within the channel's time limit.
int b200_fdchan_recv(void* chan, int* from_rank, int* fd, unsigned* generation, unsigned long long* bytes) {
  FdChannel* c = static_cast<FdChannel*>(chan);
  if (c == nullptr) return E_ARG;
  Message m;
  const int r = recv_fd(c->sock, &m, fd);
  if (r != 0) return r;
  if (from_rank) *from_rank = m.rank;
  if (generation) *generation = m.generation;
  if (bytes) *bytes = m.bytes;
  return 0;
}

int b200_fdchan_close(void* chan) {
  FdChannel* c = static_cast<FdChannel*>(chan);
  if (c == nullptr) return E_ARG;
  close(c->sock);
  delete c;
  return 0;
}

}  // extern "C"
