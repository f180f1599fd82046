// Symmetric heap runtime, fallback back-end (the primary one is vmm_heap.cu): one device
// allocation per rank, exported with CUDA IPC and mapped by every other rank of the node, so that kernels can address
// any rank's copy of a buffer as base[rank] + offset and reach it with plain
// loads/stores over NVLink.  Plays the role the external `iris` library plays
// for the reference project (benchmark.py:38-42, utils.py:48-80: a fixed-size
// heap, identical offsets on all ranks, a table of per-rank heap bases).
//
// The exchange of the 64-byte IPC handles between processes is done by the
// caller (torch.distributed all_gather); this file only creates, exports,
// opens and closes.
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include <atomic>

#include "moe_args.h"

static std::atomic<long long> g_launches{0};

extern "C" {

// Allocates `bytes` of device memory on `device`, zero-filled.
int b200_heap_create(int device, unsigned long long bytes, void** base) {
  cudaError_t e = cudaSetDevice(device);
  if (e != cudaSuccess) return static_cast<int>(e);
  e = cudaMalloc(base, bytes);
  if (e != cudaSuccess) return static_cast<int>(e);
  e = cudaMemset(*base, 0, bytes);
  if (e != cudaSuccess) return static_cast<int>(e);
  return static_cast<int>(cudaDeviceSynchronize());
}

int b200_heap_destroy(int device, void* base) {
  cudaError_t e = cudaSetDevice(device);
  if (e != cudaSuccess) return static_cast<int>(e);
  return static_cast<int>(cudaFree(base));
}

int b200_heap_handle_bytes() { return static_cast<int>(sizeof(cudaIpcMemHandle_t)); }

int b200_heap_export(int device, void* base, unsigned char* handle_out) {
  cudaError_t e = cudaSetDevice(device);
  if (e != cudaSuccess) return static_cast<int>(e);
  cudaIpcMemHandle_t h;
  e = cudaIpcGetMemHandle(&h, base);
  if (e != cudaSuccess) return static_cast<int>(e);
  memcpy(handle_out, &h, sizeof(h));
  return 0;
}

// Maps a peer's heap into this process; peer access is enabled lazily.
int b200_heap_open(int device, const unsigned char* handle, void** mapped) {
  cudaError_t e = cudaSetDevice(device);
  if (e != cudaSuccess) return static_cast<int>(e);
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  return static_cast<int>(cudaIpcOpenMemHandle(mapped, h, cudaIpcMemLazyEnablePeerAccess));
}

int b200_heap_close(int device, void* mapped) {
  cudaError_t e = cudaSetDevice(device);
  if (e != cudaSuccess) return static_cast<int>(e);
  return static_cast<int>(cudaIpcCloseMemHandle(mapped));
}

int b200_memset_async(void* ptr, int value, unsigned long long bytes, void* stream) {
  return static_cast<int>(cudaMemsetAsync(ptr, value, bytes, static_cast<cudaStream_t>(stream)));
}

// One device-to-device copy; either address may be a peer's mapped memory.
int b200_memcpy_async(void* dst, const void* src, unsigned long long bytes, void* stream) {
  return static_cast<int>(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice,
                                          static_cast<cudaStream_t>(stream)));
}

void b200_count_launches(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
long long b200_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

const char* b200_error_string(int code) {
  return cudaGetErrorString(static_cast<cudaError_t>(code));
}

}  // extern "C"
