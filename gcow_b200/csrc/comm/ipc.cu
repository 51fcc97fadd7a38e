// Peer mapping of a device buffer between the processes of one node with CUDA
// IPC handles: allocate, export a 64-byte handle, open the peers' handles.
// This is the plain fallback for the symmetric arena when no multicast-capable
// allocator is available; the handles travel over the job's host-side process
// group. All functions return a CUDA error code (0 = success).
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

extern "C" {

int gcow_ipc_alloc(uint64_t bytes, void** ptr) {
  cudaError_t e = cudaMalloc(ptr, bytes);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaMemset(*ptr, 0, bytes);
}

int gcow_ipc_free(void* ptr) { return (int)cudaFree(ptr); }

int gcow_ipc_export(void* ptr, void* handle64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
  if (e != cudaSuccess) return (int)e;
  static_assert(sizeof(h) == 64, "CUDA IPC handles are 64 bytes");
  memcpy(handle64, &h, 64);
  return 0;
}

int gcow_ipc_open(const void* handle64, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  return (int)cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
}

int gcow_ipc_close(void* ptr) { return (int)cudaIpcCloseMemHandle(ptr); }

int gcow_device_sync() { return (int)cudaDeviceSynchronize(); }

}  // extern "C"
