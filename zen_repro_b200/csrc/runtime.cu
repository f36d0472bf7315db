// Host-side runtime helpers with a C ABI: symmetric (peer-visible) memory through CUDA IPC, peer
// access set-up, and small device utilities.  One process per GPU; handles travel through the
// process group's store on the Python side.
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

extern "C" {

// Allocate `bytes` of device memory directly from the driver pool (not from a caching allocator, so
// that the IPC handle covers exactly this allocation) and zero it.
int zen_sym_alloc(void** out, uint64_t bytes) {
  cudaError_t e = cudaMalloc(out, bytes);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaMemset(*out, 0, bytes);
}

int zen_sym_free(void* p) { return (int)cudaFree(p); }

// 64-byte IPC handle of an allocation made by zen_sym_alloc.
int zen_ipc_get_handle(void* p, unsigned char* handle64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) return (int)e;
  memcpy(handle64, &h, sizeof(h));
  return 0;
}

int zen_ipc_open(const unsigned char* handle64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  return (int)cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess);
}

int zen_ipc_close(void* p) { return (int)cudaIpcCloseMemHandle(p); }

// Enable peer access from the current device to `peer` (already-enabled is not an error).
int zen_enable_peer(int peer) {
  int dev = 0;
  cudaGetDevice(&dev);
  if (peer == dev) return 0;
  int can = 0;
  cudaError_t e = cudaDeviceCanAccessPeer(&can, dev, peer);
  if (e != cudaSuccess) return (int)e;
  if (!can) return -2;
  e = cudaDeviceEnablePeerAccess(peer, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    cudaGetLastError();
    return 0;
  }
  return (int)e;
}

int zen_ipc_handle_size() { return (int)sizeof(cudaIpcMemHandle_t); }

}  // extern "C"
