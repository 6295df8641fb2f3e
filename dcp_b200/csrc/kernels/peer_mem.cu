// Peer-mapped device memory through CUDA IPC handles: the second allocation route of the symmetric
// arena, for builds of the framework's library without a symmetric-memory module.  Every rank
// allocates one buffer, exports its 64-byte handle (exchanged on the host through the process
// group) and maps every peer's buffer; the mapping enables NVLink peer access lazily.  Plain
// loads, stores and reductions into the mapped range are what the kernels use; nothing here
// launches a kernel.  Role in the reference: its peers exchange blocks through NCCL all-to-all
// buffers (dcp/runtime/flash_attention/executor.py:1975-1986); here peers address each other's
// memory directly.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>

extern "C" {

// allocates `nbytes` of device memory on the current device, zero-filled; writes the device
// address to *ptr and the 64-byte IPC handle to `handle`.  0 on success, -5 on a CUDA error.
int dcpk_ipc_alloc(size_t nbytes, void** ptr, void* handle) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  cudaError_t e = cudaMalloc(ptr, nbytes);
  if (e == cudaSuccess) e = cudaMemset(*ptr, 0, nbytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();  // zeros are in place before any peer can see the handle
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, *ptr);
  if (e != cudaSuccess) {
    fprintf(stderr, "dcpk_ipc_alloc: %s\n", cudaGetErrorString(e));
    return -5;
  }
  memcpy(handle, &h, sizeof(h));
  return 0;
}

// maps a peer's buffer (handle from dcpk_ipc_alloc in another process) into this process
int dcpk_ipc_open(const void* handle, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  cudaError_t e = cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    fprintf(stderr, "dcpk_ipc_open: %s\n", cudaGetErrorString(e));
    return -5;
  }
  return 0;
}

int dcpk_ipc_close(void* ptr) { return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? 0 : -5; }

int dcpk_ipc_free(void* ptr) { return cudaFree(ptr) == cudaSuccess ? 0 : -5; }

}  // extern "C"
