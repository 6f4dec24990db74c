// Symmetric memory for one-process-per-GPU jobs on an NVSwitch node: every rank allocates the same
// buffers with cudaMalloc, exports them as CUDA IPC handles, and maps every peer's buffer, so
// kernels address peers with plain loads and stores over NVLink. Exchange of the 64-byte handles
// goes over the host control plane (torch.distributed object collectives).
//
// This replaces the transport zoo the reference composes for tensors that cross processes (NCCL
// p2p groups, UCX, Gloo, CUDA-IPC via pickled storages, TCP, files:
// RPEG/runtime/semantic_worker.py:9840-10028, 11281-12496).
#include "common.cuh"
#include "rpeg_kernels.h"
#include <string.h>

extern "C" int rpeg_symm_alloc(unsigned long long bytes, void** out) {
  if (out == nullptr || bytes == 0) return -2;
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) {
    cudaGetLastError();
    return -40;
  }
  *out = p;
  return 0;
}

extern "C" int rpeg_symm_free(void* p) { return cudaFree(p) == cudaSuccess ? 0 : -41; }

// handle: 64 bytes (cudaIpcMemHandle_t)
extern "C" int rpeg_ipc_export(void* p, void* handle64) {
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) {
    cudaGetLastError();
    return -42;
  }
  memcpy(handle64, &h, sizeof(h));
  return 0;
}

extern "C" int rpeg_ipc_open(const void* handle64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  void* p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
    cudaGetLastError();
    return -43;
  }
  *out = p;
  return 0;
}

extern "C" int rpeg_ipc_close(void* p) { return cudaIpcCloseMemHandle(p) == cudaSuccess ? 0 : -44; }

extern "C" int rpeg_memset_async(void* p, int value, unsigned long long bytes, void* stream) {
  return cudaMemsetAsync(p, value, bytes, reinterpret_cast<cudaStream_t>(stream)) == cudaSuccess ? 0 : -45;
}
