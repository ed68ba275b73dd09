// Allocation and inter-process mapping of symmetric buffers (one process per GPU, all
// GPUs of a node).  A buffer is a plain cudaMalloc allocation whose CUDA IPC handle is
// exchanged through the host-side communicator; opening a peer's handle maps that GPU's
// memory into this process with peer access enabled, after which the collective kernels
// reach it with ordinary loads and stores over NVLink.  This is the role the reference
// delegates to its "p2p" CUDA-IPC library and to NVSHMEM (src/utils/distconv.cpp:45,301,
// src/utils/nvshmem.cu:43-71).
#include "common.cuh"
#include <cstdio>
#include <cstring>

extern "C" {

// Returns a zero-filled device allocation (nullptr on failure).
void* lb_symm_alloc(long long bytes) {
  void* p = nullptr;
  if (cudaMalloc(&p, (size_t)bytes) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  cudaMemset(p, 0, (size_t)bytes);
  cudaDeviceSynchronize();
  return p;
}

int lb_symm_free(void* p) { return (int)cudaFree(p); }

int lb_ipc_handle_bytes() { return (int)sizeof(cudaIpcMemHandle_t); }

// out must hold lb_ipc_handle_bytes() bytes.
int lb_ipc_get_handle(void* p, void* out) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return (int)e;
  }
  memcpy(out, &h, sizeof(h));
  return 0;
}

// Maps a peer's allocation; returns the local address (nullptr on failure).
void* lb_ipc_open(const void* handle) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    fprintf(stderr, "[lbann_b200] cudaIpcOpenMemHandle failed: %s\n", cudaGetErrorString(e));
    cudaGetLastError();
    return nullptr;
  }
  return p;
}

int lb_ipc_close(void* p) { return (int)cudaIpcCloseMemHandle(p); }

}  // extern "C"
