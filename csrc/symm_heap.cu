// Symmetric heap: one device allocation per rank, mapped into every other rank's address space.
//
// The role NVSHMEM's symmetric heap plays in the reference (maco/csrc/nvshmem_ops.cu:37-147:
// MPI bootstrap + nvshmem_malloc). Here the heap is a plain cudaMalloc block exported with a CUDA
// IPC handle; the handles travel through the torch.distributed store that the process group
// already owns (Python side), and each rank opens its peers' blocks with peer access enabled, so
// kernels can ld/st/red another GPU's memory over NVLink with ordinary instructions.
// No NVSHMEM, no MPI.
#include "host_common.h"
#include <string.h>

extern "C" {

// Allocates `bytes` of device memory, zeroes it and writes the 64-byte IPC handle.
int maco_heap_create(unsigned long long bytes, void** base_out, void* handle_out64) {
  void* p = nullptr;
  MACO_CHECK_CUDA(cudaMalloc(&p, bytes));
  MACO_CHECK_CUDA(cudaMemset(p, 0, bytes));
  cudaIpcMemHandle_t h;
  MACO_CHECK_CUDA(cudaIpcGetMemHandle(&h, p));
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle is 64 bytes");
  memcpy(handle_out64, &h, 64);
  MACO_CHECK_CUDA(cudaDeviceSynchronize());
  *base_out = p;
  return 0;
}

// Maps a peer's heap into this process. Peer access between the two devices is enabled lazily.
int maco_heap_open(const void* handle64, void** peer_base_out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* p = nullptr;
  MACO_CHECK_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  *peer_base_out = p;
  return 0;
}

int maco_heap_close(void* peer_base) {
  MACO_CHECK_CUDA(cudaIpcCloseMemHandle(peer_base));
  return 0;
}

int maco_heap_destroy(void* base) {
  MACO_CHECK_CUDA(cudaFree(base));
  return 0;
}

}  // extern "C"
