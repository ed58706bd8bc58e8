// Host-side helpers shared by the translation units of libmaco_b200: error reporting,
// driver entry points fetched at run time (so the library loads on a machine without a GPU
// driver), tensor-map encoding and the host-mapped status block kernels report into.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string>
#include "maco_types.h"

namespace maco_host {

void set_error(const std::string& msg);
const char* last_error();

#define MACO_CHECK_CUDA(expr)                                                              \
  do {                                                                                     \
    cudaError_t _e = (expr);                                                               \
    if (_e != cudaSuccess) {                                                               \
      maco_host::set_error(std::string(#expr) + ": " + cudaGetErrorString(_e));            \
      return -1;                                                                           \
    }                                                                                      \
  } while (0)

// Encodes a 2-D tiled tensor map over a row-major [rows, cols] tensor of 16-bit elements with a
// 128-byte swizzle. box = (box_cols, box_rows). Returns 0 on success.
int encode_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t rows, uint64_t cols,
                   uint64_t row_stride_bytes, uint32_t box_cols, uint32_t box_rows);

// Device pointer of the per-process status block (host-mapped, zero-copy) and its host view.
uint32_t* status_device_ptr();
MacoStatusBlock* status_host_ptr();

int sm_count();

}  // namespace maco_host
