// Stand-alone split-KV decode attention: one CTA per (batch, kv-head, split) runs the same task body
// the persistent kernel uses (attention_decode.cuh), a second launch merges the splits.
//
// Layouts (row-major, 16-bit):
//   q   [B, Hq, 128]          Hq = Hkv * G query heads, the G heads of one KV head are adjacent
//   k,v [B, Hkv, S, 128]      S = keys per sequence (cache length)
//   out [B, Hq, 128]
//   scratch fp32 [B * Hkv * splits, G*128 + 2G]   unnormalised partial outputs, running max and sum
#include "attention_decode.cuh"
#include "host_common.h"

using namespace maco;

namespace {

struct AttnParams {
  const void* q; const void* k; const void* v; void* out; float* scratch;
  int B, Hkv, G, S, splits, dtype;
  long long kv_batch_stride, kv_head_stride;   // in elements
  float scale;
};

__global__ void __launch_bounds__(128) attn_decode_kernel(AttnParams p) {
  __shared__ __align__(16) uint8_t scratch_smem[kAttnScratchBytes];
  const int split = blockIdx.x % p.splits;
  const int bh = blockIdx.x / p.splits;            // b * Hkv + kvh
  const int b = bh / p.Hkv, kvh = bh % p.Hkv;
  const int per = (p.S + p.splits - 1) / p.splits;
  const int s0 = split * per;
  int rows = p.S - s0;
  if (rows > per) rows = per;
  if (rows < 0) rows = 0;
  const int rec = p.G * kAttnD + 2 * p.G;
  MacoEltArgs a;
  const size_t esz = 2;
  a.in0 = reinterpret_cast<const uint8_t*>(p.q) + ((size_t)(b * p.Hkv + kvh) * p.G * kAttnD) * esz;
  const size_t kv_off = ((size_t)b * p.kv_batch_stride + (size_t)kvh * p.kv_head_stride + (size_t)s0 * kAttnD) * esz;
  a.in1 = reinterpret_cast<const uint8_t*>(p.k) + kv_off;
  a.in2 = reinterpret_cast<const uint8_t*>(p.v) + kv_off;
  a.out = p.scratch + (size_t)blockIdx.x * rec;
  a.row0 = 0; a.rows = rows; a.cols = kAttnD; a.dtype = p.dtype; a.ld_in = kAttnD; a.ld_out = 0;
  a.f0 = p.scale; a.f1 = 0.f; a.i0 = p.G; a.i1 = 0;
  attn_decode_task(a, threadIdx.x, scratch_smem);
}

__global__ void __launch_bounds__(128) attn_merge_kernel(AttnParams p) {
  const int bh = blockIdx.x;
  const int rec = p.G * kAttnD + 2 * p.G;
  MacoEltArgs a;
  a.in0 = p.scratch + (size_t)bh * p.splits * rec;
  a.in1 = nullptr; a.in2 = nullptr;
  a.out = reinterpret_cast<uint8_t*>(p.out) + (size_t)bh * p.G * kAttnD * 2;
  a.row0 = 0; a.rows = 0; a.cols = kAttnD; a.dtype = p.dtype; a.ld_in = 0; a.ld_out = 0;
  a.f0 = 0.f; a.f1 = 0.f; a.i0 = p.G; a.i1 = p.splits;
  attn_merge_task(a, threadIdx.x);
}

int check_and_fill(AttnParams& p, const void* q, const void* k, const void* v, void* out, float* scratch, int B,
                   int Hq, int Hkv, int S, int head_dim, int splits, int dtype, long long kv_batch_stride,
                   long long kv_head_stride, float scale) {
  if (head_dim != kAttnD) { maco_host::set_error("attention_decode: head_dim must be 128"); return -1; }
  if (Hkv <= 0 || Hq % Hkv != 0 || Hq / Hkv > kAttnMaxG) { maco_host::set_error("attention_decode: need 1..8 query heads per KV head"); return -1; }
  if (dtype != MACO_DT_BF16 && dtype != MACO_DT_F16) { maco_host::set_error("attention_decode: bf16 or fp16 only"); return -1; }
  if (splits < 1 || S < 1 || B < 1) { maco_host::set_error("attention_decode: empty problem"); return -1; }
  // the kernels read K / V rows and q with 16-byte vector loads and launch B * Hkv * splits CTAs
  if (((reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(q) |
        reinterpret_cast<uintptr_t>(out)) & 15) != 0) {
    maco_host::set_error("attention_decode: q, k, v and out must be 16-byte aligned");
    return -1;
  }
  if (kv_batch_stride % 8 != 0 || kv_head_stride % 8 != 0) {
    maco_host::set_error("attention_decode: KV batch and head strides must be multiples of 8 elements (16 bytes)");
    return -1;
  }
  if ((long long)B * Hkv * splits > 2147483647LL) { maco_host::set_error("attention_decode: B * Hkv * splits exceeds the grid limit"); return -1; }
  p.q = q; p.k = k; p.v = v; p.out = out; p.scratch = scratch; p.B = B; p.Hkv = Hkv; p.G = Hq / Hkv; p.S = S;
  p.splits = splits; p.dtype = dtype; p.kv_batch_stride = kv_batch_stride; p.kv_head_stride = kv_head_stride;
  p.scale = scale;
  return 0;
}

}  // namespace

extern "C" {

// Bytes of fp32 scratch the call needs.
unsigned long long maco_attention_decode_scratch_bytes(int B, int Hq, int Hkv, int splits) {
  const int G = Hq / (Hkv > 0 ? Hkv : 1);
  return (unsigned long long)B * Hkv * splits * (G * kAttnD + 2 * G) * sizeof(float);
}

int maco_attention_decode(const void* q, const void* k, const void* v, void* out, void* scratch, int B, int Hq, int Hkv,
                          int S, int head_dim, int splits, int dtype, long long kv_batch_stride,
                          long long kv_head_stride, float scale, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  AttnParams p;
  int rc = check_and_fill(p, q, k, v, out, reinterpret_cast<float*>(scratch), B, Hq, Hkv, S, head_dim, splits, dtype,
                          kv_batch_stride, kv_head_stride, scale);
  if (rc != 0) return rc;
  if (scratch == nullptr) { maco_host::set_error("attention_decode: scratch is null"); return -1; }
  attn_decode_kernel<<<B * Hkv * splits, 128, 0, stream>>>(p);
  attn_merge_kernel<<<B * Hkv, 128, 0, stream>>>(p);
  MACO_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // extern "C"

// ---- no-allocation variant ---------------------------------------------------------------------
// See maco_no_alloc.h for the contract. The scratch of the split-KV partials lives in this
// file-scope device array; the name below is only a host-side handle for it, so host code asks the
// runtime for the real device address once per device and hands that pointer to the kernels.
#include "maco_no_alloc.h"
#include <mutex>

static __device__ __align__(256) float g_static_attn_scratch[MACO_STATIC_SCRATCH_BYTES / sizeof(float)];

namespace {
std::mutex g_static_mu;
float* g_static_ptr[64] = {};

// Device address of the static scratch on the current device (looked up on first use).
int static_scratch_ptr(float** out) {
  int dev = 0;
  MACO_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) { maco_host::set_error("attention_decode_static: device index out of range"); return -1; }
  std::lock_guard<std::mutex> lk(g_static_mu);
  if (g_static_ptr[dev] == nullptr) {
    float* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_attn_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      maco_host::set_error(std::string("attention_decode_static: cudaGetSymbolAddress failed: ") + cudaGetErrorString(e));
      return -1;
    }
    g_static_ptr[dev] = ptr;
  }
  *out = g_static_ptr[dev];
  return 0;
}
}  // namespace

extern "C" int maco_attention_decode_static(const void* q, const void* k, const void* v, void* out, int B, int Hq,
                                            int Hkv, int S, int head_dim, int splits, int dtype,
                                            long long kv_batch_stride, long long kv_head_stride, float scale,
                                            void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  AttnParams p;
  int rc = check_and_fill(p, q, k, v, out, nullptr, B, Hq, Hkv, S, head_dim, splits, dtype, kv_batch_stride,
                          kv_head_stride, scale);
  if (rc != 0) return rc;
  const unsigned long long need = maco_attention_decode_scratch_bytes(B, Hq, Hkv, splits);
  if (need > MACO_STATIC_SCRATCH_BYTES) {
    char buf[200];
    snprintf(buf, sizeof buf,
             "attention_decode_static: needs %llu bytes of scratch, the built-in array holds %u; use fewer splits "
             "or maco_attention_decode with your own scratch", need, (unsigned)MACO_STATIC_SCRATCH_BYTES);
    maco_host::set_error(buf);
    return -3;
  }
  float* scratch = nullptr;
  rc = static_scratch_ptr(&scratch);
  if (rc != 0) return rc;
  p.scratch = scratch;
  attn_decode_kernel<<<B * Hkv * splits, 128, 0, stream>>>(p);
  attn_merge_kernel<<<B * Hkv, 128, 0, stream>>>(p);
  MACO_CHECK_CUDA(cudaGetLastError());
  return 0;
}
