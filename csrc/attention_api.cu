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
  __shared__ __align__(16) uint8_t scratch_smem[(2 * kAttnMaxG * kAttnD + 8 * kAttnMaxG) * 4];
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
