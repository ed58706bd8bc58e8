// Host launchers for the GEMM operators.
//
//   maco_gemm        tcgen05 / TMEM / TMA pipeline (bf16 or fp16 inputs, 16-byte aligned rows)
//   maco_gemm_simt   CUDA-core tiled GEMM for fp32 inputs and for shapes TMA cannot address
//
// Both compute D = epilogue(alpha * op(A) · op(B)^T) with A logically [M,K] and B logically
// [N,K]; `a_mn` / `b_mn` say that the operand is stored transposed ([K,M] / [K,N] row-major).
#include "gemm_tcgen05.cuh"
#include "host_common.h"

using namespace maco;

namespace {

// Optional per-CTA cycle counters of the stand-alone GEMM kernels (8 x int64 per CTA), off unless set.
long long* g_gemm_dbg = nullptr;

template <int BN, int STAGES, bool A_MN, bool B_MN>
int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmEpilogue& epi, int K, uint32_t idesc,
                int max_ctas, uint64_t budget_ns, cudaStream_t stream) {
  using L = GemmSmemLayout<BN, STAGES>;
  auto kern = gemm_tcgen05_kernel<BN, STAGES, A_MN, B_MN>;
  static bool attr_set[64] = {};
  int dev = 0;
  MACO_CHECK_CUDA(cudaGetDevice(&dev));
  if (!attr_set[dev]) {
    MACO_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotalBytes));
    attr_set[dev] = true;
  }
  const int m_tiles = (epi.M + kBM - 1) / kBM, n_tiles = (epi.N + BN - 1) / BN;
  int grid = m_tiles * n_tiles;
  int sms = maco_host::sm_count();
  if (max_ctas > 0 && max_ctas < sms) sms = max_ctas;
  if (grid > sms) grid = sms;
  if (grid <= 0) return 0;
  uint32_t* status = maco_host::status_device_ptr();
  kern<<<grid, kGemmThreads, L::kTotalBytes, stream>>>(tmA, tmB, epi, K, idesc, budget_ns, status, g_gemm_dbg);
  MACO_CHECK_CUDA(cudaGetLastError());
  return 0;
}

template <int BN, int STAGES>
int dispatch_major(bool a_mn, bool b_mn, const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmEpilogue& epi,
                   int K, uint32_t idesc, int max_ctas, uint64_t budget_ns, cudaStream_t stream) {
  if (!a_mn && !b_mn) return launch_gemm<BN, STAGES, false, false>(tmA, tmB, epi, K, idesc, max_ctas, budget_ns, stream);
  if (!a_mn && b_mn) return launch_gemm<BN, STAGES, false, true>(tmA, tmB, epi, K, idesc, max_ctas, budget_ns, stream);
  if (a_mn && !b_mn) return launch_gemm<BN, STAGES, true, false>(tmA, tmB, epi, K, idesc, max_ctas, budget_ns, stream);
  return launch_gemm<BN, STAGES, true, true>(tmA, tmB, epi, K, idesc, max_ctas, budget_ns, stream);
}

// fp32 operands on the tensor cores (kind::tf32): K-major operands only, 128 x 256 tiles.
int launch_gemm_tf32(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmEpilogue& epi, int K, uint32_t idesc,
                     int max_ctas, uint64_t budget_ns, cudaStream_t stream) {
  using L = GemmSmemLayout<256, 4>;
  auto kern = gemm_tcgen05_kernel<256, 4, false, false, true>;
  static bool attr_set[64] = {};
  int dev = 0;
  MACO_CHECK_CUDA(cudaGetDevice(&dev));
  if (!attr_set[dev]) {
    MACO_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotalBytes));
    attr_set[dev] = true;
  }
  int grid = ((epi.M + kBM - 1) / kBM) * ((epi.N + 255) / 256);
  int sms = maco_host::sm_count();
  if (max_ctas > 0 && max_ctas < sms) sms = max_ctas;
  if (grid > sms) grid = sms;
  if (grid <= 0) return 0;
  kern<<<grid, kGemmThreads, L::kTotalBytes, stream>>>(tmA, tmB, epi, K, idesc, budget_ns, maco_host::status_device_ptr(), g_gemm_dbg);
  MACO_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// Two-CTA tiles: clusters of two CTAs, 256 x BN per pair.
template <int BN, bool A_MN, bool B_MN>
int launch_gemm_pair(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmEpilogue& epi, int K, uint32_t idesc,
                     int max_ctas, uint64_t budget_ns, cudaStream_t stream) {
  using L = PairSmemLayout<kPairStages>;
  auto kern = gemm_tcgen05_pair_kernel<BN, A_MN, B_MN>;
  static bool attr_set[64] = {};
  int dev = 0;
  MACO_CHECK_CUDA(cudaGetDevice(&dev));
  if (!attr_set[dev]) {
    MACO_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotalBytes));
    attr_set[dev] = true;
  }
  const int m_pairs = (epi.M + 2 * kBM - 1) / (2 * kBM), n_tiles = (epi.N + BN - 1) / BN;
  int pairs = m_pairs * n_tiles;
  int sms = maco_host::sm_count();
  if (max_ctas > 0 && max_ctas < sms) sms = max_ctas;
  if (pairs > sms / 2) pairs = sms / 2;
  if (pairs <= 0) return 0;
  uint32_t* status = maco_host::status_device_ptr();
  kern<<<2 * pairs, kGemmThreads, L::kTotalBytes, stream>>>(tmA, tmB, epi, K, idesc, budget_ns, status, g_gemm_dbg);
  MACO_CHECK_CUDA(cudaGetLastError());
  return 0;
}

template <int BN>
int dispatch_major_pair(bool a_mn, bool b_mn, const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmEpilogue& epi,
                        int K, uint32_t idesc, int max_ctas, uint64_t budget_ns, cudaStream_t stream) {
  if (!a_mn && !b_mn) return launch_gemm_pair<BN, false, false>(tmA, tmB, epi, K, idesc, max_ctas, budget_ns, stream);
  if (!a_mn && b_mn) return launch_gemm_pair<BN, false, true>(tmA, tmB, epi, K, idesc, max_ctas, budget_ns, stream);
  if (a_mn && !b_mn) return launch_gemm_pair<BN, true, false>(tmA, tmB, epi, K, idesc, max_ctas, budget_ns, stream);
  return launch_gemm_pair<BN, true, true>(tmA, tmB, epi, K, idesc, max_ctas, budget_ns, stream);
}

// ---- CUDA-core GEMM: 64x64 tile, 256 threads, 4x4 outputs per thread ---------------------------
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }

template <typename T>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const T* __restrict__ A, const T* __restrict__ B, long long sam, long long sak, long long sbn,
                 long long sbk, GemmEpilogue e, int K) {
  __shared__ float sA[16][64 + 1];
  __shared__ float sB[16][64 + 1];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += 16) {
    for (int i = threadIdx.x; i < 64 * 16; i += 256) {
      int r = i >> 4, kk = i & 15;
      int m = m0 + r, n = n0 + r, k = k0 + kk;
      sA[kk][r] = (m < e.M && k < K) ? to_f32<T>(A[m * sam + k * sak]) : 0.f;
      sB[kk][r] = (n < e.N && k < K) ? to_f32<T>(B[n * sbn + k * sbk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { a[i] = sA[kk][ty * 4 + i]; b[i] = sB[kk][tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= e.M) continue;
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= e.N) continue;
      float v = acc[i][j] * e.alpha;
      if (e.bias != nullptr) v += epi_bias(e, n);
      if (e.mode == MACO_EPI_GELU) v = gelu_tanh(v);
      else if (e.mode == MACO_EPI_SILU) v = silu(v);
      else if (e.mode == MACO_EPI_GELU_BWD) v *= gelu_tanh_grad(epi_load_aux(e, m, n));
      else if (e.mode == MACO_EPI_RESIDUAL) v += epi_load_aux(e, m, n);
      const long long o = (long long)m * e.ld_out + n;
      if (e.out_type == MACO_DT_F32) {
        float* p = reinterpret_cast<float*>(e.out) + o;
        *p = (e.mode == MACO_EPI_F32_ACC) ? *p + v : v;
      } else if (e.out_type == MACO_DT_F16) {
        reinterpret_cast<__half*>(e.out)[o] = __float2half_rn(v);
      } else {
        reinterpret_cast<__nv_bfloat16*>(e.out)[o] = __float2bfloat16_rn(v);
      }
    }
  }
}

}  // namespace

extern "C" {

// Cycle counters of the stand-alone GEMM kernels: `buf` (device memory, 8 x int64 per CTA, or null to switch
// them off) receives per CTA [0] producer cycles waiting for a free stage, [1] MMA warp waiting for a free
// accumulator, [2] MMA warp waiting for operands, [3] MMA warp total, [4] producer total. Word [7] of the buffer
// is read as experiment switches (results are then meaningless): 1 = epilogue does the barrier handshake only,
// 8 = the first CTA pair also logs a %globaltimer time line of its producer and MMA loops behind word 4096.
void maco_gemm_set_debug(long long* buf) { g_gemm_dbg = buf; }

// Returns 0 on success; -2 means "operands are not TMA-addressable, use maco_gemm_simt".
int maco_gemm(const void* A, const void* B, void* D, int M, int N, int K, long long lda, long long ldb,
              long long ldd, int a_mn, int b_mn, int ab_type, int out_type, int mode, const void* bias,
              int bias_type, const void* aux, long long ld_aux, int aux_type, float alpha, int bn, int max_ctas,
              double wait_budget_ms, void* stream_, int cta_pair) {
  // cta_pair: 0 = choose (two-CTA tiles when the 256 x bn tiles cover every SM pair), 1 = one-CTA tiles, 2 = two-CTA tiles
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0) return 0;
  if (ab_type != MACO_DT_BF16 && ab_type != MACO_DT_F16) { maco_host::set_error("maco_gemm: inputs must be bf16 or fp16"); return -2; }
  if (K <= 0) { maco_host::set_error("maco_gemm: K must be positive"); return -2; }
  if (bn == 0) {
    const int m_tiles = (M + kBM - 1) / kBM;
    const int sms = maco_host::sm_count();
    bn = (N <= 128 || m_tiles * ((N + 255) / 256) < sms) ? 128 : 256;
    if (mode == MACO_EPI_SWIGLU) bn = 256;
  }
  if (bn != 128 && bn != 256) { maco_host::set_error("maco_gemm: bn must be 0, 128 or 256"); return -1; }
  // Output rows are written with 16-byte vectors.
  const int out_vec = out_type == MACO_DT_F32 ? 4 : 8;
  if ((reinterpret_cast<uintptr_t>(D) & 15) != 0 || (ldd % out_vec) != 0) {
    maco_host::set_error("maco_gemm: output base and row stride must be 16-byte aligned");
    return -2;
  }
  bool pair = cta_pair == 2;
  if (cta_pair == 0) {
    const int sms = maco_host::sm_count();
    pair = ((M + 255) / 256) * ((N + bn - 1) / bn) >= sms / 2;
  }
  CUtensorMap tmA, tmB;
  int r;
  if (!a_mn) r = maco_host::encode_tmap_2d(&tmA, A, 2, M, K, lda * 2, kBK, kBM);
  else       r = maco_host::encode_tmap_2d(&tmA, A, 2, K, M, lda * 2, 64, kBK);
  if (r != 0) return r == -2 ? -2 : -1;
  if (!b_mn) r = maco_host::encode_tmap_2d(&tmB, B, 2, N, K, ldb * 2, kBK, pair ? bn / 2 : bn);
  else       r = maco_host::encode_tmap_2d(&tmB, B, 2, K, N, ldb * 2, 64, kBK);
  if (r != 0) return r == -2 ? -2 : -1;
  GemmEpilogue e;
  e.out = D; e.bias = bias; e.aux = aux; e.ld_out = ldd; e.ld_aux = ld_aux; e.mode = mode; e.out_type = out_type;
  e.bias_type = bias_type; e.aux_type = aux_type; e.M = M; e.N = N; e.alpha = alpha; e.aux_pack = 0;
  const uint64_t budget_ns = (uint64_t)((wait_budget_ms > 0 ? wait_budget_ms : 2000.0) * 1e6);
  if (pair) {
    const uint32_t idesc2 = make_idesc(ab_type == MACO_DT_BF16 ? 1u : 0u, 2 * kBM, bn, a_mn ? 1u : 0u, b_mn ? 1u : 0u);
    if (bn == 256) return dispatch_major_pair<256>(a_mn, b_mn, tmA, tmB, e, K, idesc2, max_ctas, budget_ns, stream);
    return dispatch_major_pair<128>(a_mn, b_mn, tmA, tmB, e, K, idesc2, max_ctas, budget_ns, stream);
  }
  const uint32_t idesc = make_idesc(ab_type == MACO_DT_BF16 ? 1u : 0u, kBM, bn, a_mn ? 1u : 0u, b_mn ? 1u : 0u);
  if (bn == 256) return dispatch_major<256, 4>(a_mn, b_mn, tmA, tmB, e, K, idesc, max_ctas, budget_ns, stream);
  return dispatch_major<128, 6>(a_mn, b_mn, tmA, tmB, e, K, idesc, max_ctas, budget_ns, stream);
}

// fp32 inputs on the tensor cores as TF32 (10-bit mantissa: an opt-in, the default fp32 path is maco_gemm_simt).
// A [M, K] and B [N, K] row-major fp32 with 16-byte aligned rows; same epilogues as maco_gemm.
// Returns -2 when the operands are not TMA-addressable.
int maco_gemm_tf32(const void* A, const void* B, void* D, int M, int N, int K, long long lda, long long ldb, long long ldd,
                   int out_type, int mode, const void* bias, int bias_type, const void* aux, long long ld_aux,
                   int aux_type, float alpha, int max_ctas, double wait_budget_ms, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || mode == MACO_EPI_SWIGLU) { maco_host::set_error("maco_gemm_tf32: K must be positive; no SwiGLU epilogue"); return -2; }
  const int out_vec = out_type == MACO_DT_F32 ? 4 : 8;
  if ((reinterpret_cast<uintptr_t>(D) & 15) != 0 || (ldd % out_vec) != 0) {
    maco_host::set_error("maco_gemm_tf32: output base and row stride must be 16-byte aligned");
    return -2;
  }
  CUtensorMap tmA, tmB;
  int r = maco_host::encode_tmap_2d(&tmA, A, 4, M, K, lda * 4, kBK / 2, kBM);
  if (r != 0) return r == -2 ? -2 : -1;
  r = maco_host::encode_tmap_2d(&tmB, B, 4, N, K, ldb * 4, kBK / 2, 256);
  if (r != 0) return r == -2 ? -2 : -1;
  GemmEpilogue e;
  e.out = D; e.bias = bias; e.aux = aux; e.ld_out = ldd; e.ld_aux = ld_aux; e.mode = mode; e.out_type = out_type;
  e.bias_type = bias_type; e.aux_type = aux_type; e.M = M; e.N = N; e.alpha = alpha; e.aux_pack = 0;
  const uint64_t budget_ns = (uint64_t)((wait_budget_ms > 0 ? wait_budget_ms : 2000.0) * 1e6);
  return launch_gemm_tf32(tmA, tmB, e, K, make_idesc(2u, kBM, 256, 0u, 0u), max_ctas, budget_ns, stream);
}

// Element strides: A(m,k) = A[m*sam + k*sak], B(n,k) = B[n*sbn + k*sbk].
int maco_gemm_simt(const void* A, const void* B, void* D, int M, int N, int K, long long sam, long long sak,
                   long long sbn, long long sbk, long long ldd, int ab_type, int out_type, int mode, const void* bias,
                   int bias_type, const void* aux, long long ld_aux, int aux_type, float alpha, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0) return 0;
  GemmEpilogue e;
  e.out = D; e.bias = bias; e.aux = aux; e.ld_out = ldd; e.ld_aux = ld_aux; e.mode = mode; e.out_type = out_type;
  e.bias_type = bias_type; e.aux_type = aux_type; e.M = M; e.N = N; e.alpha = alpha; e.aux_pack = 0;
  dim3 grid((N + 63) / 64, (M + 63) / 64);
  if (ab_type == MACO_DT_F32)
    gemm_simt_kernel<float><<<grid, 256, 0, stream>>>((const float*)A, (const float*)B, sam, sak, sbn, sbk, e, K);
  else if (ab_type == MACO_DT_F16)
    gemm_simt_kernel<__half><<<grid, 256, 0, stream>>>((const __half*)A, (const __half*)B, sam, sak, sbn, sbk, e, K);
  else
    gemm_simt_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)A, (const __nv_bfloat16*)B, sam, sak, sbn, sbk, e, K);
  MACO_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // extern "C"
