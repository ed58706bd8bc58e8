// Element-wise and row-wise operators written as *thread-group* device functions: the same body
// runs as a task inside the persistent kernel (group = the 4 epilogue warps of a worker CTA) and
// as a stand-alone kernel (group = one CTA).
//
// Covers the reference's device tasks maco/csrc/maco_worker.cuh:66-177 (vector scale,
// LayerNorm, tanh-GELU, SiLU) and adds what the target layers need (RMSNorm, SwiGLU gate,
// residual add, RoPE, softmax, GELU backward). The reference's LayerNorm reduces with one thread
// over a 256-float shared buffer and strides rows by blockIdx (maco_worker.cuh:80-145); here one
// warp owns a row, reduces with shuffles and moves 16 bytes per lane per access.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "maco_atoms.cuh"
#include "maco_types.h"

namespace maco {

// ---- 8-wide typed access -------------------------------------------------------------------
struct F8 { float v[8]; };

MACO_DEVICE F8 load8(const void* base, long long idx, int dtype) {
  F8 r;
  if (dtype == MACO_DT_F32) {
    const float4* p = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + idx);
    float4 a = p[0], b = p[1];
    r.v[0] = a.x; r.v[1] = a.y; r.v[2] = a.z; r.v[3] = a.w; r.v[4] = b.x; r.v[5] = b.y; r.v[6] = b.z; r.v[7] = b.w;
  } else {
    uint4 u = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(base) + idx);
    uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (dtype == MACO_DT_BF16) {
        float2 f = unpack_bf16x2(w[i]);
        r.v[2 * i] = f.x; r.v[2 * i + 1] = f.y;
      } else {
        __half2 h = *reinterpret_cast<__half2*>(&w[i]);
        float2 f = __half22float2(h);
        r.v[2 * i] = f.x; r.v[2 * i + 1] = f.y;
      }
    }
  }
  return r;
}

// Raw 8-element fetch (one 16-byte vector for 16-bit types, two for fp32) and its conversion, kept
// apart so that a loop can issue several fetches before it touches the first value.
MACO_DEVICE void load8_raw(const void* base, long long idx, int dtype, uint4& lo, uint4& hi) {
  if (dtype == MACO_DT_F32) {
    const uint4* p = reinterpret_cast<const uint4*>(reinterpret_cast<const float*>(base) + idx);
    lo = p[0]; hi = p[1];
  } else {
    lo = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(base) + idx);
    hi = lo;
  }
}
MACO_DEVICE F8 cvt8(int dtype, uint4 lo, uint4 hi) {
  F8 r;
  if (dtype == MACO_DT_F32) {
    r.v[0] = __uint_as_float(lo.x); r.v[1] = __uint_as_float(lo.y); r.v[2] = __uint_as_float(lo.z); r.v[3] = __uint_as_float(lo.w);
    r.v[4] = __uint_as_float(hi.x); r.v[5] = __uint_as_float(hi.y); r.v[6] = __uint_as_float(hi.z); r.v[7] = __uint_as_float(hi.w);
  } else {
    uint32_t w[4] = {lo.x, lo.y, lo.z, lo.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = dtype == MACO_DT_BF16 ? unpack_bf16x2(w[i]) : __half22float2(*reinterpret_cast<__half2*>(&w[i]));
      r.v[2 * i] = f.x; r.v[2 * i + 1] = f.y;
    }
  }
  return r;
}

MACO_DEVICE void store8(void* base, long long idx, int dtype, const F8& r) {
  if (dtype == MACO_DT_F32) {
    float4* p = reinterpret_cast<float4*>(reinterpret_cast<float*>(base) + idx);
    p[0] = make_float4(r.v[0], r.v[1], r.v[2], r.v[3]);
    p[1] = make_float4(r.v[4], r.v[5], r.v[6], r.v[7]);
  } else {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (dtype == MACO_DT_BF16) {
        w[i] = pack_bf16x2(r.v[2 * i], r.v[2 * i + 1]);
      } else {
        __half2 h = __floats2half2_rn(r.v[2 * i], r.v[2 * i + 1]);
        w[i] = *reinterpret_cast<uint32_t*>(&h);
      }
    }
    *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(base) + idx) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

MACO_DEVICE float load1(const void* base, long long idx, int dtype) {
  if (dtype == MACO_DT_F32) return reinterpret_cast<const float*>(base)[idx];
  if (dtype == MACO_DT_F16) return __half2float(reinterpret_cast<const __half*>(base)[idx]);
  return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[idx]);
}
MACO_DEVICE void store1(void* base, long long idx, int dtype, float v) {
  if (dtype == MACO_DT_F32) reinterpret_cast<float*>(base)[idx] = v;
  else if (dtype == MACO_DT_F16) reinterpret_cast<__half*>(base)[idx] = __float2half_rn(v);
  else reinterpret_cast<__nv_bfloat16*>(base)[idx] = __float2bfloat16_rn(v);
}

MACO_DEVICE int dtype_bytes(int dtype) { return dtype == MACO_DT_F32 ? 4 : 2; }

MACO_DEVICE bool elt_vec_ok(const MacoEltArgs& a) {
  const int eb = dtype_bytes(a.dtype);
  auto al = [&](const void* p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  return (a.cols % 8) == 0 && ((long long)a.ld_in * eb) % 16 == 0 && ((long long)a.ld_out * eb) % 16 == 0 &&
         al(a.in0) && al(a.in1) && al(a.in2) && al(a.out);
}

// ---- pointwise family ----------------------------------------------------------------------
MACO_DEVICE float elt_apply(uint32_t type, float x, float y, const MacoEltArgs& a) {
  switch (type) {
    case MACO_TASK_GELU: return gelu_tanh(x);
    case MACO_TASK_SILU: return silu(x);
    case MACO_TASK_SCALE: return x * a.f0;
    case MACO_TASK_ADD: return x + y;
    case MACO_TASK_SILU_GATE: return silu(x) * y;
    case MACO_TASK_GELU_BWD: return x * gelu_tanh_grad(y);
    case MACO_TASK_AXPBY: return a.f0 * x + a.f1 * y;
    case MACO_TASK_COPY: return x;
    default: return x;
  }
}

MACO_DEVICE bool elt_is_binary(uint32_t type) {
  return type == MACO_TASK_ADD || type == MACO_TASK_SILU_GATE || type == MACO_TASK_GELU_BWD || type == MACO_TASK_AXPBY;
}

// Vector path, specialised on element type AND operator: the fetch loop is branch-free, the
// operator is resolved at compile time, and the descriptor fields are copied into registers
// first (stores through `out` could alias the descriptor otherwise, forcing reloads). Each
// instance is its own function, so its register allocation is independent of the others.
template <int OP>
MACO_DEVICE float elt_op(float x, float y, float f0, float f1) {
  if constexpr (OP == MACO_TASK_GELU) return gelu_tanh(x);
  else if constexpr (OP == MACO_TASK_SILU) return silu(x);
  else if constexpr (OP == MACO_TASK_SCALE) return x * f0;
  else if constexpr (OP == MACO_TASK_ADD) return x + y;
  else if constexpr (OP == MACO_TASK_SILU_GATE) return silu(x) * y;
  else if constexpr (OP == MACO_TASK_GELU_BWD) return x * gelu_tanh_grad(y);
  else if constexpr (OP == MACO_TASK_AXPBY) return f0 * x + f1 * y;
  else return x;
}

template <int DT, int U, int OP>
__device__ __noinline__ void elt_pointwise_vec(const MacoEltArgs& a, int tid, int nthreads) {
  constexpr bool bin = OP == MACO_TASK_ADD || OP == MACO_TASK_SILU_GATE || OP == MACO_TASK_GELU_BWD || OP == MACO_TASK_AXPBY;
  const void* in0 = a.in0;
  const void* in1 = a.in1;
  void* out = a.out;
  const float f0 = a.f0, f1 = a.f1;
  const long long row0 = a.row0, ld_in = a.ld_in, ld_out = a.ld_out;
  const uint32_t vpr = a.cols / 8;                  // vectors per row
  const uint32_t total = (uint32_t)a.rows * vpr;    // one task's rows: far below 2^32 (64-bit division is emulated)
  for (uint32_t base = tid; base < total; base += (uint32_t)nthreads * U) {
    uint4 xl[U], xh[U], yl[U], yh[U];
    long long io[U], oo[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t i = base + (uint32_t)u * nthreads;
      const uint32_t ii = i < total ? i : 0;
      const uint32_t rr = ii / vpr;
      const int c = (int)(ii - rr * vpr) * 8;
      io[u] = (row0 + rr) * ld_in + c; oo[u] = (row0 + rr) * ld_out + c;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) load8_raw(in0, io[u], DT, xl[u], xh[u]);
    if constexpr (bin) {
#pragma unroll
      for (int u = 0; u < U; ++u) load8_raw(in1, io[u], DT, yl[u], yh[u]);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t i = base + (uint32_t)u * nthreads;
      if (i >= total) continue;
      const F8 x = cvt8(DT, xl[u], xh[u]);
      F8 y;
      if constexpr (bin) y = cvt8(DT, yl[u], yh[u]);
      F8 o;
#pragma unroll
      for (int j = 0; j < 8; ++j) o.v[j] = elt_op<OP>(x.v[j], bin ? y.v[j] : 0.f, f0, f1);
      store8(out, oo[u], DT, o);
    }
  }
}

template <int DT, int U>
MACO_DEVICE void elt_pointwise_dispatch(uint32_t type, const MacoEltArgs& a, int tid, int nthreads) {
  switch (type) {
    case MACO_TASK_GELU: elt_pointwise_vec<DT, U, MACO_TASK_GELU>(a, tid, nthreads); break;
    case MACO_TASK_SILU: elt_pointwise_vec<DT, U, MACO_TASK_SILU>(a, tid, nthreads); break;
    case MACO_TASK_SCALE: elt_pointwise_vec<DT, U, MACO_TASK_SCALE>(a, tid, nthreads); break;
    case MACO_TASK_ADD: elt_pointwise_vec<DT, U, MACO_TASK_ADD>(a, tid, nthreads); break;
    case MACO_TASK_SILU_GATE: elt_pointwise_vec<DT, U, MACO_TASK_SILU_GATE>(a, tid, nthreads); break;
    case MACO_TASK_GELU_BWD: elt_pointwise_vec<DT, U, MACO_TASK_GELU_BWD>(a, tid, nthreads); break;
    case MACO_TASK_AXPBY: elt_pointwise_vec<DT, U, MACO_TASK_AXPBY>(a, tid, nthreads); break;
    default: elt_pointwise_vec<DT, U, MACO_TASK_COPY>(a, tid, nthreads); break;
  }
}

MACO_DEVICE void elt_pointwise(uint32_t type, const MacoEltArgs& a, int tid, int nthreads) {
  const bool bin = elt_is_binary(type);
  if (elt_vec_ok(a)) {
    if (a.dtype == MACO_DT_BF16) elt_pointwise_dispatch<MACO_DT_BF16, 8>(type, a, tid, nthreads);
    else if (a.dtype == MACO_DT_F16) elt_pointwise_dispatch<MACO_DT_F16, 8>(type, a, tid, nthreads);
    else elt_pointwise_dispatch<MACO_DT_F32, 4>(type, a, tid, nthreads);
  } else {
    const uint32_t total = (uint32_t)a.rows * (uint32_t)a.cols;
    for (uint32_t i = tid; i < total; i += nthreads) {
      const uint32_t rr = i / (uint32_t)a.cols;
      const long long r = a.row0 + rr;
      const int c = (int)(i - rr * (uint32_t)a.cols);
      float x = load1(a.in0, r * a.ld_in + c, a.dtype);
      float y = bin ? load1(a.in1, r * a.ld_in + c, a.dtype) : 0.f;
      store1(a.out, r * a.ld_out + c, a.dtype, elt_apply(type, x, y, a));
    }
  }
}

// ---- row-wise family: one warp per row ----------------------------------------------------
// RMSNORM: out = x * rsqrt(mean(x^2) + eps) * w          (in0 = x, in1 = w, f0 = eps)
// LAYERNORM: out = (x - mean) * rsqrt(var + eps) * w + b  (in2 = b)
// SOFTMAX: out = exp(x - max) / sum
template <int DTT, int type>
__device__ __noinline__ void elt_rowwise_t(const MacoEltArgs& ar, int tid, int nthreads) {
  const MacoEltArgs a = ar;                              // private copy: stores cannot alias it
  const int warp = tid >> 5, lane = tid & 31, nwarps = nthreads >> 5;
  const bool vec = elt_vec_ok(a);
  constexpr int U = 4;                                   // 16-byte vectors per lane fetched together
  for (int rr = warp; rr < a.rows; rr += nwarps) {
    const long long r = a.row0 + rr;
    const long long ib = r * a.ld_in, ob = r * a.ld_out;
    float s1 = 0.f, s2 = 0.f, mx = -INFINITY;
    if (vec) {
      for (int c0 = lane * 8; c0 < a.cols; c0 += 256 * U) {
        uint4 lo[U], hi[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int c = c0 + u * 256;
          if (c < a.cols) load8_raw(a.in0, ib + c, DTT, lo[u], hi[u]);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (c0 + u * 256 < a.cols) {
            const F8 x = cvt8(DTT, lo[u], hi[u]);
#pragma unroll
            for (int j = 0; j < 8; ++j) { s1 += x.v[j]; s2 += x.v[j] * x.v[j]; mx = fmaxf(mx, x.v[j]); }
          }
        }
      }
    } else {
      for (int c = lane; c < a.cols; c += 32) {
        float x = load1(a.in0, ib + c, DTT);
        s1 += x; s2 += x * x; mx = fmaxf(mx, x);
      }
    }
    float mean = 0.f, rstd = 0.f, denom = 0.f;
    if (type == MACO_TASK_RMSNORM) {
      s2 = warp_sum(s2);
      rstd = rsqrtf(s2 / a.cols + a.f0);
    } else if (type == MACO_TASK_LAYERNORM) {
      s1 = warp_sum(s1); s2 = warp_sum(s2);
      mean = s1 / a.cols;
      rstd = rsqrtf(fmaxf(s2 / a.cols - mean * mean, 0.f) + a.f0);
    } else {  // softmax
      mx = warp_max(mx);
      float e = 0.f;
      if (vec) {
        for (int c = lane * 8; c < a.cols; c += 256) {
          F8 x = load8(a.in0, ib + c, DTT);
#pragma unroll
          for (int j = 0; j < 8; ++j) e += __expf(x.v[j] - mx);
        }
      } else {
        for (int c = lane; c < a.cols; c += 32) e += __expf(load1(a.in0, ib + c, DTT) - mx);
      }
      denom = 1.f / warp_sum(e);
    }
    if (vec) {
      // second pass: the row is in L1/L2 now; fetch row and parameters in batches again
      for (int c0 = lane * 8; c0 < a.cols; c0 += 256 * U) {
        uint4 lo[U], hi[U], wl[U], wh[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int c = c0 + u * 256;
          if (c < a.cols) {
            load8_raw(a.in0, ib + c, DTT, lo[u], hi[u]);
            if (type != MACO_TASK_SOFTMAX) load8_raw(a.in1, c, DTT, wl[u], wh[u]);
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int c = c0 + u * 256;
          if (c >= a.cols) continue;
          const F8 x = cvt8(DTT, lo[u], hi[u]);
          F8 o;
          if (type == MACO_TASK_SOFTMAX) {
#pragma unroll
            for (int j = 0; j < 8; ++j) o.v[j] = __expf(x.v[j] - mx) * denom;
          } else {
            const F8 w = cvt8(DTT, wl[u], wh[u]);
            if (type == MACO_TASK_RMSNORM) {
#pragma unroll
              for (int j = 0; j < 8; ++j) o.v[j] = x.v[j] * rstd * w.v[j];
            } else {
              F8 b = load8(a.in2, c, DTT);
#pragma unroll
              for (int j = 0; j < 8; ++j) o.v[j] = (x.v[j] - mean) * rstd * w.v[j] + b.v[j];
            }
          }
          store8(a.out, ob + c, DTT, o);
        }
      }
    } else {
      for (int c = lane; c < a.cols; c += 32) {
        float x = load1(a.in0, ib + c, DTT), o;
        if (type == MACO_TASK_SOFTMAX) o = __expf(x - mx) * denom;
        else if (type == MACO_TASK_RMSNORM) o = x * rstd * load1(a.in1, c, DTT);
        else o = (x - mean) * rstd * load1(a.in1, c, DTT) + load1(a.in2, c, DTT);
        store1(a.out, ob + c, DTT, o);
      }
    }
  }
}

// RMSNorm with all 128 threads on one row (decode: fewer rows than warps in the machine). Every load of
// the row and of the weights is issued before the first use and the row stays in registers between the
// sum of squares and the scaling: one memory round trip per row. cols <= 8192, a multiple of 8.
template <int DTT>
__device__ __noinline__ void elt_rmsnorm_block_t(const MacoEltArgs& ar, int tid) {
  const MacoEltArgs a = ar;
  __shared__ float red[2][4];
  constexpr int U = 8;
  const int lane = tid & 31, warp = tid >> 5;
  for (int rr = 0; rr < a.rows; ++rr) {
    const long long r = a.row0 + rr;
    const long long ib = r * a.ld_in, ob = r * a.ld_out;
    uint4 lo[U], hi[U], wl[U], wh[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int c = (tid + u * 128) * 8;
      if (c < a.cols) { load8_raw(a.in0, ib + c, DTT, lo[u], hi[u]); load8_raw(a.in1, c, DTT, wl[u], wh[u]); }
    }
    float s2 = 0.f;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if ((tid + u * 128) * 8 < a.cols) {
        const F8 x = cvt8(DTT, lo[u], hi[u]);
#pragma unroll
        for (int j = 0; j < 8; ++j) s2 += x.v[j] * x.v[j];
      }
    }
    s2 = warp_sum(s2);
    if (lane == 0) red[rr & 1][warp] = s2;
    asm volatile("bar.sync 1, 128;" ::: "memory");
    const float rstd = rsqrtf((red[rr & 1][0] + red[rr & 1][1] + red[rr & 1][2] + red[rr & 1][3]) / a.cols + a.f0);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int c = (tid + u * 128) * 8;
      if (c < a.cols) {
        const F8 x = cvt8(DTT, lo[u], hi[u]), w = cvt8(DTT, wl[u], wh[u]);
        F8 o;
#pragma unroll
        for (int j = 0; j < 8; ++j) o.v[j] = x.v[j] * rstd * w.v[j];
        store8(a.out, ob + c, DTT, o);
      }
    }
  }
}

MACO_DEVICE void elt_rowwise(uint32_t type, const MacoEltArgs& a, int tid, int nthreads) {
  // i1 = 1 asks for the one-row-per-CTA form of RMSNorm
  if (type == MACO_TASK_RMSNORM && a.i1 == 1 && nthreads == 128 && a.cols <= 8192 && elt_vec_ok(a)) {
    if (a.dtype == MACO_DT_BF16) elt_rmsnorm_block_t<MACO_DT_BF16>(a, tid);
    else if (a.dtype == MACO_DT_F16) elt_rmsnorm_block_t<MACO_DT_F16>(a, tid);
    else elt_rmsnorm_block_t<MACO_DT_F32>(a, tid);
    return;
  }
#define MACO_ROWWISE_CASE(T)                                                              \
  case T:                                                                                 \
    if (a.dtype == MACO_DT_BF16) elt_rowwise_t<MACO_DT_BF16, T>(a, tid, nthreads);        \
    else if (a.dtype == MACO_DT_F16) elt_rowwise_t<MACO_DT_F16, T>(a, tid, nthreads);     \
    else elt_rowwise_t<MACO_DT_F32, T>(a, tid, nthreads);                                 \
    break;
  switch (type) {
    MACO_ROWWISE_CASE(MACO_TASK_RMSNORM)
    MACO_ROWWISE_CASE(MACO_TASK_LAYERNORM)
    default:
    MACO_ROWWISE_CASE(MACO_TASK_SOFTMAX)
  }
#undef MACO_ROWWISE_CASE
}

// ---- RoPE (half-rotation form) -------------------------------------------------------------
// Rows are (token, head) pairs: row = token * heads + head, cols = head_dim, i0 = heads;
// ld_in / ld_out are the TOKEN strides (heads * head_dim when packed), heads are `cols` apart.
// in1 = cos [tokens, head_dim/2], in2 = sin (same dtype as x); i1 = token index of row 0's token
// in the cos/sin tables minus row0 / heads (0 when the tables start at the first row's token).
MACO_DEVICE void elt_rope(const MacoEltArgs& ar, int tid, int nthreads) {
  const MacoEltArgs a = ar;                              // private copy: stores cannot alias it
  const int half = a.cols / 2;
  const uint32_t total = (uint32_t)a.rows * (uint32_t)half;
  for (uint32_t i = tid; i < total; i += nthreads) {
    const uint32_t rr = i / (uint32_t)half;
    const long long r = a.row0 + rr;
    const int c = (int)(i - rr * (uint32_t)half);
    const long long tok = r / a.i0 + a.i1;
    const long long ib = (r / a.i0) * a.ld_in + (r % a.i0) * a.cols, ob = (r / a.i0) * a.ld_out + (r % a.i0) * a.cols;
    const float cs = load1(a.in1, tok * half + c, a.dtype), sn = load1(a.in2, tok * half + c, a.dtype);
    const float x1 = load1(a.in0, ib + c, a.dtype), x2 = load1(a.in0, ib + c + half, a.dtype);
    store1(a.out, ob + c, a.dtype, x1 * cs - x2 * sn);
    store1(a.out, ob + c + half, a.dtype, x2 * cs + x1 * sn);
  }
}

// Per-head RMSNorm followed by RoPE, one warp per (token, head) row (Qwen3's QK-norm):
// in0 = x rows [rows, head_dim], in1 = norm weight [head_dim], in2 = cos|sin packed as
// [tokens, head_dim] (first half cos, second half sin), f0 = eps, f1 = 1 selects this fused form,
// i0 = heads, i1 = token offset into the cos/sin table.
MACO_DEVICE void elt_qknorm_rope(const MacoEltArgs& ar, int tid, int nthreads) {
  const MacoEltArgs a = ar;                              // private copy: stores cannot alias it
  const int warp = tid >> 5, lane = tid & 31, nwarps = nthreads >> 5;
  const int half = a.cols / 2;
  if (a.cols == 128 && a.dtype != MACO_DT_F32) {
    // head_dim 128, 16-bit values: a lane owns elements {2l, 2l+1} of both halves; every load of a row is
    // issued before the first use (one memory round trip per row instead of three)
    const bool bf = a.dtype == MACO_DT_BF16;
    auto up = [bf](uint32_t w) { return bf ? unpack_bf16x2(w) : __half22float2(*reinterpret_cast<const __half2*>(&w)); };
    auto pk = [bf](float x, float y) {
      if (bf) return pack_bf16x2(x, y);
      const __half2 h = __floats2half2_rn(x, y);
      return *reinterpret_cast<const uint32_t*>(&h);
    };
    const uint32_t* wv = reinterpret_cast<const uint32_t*>(a.in1);
    const uint32_t w1r = wv[lane], w2r = wv[32 + lane];
    for (int rr = warp; rr < a.rows; rr += nwarps) {
      const long long r = a.row0 + rr;
      const long long tokr = r / a.i0, head = r - tokr * a.i0;
      const uint32_t* x = reinterpret_cast<const uint32_t*>(reinterpret_cast<const uint16_t*>(a.in0) + tokr * a.ld_in + head * 128);
      const uint32_t* cs = reinterpret_cast<const uint32_t*>(reinterpret_cast<const uint16_t*>(a.in2) + (tokr + a.i1) * 128);
      uint32_t* o = reinterpret_cast<uint32_t*>(reinterpret_cast<uint16_t*>(a.out) + tokr * a.ld_out + head * 128);
      const uint32_t x1r = x[lane], x2r = x[32 + lane], cr = cs[lane], sr = cs[32 + lane];
      float2 x1 = up(x1r), x2 = up(x2r);
      const float2 c = up(cr), sn = up(sr), w1 = up(w1r), w2 = up(w2r);
      const float rstd = rsqrtf(warp_sum(x1.x * x1.x + x1.y * x1.y + x2.x * x2.x + x2.y * x2.y) / 128.f + a.f0);
      x1.x *= rstd * w1.x; x1.y *= rstd * w1.y; x2.x *= rstd * w2.x; x2.y *= rstd * w2.y;
      o[lane] = pk(x1.x * c.x - x2.x * sn.x, x1.y * c.y - x2.y * sn.y);
      o[32 + lane] = pk(x2.x * c.x + x1.x * sn.x, x2.y * c.y + x1.y * sn.y);
    }
    return;
  }
  for (int rr = warp; rr < a.rows; rr += nwarps) {
    const long long r = a.row0 + rr;
    const long long tok = r / a.i0 + a.i1;
    const long long ib = (r / a.i0) * a.ld_in + (r % a.i0) * a.cols, ob = (r / a.i0) * a.ld_out + (r % a.i0) * a.cols;
    float s2 = 0.f;
    for (int c = lane; c < a.cols; c += 32) { float x = load1(a.in0, ib + c, a.dtype); s2 += x * x; }
    const float rstd = rsqrtf(warp_sum(s2) / a.cols + a.f0);
    for (int c = lane; c < half; c += 32) {
      const float x1 = load1(a.in0, ib + c, a.dtype) * rstd * load1(a.in1, c, a.dtype);
      const float x2 = load1(a.in0, ib + c + half, a.dtype) * rstd * load1(a.in1, c + half, a.dtype);
      const float cs = load1(a.in2, tok * a.cols + c, a.dtype), sn = load1(a.in2, tok * a.cols + half + c, a.dtype);
      store1(a.out, ob + c, a.dtype, x1 * cs - x2 * sn);
      store1(a.out, ob + c + half, a.dtype, x2 * cs + x1 * sn);
    }
  }
}

// Dispatch by task type. Returns false for a type this file does not implement.
MACO_DEVICE bool elt_run(uint32_t type, const MacoEltArgs& a, int tid, int nthreads) {
  switch (type) {
    case MACO_TASK_GELU: case MACO_TASK_SILU: case MACO_TASK_SCALE: case MACO_TASK_ADD:
    case MACO_TASK_SILU_GATE: case MACO_TASK_GELU_BWD: case MACO_TASK_COPY: case MACO_TASK_AXPBY:
      elt_pointwise(type, a, tid, nthreads); return true;
    case MACO_TASK_RMSNORM: case MACO_TASK_LAYERNORM: case MACO_TASK_SOFTMAX:
      elt_rowwise(type, a, tid, nthreads); return true;
    case MACO_TASK_FILL: {
      uint32_t* o = reinterpret_cast<uint32_t*>(a.out);
      const uint32_t n = (uint32_t)a.rows * (uint32_t)a.cols;
      for (uint32_t i = tid; i < n; i += nthreads) o[i] = (uint32_t)a.i0;
      return true;
    }
    case MACO_TASK_ROPE:
      if (a.f1 == 0.f) elt_rope(a, tid, nthreads); else elt_qknorm_rope(a, tid, nthreads);
      return true;
    default: return false;
  }
}

}  // namespace maco
