// Split-K decode GEMMs: second half.
//
// A GEMM with very few rows (decode: 1..128 tokens) is bound by how fast its weight matrix streams
// out of HBM, and a single SM can only keep a few hundred KB in flight. The builder therefore cuts the
// K dimension into S slices, so that (column tiles x S) covers every SM, and the tcgen05 tiles add
// their fp32 partial sums into one [M, N] workspace with vector reductions (MACO_EPI_F32_ATOMIC).
// This task is the other half: once all slices of its rows have arrived it reads the sums, applies
// the epilogue operator, writes the 16-bit result (to local memory, or straight into every rank's
// symmetric heap for the one-shot all-reduce that follows o-proj / down-proj) and puts zeros back, so
// the workspace is clean for the next launch without a separate clearing pass.
//
// The reference runs these GEMMs as one torch.mm each (maco/task_graph/runtime.py:188-209).
//
//   in0  fp32 workspace [M, ld_in]            in1  aux rows (output dtype, stride ld_out) or null
//   in2  byte offset inside the heap (i1 = -2)  out  local destination (i1 = -1)
//   row0, rows; cols = OUTPUT columns; dtype = output type; ld_out = output row stride (elements)
//   i0   0: out = sum   1: SwiGLU over 256-column blocks [gate 128 | up 128]   2: out = sum + aux
//   i1   -1: store to `out`   -2: store to every rank's heap at in2
#pragma once
#include "elementwise.cuh"

namespace maco {

template <typename Program>
__device__ __noinline__ void splitk_finalize(const Program& p, const MacoEltArgs& ar, int tid) {
  const MacoEltArgs a = ar;
  constexpr int U = 4;
  const uint32_t nv = (uint32_t)a.cols >> 3, total = (uint32_t)a.rows * nv;
  float* ws = const_cast<float*>(reinterpret_cast<const float*>(a.in0));
  const bool swiglu = a.i0 == 1;
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  for (uint32_t base = tid; base < total; base += 128 * U) {
    float4 x[U][2], y[U][2];
    uint4 ax[U];
    float* src[U];
    long long oidx[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t i = base + u * 128;
      src[u] = nullptr;
      if (i < total) {
        const uint32_t r = i / nv, c = (i - r * nv) << 3;
        const long long row = a.row0 + r;
        src[u] = ws + row * a.ld_in + (swiglu ? ((c >> 7) << 8) + (c & 127) : c);
        oidx[u] = row * a.ld_out + c;
        x[u][0] = __ldcg(reinterpret_cast<const float4*>(src[u]));
        x[u][1] = __ldcg(reinterpret_cast<const float4*>(src[u]) + 1);
        if (swiglu) {
          y[u][0] = __ldcg(reinterpret_cast<const float4*>(src[u] + 128));
          y[u][1] = __ldcg(reinterpret_cast<const float4*>(src[u] + 128) + 1);
        }
        if (a.i0 == 2) ax[u] = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(a.in1) + oidx[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (src[u] == nullptr) continue;
      reinterpret_cast<float4*>(src[u])[0] = zero;
      reinterpret_cast<float4*>(src[u])[1] = zero;
      F8 v;
      v.v[0] = x[u][0].x; v.v[1] = x[u][0].y; v.v[2] = x[u][0].z; v.v[3] = x[u][0].w;
      v.v[4] = x[u][1].x; v.v[5] = x[u][1].y; v.v[6] = x[u][1].z; v.v[7] = x[u][1].w;
      if (swiglu) {
        reinterpret_cast<float4*>(src[u] + 128)[0] = zero;
        reinterpret_cast<float4*>(src[u] + 128)[1] = zero;
        const float up[8] = {y[u][0].x, y[u][0].y, y[u][0].z, y[u][0].w, y[u][1].x, y[u][1].y, y[u][1].z, y[u][1].w};
#pragma unroll
        for (int j = 0; j < 8; ++j) v.v[j] = silu(v.v[j]) * up[j];
      } else if (a.i0 == 2) {
        const F8 r = cvt8(a.dtype, ax[u], ax[u]);
#pragma unroll
        for (int j = 0; j < 8; ++j) v.v[j] += r.v[j];
      }
      if (a.i1 == -2) {
        const unsigned long long off = reinterpret_cast<unsigned long long>(a.in2);
        for (int k = 0; k < (int)p.world; ++k) store8(p.peer_heap[k] + off, oidx[u], a.dtype, v);
      } else {
        store8(a.out, oidx[u], a.dtype, v);
      }
    }
  }
}

}  // namespace maco
