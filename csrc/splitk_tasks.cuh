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
//        (all four already offset to the task's first column)
//   row0, rows; cols = output columns of this task; dtype = output type; ld_out = output row stride (elements)
//   i0   0: out = sum   1: SwiGLU over 256-column blocks [gate 128 | up 128]   2: out = sum + aux
//        3: QK-norm + RoPE + scatter into q / the K and V caches (splitk_finalize_qkrope; in1 = MacoQkRopeParams)
//   i1   -1: store to `out`   -2: store to every rank's heap at in2
#pragma once
#include "elementwise.cuh"

namespace maco {

// SW: SwiGLU layout. Four vectors per thread per pass, every load issued before the first use: the four
// general warps of a worker reach only 10-20 GB/s with loads that wait for one another (a round trip to
// L2 / HBM is 0.5-1 us here), so the builder also cuts each row into column chunks, one task each.
template <bool SW, typename Program>
MACO_DEVICE void splitk_finalize_t(const Program& p, const MacoEltArgs& a, int tid) {
  constexpr int U = 4;
  const uint32_t nv = (uint32_t)a.cols >> 3, total = (uint32_t)a.rows * nv;
  float* ws = const_cast<float*>(reinterpret_cast<const float*>(a.in0));
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  for (uint32_t base = tid; base < total; base += 128 * U) {
    float4 x[U][SW ? 4 : 2];
    uint4 ax[U];
    float* src[U];
    long long oidx[U];
    bool live[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      uint32_t i = base + u * 128;
      live[u] = i < total;
      if (!live[u]) i = total - 1;                      // clamped: the load is issued anyway, the result dropped
      const uint32_t r = i / nv, c = (i - r * nv) << 3;
      const long long row = a.row0 + r;
      src[u] = ws + row * a.ld_in + (SW ? ((c >> 7) << 8) + (c & 127) : c);
      oidx[u] = row * a.ld_out + c;
      const float4* q = reinterpret_cast<const float4*>(src[u]);
      x[u][0] = __ldcg(q); x[u][1] = __ldcg(q + 1);
      if (SW) { x[u][2] = __ldcg(q + 32); x[u][3] = __ldcg(q + 33); }
      ax[u] = make_uint4(0, 0, 0, 0);
      if (a.i0 == 2) ax[u] = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(a.in1) + oidx[u]);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (!live[u]) continue;
      float4* q = reinterpret_cast<float4*>(src[u]);
      q[0] = zero; q[1] = zero;
      if (SW) { q[32] = zero; q[33] = zero; }
      F8 v;
      v.v[0] = x[u][0].x; v.v[1] = x[u][0].y; v.v[2] = x[u][0].z; v.v[3] = x[u][0].w;
      v.v[4] = x[u][1].x; v.v[5] = x[u][1].y; v.v[6] = x[u][1].z; v.v[7] = x[u][1].w;
      if (SW) {
        const float up[8] = {x[u][2].x, x[u][2].y, x[u][2].z, x[u][2].w, x[u][3].x, x[u][3].y, x[u][3].z, x[u][3].w};
#pragma unroll
        for (int j = 0; j < 8; ++j) v.v[j] = silu(v.v[j]) * up[j];
      } else if (a.i0 == 2) {
        const F8 rr = cvt8(a.dtype, ax[u], ax[u]);
#pragma unroll
        for (int j = 0; j < 8; ++j) v.v[j] += rr.v[j];
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

// Operator 3: the sums of a QKV projection become rotated queries, and keys / values in their cache rows, without
// an intermediate QKV buffer or a separate QK-norm + RoPE pass. One warp per (row, head); a lane owns elements
// {2l, 2l+1} of both halves of the head (the pairs RoPE rotates), as in elt_qknorm_rope.
//   in0 = fp32 sums at the first head of this block, ld_in = row stride; in1 = MacoQkRopeParams;
//   rows = batch rows; cols = columns of the block (a multiple of 128); ld_out = index of the block's first head.
__device__ __noinline__ void splitk_finalize_qkrope(const MacoEltArgs& ar, int tid) {
  const MacoEltArgs a = ar;
  const MacoQkRopeParams q = *reinterpret_cast<const MacoQkRopeParams*>(a.in1);
  const int warp = tid >> 5, lane = tid & 31;
  const int heads = a.cols / 128;
  const bool bf = q.dtype == MACO_DT_BF16;
  auto up = [bf](uint32_t w) { return bf ? unpack_bf16x2(w) : __half22float2(*reinterpret_cast<const __half2*>(&w)); };
  auto pk = [bf](float x, float y) {
    if (bf) return pack_bf16x2(x, y);
    const __half2 h = __floats2half2_rn(x, y);
    return *reinterpret_cast<const uint32_t*>(&h);
  };
  float* ws = const_cast<float*>(reinterpret_cast<const float*>(a.in0));
  const float2 zero = make_float2(0.f, 0.f);
  const int units = a.rows * heads;
  constexpr int U = 4;             // (row, head) units per warp and pass: every load of a pass is issued before the first use
  for (int u0 = warp * U; u0 < units; u0 += 4 * U) {
    float2 x1[U], x2[U];
    uint32_t cr[U], sr[U];
    float2* src[U];
    int head[U];
    long long row[U];
#pragma unroll
    for (int k = 0; k < U; ++k) {
      const int u = u0 + k < units ? u0 + k : units - 1;        // clamped: loaded anyway, dropped below
      const int r = u / heads, hl = u - r * heads;
      head[k] = a.ld_out + hl;
      row[k] = a.row0 + r;
      src[k] = reinterpret_cast<float2*>(ws + row[k] * a.ld_in + hl * 128);
      x1[k] = __ldcg(src[k] + lane); x2[k] = __ldcg(src[k] + 32 + lane);
      const uint32_t* cs = reinterpret_cast<const uint32_t*>(reinterpret_cast<const uint16_t*>(q.cos_sin) + row[k] * 128);
      cr[k] = cs[lane]; sr[k] = cs[32 + lane];
    }
    const uint32_t* wq = reinterpret_cast<const uint32_t*>(q.q_norm);
    const uint32_t* wk = reinterpret_cast<const uint32_t*>(q.k_norm);
    const float2 wq1 = up(wq[lane]), wq2 = up(wq[32 + lane]), wk1 = up(wk[lane]), wk2 = up(wk[32 + lane]);
#pragma unroll
    for (int k = 0; k < U; ++k) {
      if (u0 + k >= units) break;                               // uniform over the warp
      src[k][lane] = zero; src[k][32 + lane] = zero;
      // the projection's result in the layer's 16-bit type first (what a separate pass would have read)
      float2 a1 = up(pk(x1[k].x, x1[k].y)), a2 = up(pk(x2[k].x, x2[k].y));
      if (head[k] >= q.hq + q.hkv) {                             // value head: into the cache row of the new token
        uint32_t* o = reinterpret_cast<uint32_t*>(reinterpret_cast<uint16_t*>(q.v_cache) + row[k] * q.kv_batch_stride +
                                                  (long long)(head[k] - q.hq - q.hkv) * q.kv_head_stride + (long long)q.pos * 128);
        o[lane] = pk(a1.x, a1.y); o[32 + lane] = pk(a2.x, a2.y);
        continue;
      }
      const bool is_q = head[k] < q.hq;
      const float2 w1 = is_q ? wq1 : wk1, w2 = is_q ? wq2 : wk2, c = up(cr[k]), sn = up(sr[k]);
      const float rstd = rsqrtf(warp_sum(a1.x * a1.x + a1.y * a1.y + a2.x * a2.x + a2.y * a2.y) / 128.f + q.eps);
      a1.x *= rstd * w1.x; a1.y *= rstd * w1.y; a2.x *= rstd * w2.x; a2.y *= rstd * w2.y;
      uint32_t* o = is_q ? reinterpret_cast<uint32_t*>(reinterpret_cast<uint16_t*>(q.q_out) + (row[k] * q.hq + head[k]) * 128)
                         : reinterpret_cast<uint32_t*>(reinterpret_cast<uint16_t*>(q.k_cache) + row[k] * q.kv_batch_stride +
                                                       (long long)(head[k] - q.hq) * q.kv_head_stride + (long long)q.pos * 128);
      o[lane] = pk(a1.x * c.x - a2.x * sn.x, a1.y * c.y - a2.y * sn.y);
      o[32 + lane] = pk(a2.x * c.x + a1.x * sn.x, a2.y * c.y + a1.y * sn.y);
    }
  }
}

template <typename Program>
__device__ __noinline__ void splitk_finalize(const Program& p, const MacoEltArgs& ar, int tid) {
  const MacoEltArgs a = ar;
  if (a.i0 == 3) splitk_finalize_qkrope(a, tid);
  else if (a.i0 == 1) splitk_finalize_t<true>(p, a, tid);
  else splitk_finalize_t<false>(p, a, tid);
}

}  // namespace maco
