// Split-KV decode attention for grouped-query attention (one KV head shared by G <= 8 query
// heads, head_dim 128), as tasks of the persistent kernel, plus the merge of the split partials.
//
// The reference only names ATTENTION / SOFTMAX in its task enum (maco/csrc/maco_types.h:48,53)
// and computes attention as softmax(QK^T)V with O(S^2) memory in an example
// (examples/test_overlap_attention.py:111-113). Decode attention is bound by streaming the KV
// cache from HBM, so the task reads every K and V row exactly once with 16-byte loads, keeps the
// G query rows in shared memory and carries the usual running (max, sum, output) triple, which
// also is what a ring / context-parallel merge needs.
//
// Task ATTENTION, arguments in MacoEltArgs:
//   in0 = q [G, 128]   in1 = K rows [rows, ld_in]   in2 = V rows [rows, ld_in]   (bf16 or fp16)
//   out = fp32 partial: o[G*128] (unnormalised), m[G], l[G]
//   rows = keys in this split, cols = 128, i0 = G, f0 = softmax scale
// Task ATTN_MERGE:
//   in0 = partials [i1 splits][G*128 + 2G] fp32, out = o [G, 128] (dtype), i0 = G, i1 = splits
#pragma once
#include "elementwise.cuh"

namespace maco {

constexpr int kAttnD = 128;
constexpr int kAttnMaxG = 8;

__device__ __forceinline__ void attn_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Shared memory needed by attn_decode_task.
constexpr int kAttnVStageKeys = 64;
constexpr int kAttnScratchBytes = (2 * kAttnMaxG * kAttnD + 8 * kAttnMaxG) * 4 + kAttnVStageKeys * kAttnD * 2;

template <int DTT>
__device__ __noinline__ void attn_decode_task_t(const MacoEltArgs& ar, int tid, uint8_t* scratch) {
  const MacoEltArgs a = ar;
  const int G = a.i0 < kAttnMaxG ? a.i0 : kAttnMaxG;
  float* q_s = reinterpret_cast<float*>(scratch);                 // [G][128]
  float* p_s = q_s + kAttnMaxG * kAttnD;                          // [G][128] probabilities of the chunk
  float* red = p_s + kAttnMaxG * kAttnD;                          // [4][G] cross-warp scratch
  uint16_t* v_s = reinterpret_cast<uint16_t*>(red + 8 * kAttnMaxG);   // [64][128] staged V rows (16-byte aligned)
  const int warp = tid >> 5, lane = tid & 31;
  for (int i = tid; i < G * kAttnD; i += 128) q_s[i] = load1(a.in0, i, DTT) * a.f0;
  float m_run[kAttnMaxG], l_run[kAttnMaxG], o[kAttnMaxG];
#pragma unroll
  for (int g = 0; g < kAttnMaxG; ++g) { m_run[g] = -INFINITY; l_run[g] = 0.f; o[g] = 0.f; }
  attn_bar();
  const uint16_t* K = reinterpret_cast<const uint16_t*>(a.in1);
  const uint16_t* V = reinterpret_cast<const uint16_t*>(a.in2);
  for (int base = 0; base < a.rows; base += 128) {
    const int j = base + tid;
    const bool valid = j < a.rows;
    float s[kAttnMaxG];
#pragma unroll
    for (int g = 0; g < kAttnMaxG; ++g) s[g] = 0.f;
    // one key row per thread: all 16 vector loads of the row are issued before the first use
    uint4 kr[kAttnD / 8];
    const uint4* krow = reinterpret_cast<const uint4*>(K + (long long)(valid ? j : 0) * a.ld_in);
#pragma unroll
    for (int v = 0; v < kAttnD / 8; ++v) kr[v] = valid ? ld_global_nc_v4(krow + v) : make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int v = 0; v < kAttnD / 8; ++v) {
      float kf[8];
      const uint32_t w[4] = {kr[v].x, kr[v].y, kr[v].z, kr[v].w};
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        float2 f = DTT == MACO_DT_BF16 ? unpack_bf16x2(w[t]) : __half22float2(*reinterpret_cast<const __half2*>(&w[t]));
        kf[2 * t] = f.x; kf[2 * t + 1] = f.y;
      }
#pragma unroll
      for (int g = 0; g < kAttnMaxG; ++g) {
        if (g < G) {
          const float4 q0 = *reinterpret_cast<const float4*>(q_s + g * kAttnD + v * 8);
          const float4 q1 = *reinterpret_cast<const float4*>(q_s + g * kAttnD + v * 8 + 4);
          s[g] += q0.x * kf[0] + q0.y * kf[1] + q0.z * kf[2] + q0.w * kf[3] + q1.x * kf[4] + q1.y * kf[5] +
                  q1.z * kf[6] + q1.w * kf[7];
        }
      }
    }
    // chunk maximum per head
#pragma unroll
    for (int g = 0; g < kAttnMaxG; ++g) {
      float mx = warp_max(valid ? s[g] : -INFINITY);
      if (lane == 0) red[warp * kAttnMaxG + g] = mx;
    }
    attn_bar();
    float corr[kAttnMaxG];
#pragma unroll
    for (int g = 0; g < kAttnMaxG; ++g) {
      const float cm = fmaxf(fmaxf(red[g], red[kAttnMaxG + g]), fmaxf(red[2 * kAttnMaxG + g], red[3 * kAttnMaxG + g]));
      const float m_new = fmaxf(m_run[g], cm);
      corr[g] = (m_run[g] == -INFINITY) ? 0.f : __expf(m_run[g] - m_new);
      const float pj = valid ? __expf(s[g] - m_new) : 0.f;
      p_s[g * kAttnD + tid] = pj;
      s[g] = pj;
      m_run[g] = m_new;
    }
    attn_bar();                                   // red consumed, p_s complete
#pragma unroll
    for (int g = 0; g < kAttnMaxG; ++g) {
      float sm = warp_sum(s[g]);
      if (lane == 0) red[warp * kAttnMaxG + g] = sm;
    }
#pragma unroll
    for (int g = 0; g < kAttnMaxG; ++g) o[g] *= corr[g];
    // P·V: V rows are staged 64 at a time with coalesced 16-byte loads (8 per thread in flight);
    // thread `tid` then owns output dimension `tid` of every head and reads the staged rows.
    const int nk = min(128, a.rows - base);
    for (int h0 = 0; h0 < nk; h0 += kAttnVStageKeys) {
      const int hk = min(kAttnVStageKeys, nk - h0);
      const uint4* vsrc = reinterpret_cast<const uint4*>(V + (long long)(base + h0) * a.ld_in);
      const int nvec = hk * (kAttnD / 8);
      if (a.ld_in == kAttnD) {
#pragma unroll
        for (int u = 0; u < kAttnVStageKeys * (kAttnD / 8) / 128; ++u) {
          const int i = tid + u * 128;
          if (i < nvec) reinterpret_cast<uint4*>(v_s)[i] = ld_global_nc_v4(vsrc + i);
        }
      } else {
        for (int i = tid; i < nvec; i += 128)
          reinterpret_cast<uint4*>(v_s)[i] = ld_global_nc_v4(reinterpret_cast<const uint4*>(V + (long long)(base + h0 + i / 16) * a.ld_in) + (i & 15));
      }
      attn_bar();
      int jj = 0;
      for (; jj + 4 <= hk; jj += 4) {
        float vv[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const uint16_t raw = v_s[(jj + t) * kAttnD + tid];
          vv[t] = DTT == MACO_DT_BF16 ? __uint_as_float((uint32_t)raw << 16) : __half2float(*reinterpret_cast<const __half*>(&raw));
        }
#pragma unroll
        for (int g = 0; g < kAttnMaxG; ++g) {
          if (g < G) {
            const float4 pp = *reinterpret_cast<const float4*>(p_s + g * kAttnD + h0 + jj);
            o[g] += pp.x * vv[0] + pp.y * vv[1] + pp.z * vv[2] + pp.w * vv[3];
          }
        }
      }
      for (; jj < hk; ++jj) {
        const uint16_t raw = v_s[jj * kAttnD + tid];
        const float v1 = DTT == MACO_DT_BF16 ? __uint_as_float((uint32_t)raw << 16) : __half2float(*reinterpret_cast<const __half*>(&raw));
#pragma unroll
        for (int g = 0; g < kAttnMaxG; ++g) if (g < G) o[g] += p_s[g * kAttnD + h0 + jj] * v1;
      }
      attn_bar();                                 // v_s free for the next half
    }
#pragma unroll
    for (int g = 0; g < kAttnMaxG; ++g)
      l_run[g] = l_run[g] * corr[g] + red[g] + red[kAttnMaxG + g] + red[2 * kAttnMaxG + g] + red[3 * kAttnMaxG + g];
    attn_bar();                                   // red and p_s free for the next chunk
  }
  float* out = reinterpret_cast<float*>(a.out);
#pragma unroll
  for (int g = 0; g < kAttnMaxG; ++g) if (g < G) out[g * kAttnD + tid] = o[g];
  if (tid < G) {
    float mg = -INFINITY, lg = 0.f;
#pragma unroll
    for (int g = 0; g < kAttnMaxG; ++g) if (g == tid) { mg = m_run[g]; lg = l_run[g]; }
    out[G * kAttnD + tid] = mg;
    out[G * kAttnD + G + tid] = lg;
  }
}

// ---- pipelined form (persistent kernel) ---------------------------------------------------------
// The worker's TMA warp streams the split's K and V rows through the operand ring with bulk copies
// (one 128-key chunk of K, then of V, per stage; several stages in flight), and the four general
// warps consume them from shared memory. With four warps per SM a load -> compute -> load loop is
// bound by memory latency; the ring keeps well over 100 KB in flight instead.
//   ring stage i of the task: stage_base(i) gives the shared-memory address, full[i] / empty[i] the
//   barriers; `it` is the worker's running stage counter (same convention as the GEMM pipeline).
struct AttnPipe {
  uint8_t* ring;
  uint64_t* full;
  uint64_t* empty;
  uint32_t stage_bytes, stages;
  uint64_t budget_ns;
  volatile uint32_t* abort_word;
};

MACO_DEVICE bool attn_pipelined(const MacoEltArgs& a) { return a.ld_in == kAttnD && a.rows > 0; }
MACO_DEVICE uint32_t attn_stage_uses(const MacoEltArgs& a) { return 2u * (uint32_t)((a.rows + 127) / 128); }

// Producer side: called by one thread.
MACO_DEVICE bool attn_produce(const MacoEltArgs& a, const AttnPipe& pp, uint32_t& it) {
  const uint8_t* K = reinterpret_cast<const uint8_t*>(a.in1);
  const uint8_t* V = reinterpret_cast<const uint8_t*>(a.in2);
  for (int base = 0; base < a.rows; base += 128) {
    const uint32_t bytes = (uint32_t)min(128, a.rows - base) * kAttnD * 2;
#pragma unroll
    for (int kv = 0; kv < 2; ++kv, ++it) {
      const uint32_t s = it % pp.stages, ph = (it / pp.stages) & 1;
      if (!mbar_wait(&pp.empty[s], ph ^ 1, pp.budget_ns, pp.abort_word)) return false;
      mbar_arrive_expect_tx(&pp.full[s], bytes);
      bulk_load(pp.ring + (size_t)s * pp.stage_bytes, (kv == 0 ? K : V) + (size_t)base * kAttnD * 2, bytes, &pp.full[s]);
    }
  }
  return true;
}

// Consumer side: all 128 general threads. scratch: q_s [G][128] f32, p_s [G][128] f32, red [4][G] f32.
template <int DTT>
__device__ __noinline__ bool attn_consume_t(const MacoEltArgs& ar, int tid, uint8_t* scratch, const AttnPipe& pp, uint32_t it) {
  const MacoEltArgs a = ar;
  const int G = a.i0 < kAttnMaxG ? a.i0 : kAttnMaxG;
  float* q_s = reinterpret_cast<float*>(scratch);
  float* p_s = q_s + kAttnMaxG * kAttnD;
  float* red = p_s + kAttnMaxG * kAttnD;
  const int warp = tid >> 5, lane = tid & 31;
  for (int i = tid; i < G * kAttnD; i += 128) q_s[i] = load1(a.in0, i, DTT) * a.f0;
  float m_run[kAttnMaxG], l_run[kAttnMaxG], o[kAttnMaxG];
#pragma unroll
  for (int g = 0; g < kAttnMaxG; ++g) { m_run[g] = -INFINITY; l_run[g] = 0.f; o[g] = 0.f; }
  attn_bar();
  bool ok = true;
  for (int base = 0; base < a.rows; base += 128, it += 2) {
    const int nk = min(128, a.rows - base);
    const bool valid = tid < nk;
    const uint32_t sk = it % pp.stages, phk = (it / pp.stages) & 1;
    const uint32_t sv = (it + 1) % pp.stages, phv = ((it + 1) / pp.stages) & 1;
    if (!mbar_wait(&pp.full[sk], phk, pp.budget_ns, pp.abort_word)) ok = false;
    // scores: one key row per thread, vectors visited in a per-thread rotated order (bank spread)
    float s[kAttnMaxG];
#pragma unroll
    for (int g = 0; g < kAttnMaxG; ++g) s[g] = 0.f;
    const uint8_t* krow = pp.ring + (size_t)sk * pp.stage_bytes + (size_t)tid * (kAttnD * 2);
    if (valid && ok) {
#pragma unroll
      for (int v = 0; v < kAttnD / 8; ++v) {
        const int dv = (v + tid) & 15;
        const uint4 u = *reinterpret_cast<const uint4*>(krow + dv * 16);
        float kf[8];
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          float2 f = DTT == MACO_DT_BF16 ? unpack_bf16x2(w[t]) : __half22float2(*reinterpret_cast<const __half2*>(&w[t]));
          kf[2 * t] = f.x; kf[2 * t + 1] = f.y;
        }
#pragma unroll
        for (int g = 0; g < kAttnMaxG; ++g) {
          if (g < G) {
            const float4 q0 = *reinterpret_cast<const float4*>(q_s + g * kAttnD + dv * 8);
            const float4 q1 = *reinterpret_cast<const float4*>(q_s + g * kAttnD + dv * 8 + 4);
            s[g] += q0.x * kf[0] + q0.y * kf[1] + q0.z * kf[2] + q0.w * kf[3] + q1.x * kf[4] + q1.y * kf[5] +
                    q1.z * kf[6] + q1.w * kf[7];
          }
        }
      }
    }
#pragma unroll
    for (int g = 0; g < kAttnMaxG; ++g) {
      float mx = warp_max(valid ? s[g] : -INFINITY);
      if (lane == 0) red[warp * kAttnMaxG + g] = mx;
    }
    attn_bar();                                   // K stage consumed by everybody, maxima published
    if (tid == 0) mbar_arrive(&pp.empty[sk]);
    float corr[kAttnMaxG];
#pragma unroll
    for (int g = 0; g < kAttnMaxG; ++g) {
      const float cm = fmaxf(fmaxf(red[g], red[kAttnMaxG + g]), fmaxf(red[2 * kAttnMaxG + g], red[3 * kAttnMaxG + g]));
      const float m_new = fmaxf(m_run[g], cm);
      corr[g] = (m_run[g] == -INFINITY) ? 0.f : __expf(m_run[g] - m_new);
      const float pj = valid ? __expf(s[g] - m_new) : 0.f;
      p_s[g * kAttnD + tid] = pj;
      s[g] = pj;
      m_run[g] = m_new;
      o[g] *= corr[g];
    }
    attn_bar();                                   // red consumed, p_s complete
#pragma unroll
    for (int g = 0; g < kAttnMaxG; ++g) {
      float sm = warp_sum(s[g]);
      if (lane == 0) red[warp * kAttnMaxG + g] = sm;
    }
    if (!mbar_wait(&pp.full[sv], phv, pp.budget_ns, pp.abort_word)) ok = false;
    // P.V: thread `tid` owns output dimension `tid`; the staged V rows are read straight from the ring
    const uint16_t* vcol = reinterpret_cast<const uint16_t*>(pp.ring + (size_t)sv * pp.stage_bytes) + tid;
    if (ok) {
      int jj = 0;
      for (; jj + 4 <= nk; jj += 4) {
        float vv[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const uint16_t raw = vcol[(jj + t) * kAttnD];
          vv[t] = DTT == MACO_DT_BF16 ? __uint_as_float((uint32_t)raw << 16) : __half2float(*reinterpret_cast<const __half*>(&raw));
        }
#pragma unroll
        for (int g = 0; g < kAttnMaxG; ++g) {
          if (g < G) {
            const float4 pp4 = *reinterpret_cast<const float4*>(p_s + g * kAttnD + jj);
            o[g] += pp4.x * vv[0] + pp4.y * vv[1] + pp4.z * vv[2] + pp4.w * vv[3];
          }
        }
      }
      for (; jj < nk; ++jj) {
        const uint16_t raw = vcol[jj * kAttnD];
        const float v1 = DTT == MACO_DT_BF16 ? __uint_as_float((uint32_t)raw << 16) : __half2float(*reinterpret_cast<const __half*>(&raw));
#pragma unroll
        for (int g = 0; g < kAttnMaxG; ++g) if (g < G) o[g] += p_s[g * kAttnD + jj] * v1;
      }
    }
    attn_bar();                                   // V stage and p_s consumed, sums published
    if (tid == 0) mbar_arrive(&pp.empty[sv]);
#pragma unroll
    for (int g = 0; g < kAttnMaxG; ++g)
      l_run[g] = l_run[g] * corr[g] + red[g] + red[kAttnMaxG + g] + red[2 * kAttnMaxG + g] + red[3 * kAttnMaxG + g];
    attn_bar();                                   // red free for the next chunk
  }
  float* out = reinterpret_cast<float*>(a.out);
#pragma unroll
  for (int g = 0; g < kAttnMaxG; ++g) if (g < G) out[g * kAttnD + tid] = o[g];
  if (tid < G) {
    float mg = -INFINITY, lg = 0.f;
#pragma unroll
    for (int g = 0; g < kAttnMaxG; ++g) if (g == tid) { mg = m_run[g]; lg = l_run[g]; }
    out[G * kAttnD + tid] = mg;
    out[G * kAttnD + G + tid] = lg;
  }
  return ok;
}

MACO_DEVICE bool attn_consume(const MacoEltArgs& a, int tid, uint8_t* scratch, const AttnPipe& pp, uint32_t it) {
  if (a.dtype == MACO_DT_BF16) return attn_consume_t<MACO_DT_BF16>(a, tid, scratch, pp, it);
  return attn_consume_t<MACO_DT_F16>(a, tid, scratch, pp, it);
}

MACO_DEVICE void attn_decode_task(const MacoEltArgs& a, int tid, uint8_t* scratch) {
  if (a.dtype == MACO_DT_BF16) attn_decode_task_t<MACO_DT_BF16>(a, tid, scratch);
  else attn_decode_task_t<MACO_DT_F16>(a, tid, scratch);
}

MACO_DEVICE void attn_merge_task(const MacoEltArgs& a, int tid) {
  const int G = a.i0, S = a.i1;
  const int rec = G * kAttnD + 2 * G;
  const float* part = reinterpret_cast<const float*>(a.in0);
  for (int g = 0; g < G; ++g) {
    float M = -INFINITY;
    for (int s = 0; s < S; ++s) M = fmaxf(M, part[s * rec + G * kAttnD + g]);
    float L = 0.f, acc = 0.f;
    for (int s = 0; s < S; ++s) {
      const float ms = part[s * rec + G * kAttnD + g];
      const float w = (ms == -INFINITY) ? 0.f : __expf(ms - M);
      L += part[s * rec + G * kAttnD + G + g] * w;
      acc += part[s * rec + g * kAttnD + tid] * w;
    }
    store1(a.out, g * kAttnD + tid, a.dtype, L > 0.f ? acc / L : 0.f);
  }
}

MACO_DEVICE void attn_run(uint32_t type, const MacoEltArgs& a, int tid, int nthreads, uint8_t* scratch) {
  (void)nthreads;
  if (type == MACO_TASK_ATTENTION) attn_decode_task(a, tid, scratch); else attn_merge_task(a, tid);
}

}  // namespace maco
