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
#include <cuda.h>
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

// ---- tensor-core form (persistent kernel) -------------------------------------------------------
// Decode attention of one (sequence, kv head, split) on the 5th-generation tensor cores, fed by the
// worker's TMA warp:
//
//   per 128-key chunk   S^T[key, head]  = K[key, :] . Q[head, :]^T      tcgen05.mma 128 x 16 x 128
//                       P = exp(S * scale - m_ref)  (registers -> bf16/fp16 tile in shared memory)
//                       O^T[dim, head] += V[key, dim]^T . P[head, key]  tcgen05.mma 128 x 16 x 128
//
// The keys (then the head dimensions) take the M = 128 rows of the instruction and the G <= 8 query
// heads of the group, padded to 16, its N columns, so the big operand of both products is the K / V
// chunk exactly as TMA delivers it: K rows as a K-major A operand (two 64-dim boxes), V rows as an
// MN-major A operand (four 64 x 64 panels). Only the small operands are built by threads: Q once per
// task, P once per chunk, both written in the 128-byte-swizzled K-major layout the descriptors expect.
//
// Three roles share a task: the worker's TMA warp streams K / V (attn_produce), its MMA warp issues every
// product (attn_mma), the four general warps do the softmax (attn_consume). A split is read once and nothing is
// reused, so the K / V chunks go through their own ring of six 32 KB stages over the worker's operand memory
// (192 KB in flight per SM) with barriers of their own, and the per-chunk dependency chain is kept
// short:
//   * scores run one chunk ahead (S double buffered in TMEM columns 0-15 / 16-31);
//   * the softmax reference m_ref is lazy: it only moves when some score exceeds it by more than
//     kAttnLazyMargin, which one barrier with an OR-reduction (also the "P complete" barrier) decides.
//     While it stands still P.V accumulates in TMEM (columns 32-47) across chunks and nothing is read
//     back; when it moves, the accumulator is drained into registers, rescaled, and restarted;
//   * the softmax denominator is kept per thread (one key per thread) and summed once per task.
//
// The reference has no attention task at all (maco/csrc/maco_types.h:24-40 lists ATTENTION, the
// worker never implements it).
struct AttnPipe {
  uint8_t* ring;
  uint64_t* full;         // [kAttnStages]
  uint64_t* empty;        // [kAttnStages]
  uint64_t budget_ns;
  volatile uint32_t* abort_word;
  const CUtensorMap* tmaps;
  uint64_t* mma_bars;     // [4]: scores ready (two buffers), P.V issued from P buffer 0 / 1 finished
  uint32_t tmem_base;
  uint64_t* p_ready;      // [3]: P buffer 0 / 1 staged by the softmax warps; [2]: Q tile staged (once per task)
  volatile uint32_t* pv_flags;   // [2]: 1 = the P.V product of this buffer adds to the accumulator, 0 = it starts a new sum
  uint32_t task_idx;      // pipelined attention tasks this worker has run before this one (parity of p_ready[2])
};

constexpr int kAttnStages = 6;
constexpr int kAttnStageBytes = 32768;               // one 128-key chunk of K or of V
constexpr int kAttnTileBytes = 4096;                 // 16 rows x 128 columns of 16-bit values, swizzled
constexpr int kAttnTcScratchBytes = 1024 + 3 * kAttnTileBytes + 4 * kAttnMaxG * 4;
constexpr float kAttnLazyMargin = 8.f;               // P <= e^8 between two moves of the reference

// ld_out carries the tensor-map indices of the K and V caches (+1 each, 16 bits each); row0 is the first
// key's row in the flattened [rows, 128] view both maps describe.
MACO_DEVICE bool attn_pipelined(const MacoEltArgs& a) { return a.ld_in == kAttnD && a.rows > 0 && a.ld_out != 0; }
MACO_DEVICE uint32_t attn_stage_uses(const MacoEltArgs& a) { return 2u * (uint32_t)((a.rows + 127) / 128); }

// Producer side: called by one thread. `ait` counts the stage uses of the attention ring on this worker.
// Called by all 32 lanes of the producer warp, converged. Lane 0 waits for the two stages of a chunk (K, then V)
// to be free and arms their barriers; lanes 0-5 then issue the chunk's six boxes with one warp instruction: lanes
// 0, 1 the two 64-dim halves of the 128 keys of K, lanes 2-5 the (64-key block, 64-dim half) boxes of V. One thread
// alone issues only a few TMA operations per microsecond, which capped this stream at about 4 TB/s over the GPU.
// `ait` advances identically in every lane.
MACO_DEVICE bool attn_produce(const MacoEltArgs& ar, const AttnPipe& pp, uint32_t& ait, uint32_t lane) {
  const MacoEltArgs a = ar;
  const CUtensorMap* tmK = pp.tmaps + ((a.ld_out & 0xffff) - 1);
  const CUtensorMap* tmV = pp.tmaps + (((uint32_t)a.ld_out >> 16) - 1);
  const bool is_k = lane < 2;
  const uint32_t vb = lane - 2;                                       // V box: bit 0 dim half, bit 1 key block
  const CUtensorMap* tm = is_k ? tmK : tmV;
  const int x = is_k ? (int)lane * 64 : (int)(vb & 1u) * 64;
  const int y_off = is_k ? 0 : (int)(vb >> 1) * 64;
  const uint32_t s_off = is_k ? lane * 16384u : (vb >> 1) * 16384u + (vb & 1u) * 8192u;
  for (int base = 0; base < a.rows; base += 128) {
    const int y = a.row0 + base;
    const uint32_t sk = ait % kAttnStages, phk = (ait / kAttnStages) & 1;
    const uint32_t sv = (ait + 1) % kAttnStages, phv = ((ait + 1) / kAttnStages) & 1;
    uint32_t good = 1;
    if (lane == 0) {
      good = (mbar_wait(&pp.empty[sk], phk ^ 1, pp.budget_ns, pp.abort_word) &&
              mbar_wait(&pp.empty[sv], phv ^ 1, pp.budget_ns, pp.abort_word)) ? 1u : 0u;
      if (good) {
        mbar_arrive_expect_tx(&pp.full[sk], kAttnStageBytes);
        mbar_arrive_expect_tx(&pp.full[sv], kAttnStageBytes);
      }
    }
    good = __shfl_sync(0xffffffffu, good, 0);
    if (!good) return false;
    if (lane < 6) {
      const uint32_t s = is_k ? sk : sv;
      tma_load_2d(pp.ring + (size_t)s * kAttnStageBytes + s_off, tm, &pp.full[s], x, y + y_off);
    }
    __syncwarp();
    ait += 2;
  }
  return true;
}

// Waits (bounded) until the last uses of the attention ring have been released by the consumer: the
// operand memory may then be handed to another pipeline.
MACO_DEVICE bool attn_ring_drained(const AttnPipe& pp, uint32_t ait) {
  for (uint32_t u = ait > (uint32_t)kAttnStages ? ait - kAttnStages : 0; u < ait; ++u)
    if (!mbar_wait(&pp.empty[u % kAttnStages], (u / kAttnStages) & 1, pp.budget_ns, pp.abort_word)) return false;
  return true;
}

// After an abort: loads still in flight get a bounded time to land (their destination is this CTA's memory).
MACO_DEVICE void attn_drain_loads(const AttnPipe& pp, uint32_t ait) {
  for (uint32_t u = ait > (uint32_t)kAttnStages ? ait - kAttnStages : 0; u < ait; ++u) {
    const uint64_t t0 = globaltimer_ns();
    while (!mbar_try_wait(&pp.full[u % kAttnStages], (u / kAttnStages) & 1)) {
      if (globaltimer_ns() - t0 > 2000000ull) break;
    }
  }
}

// Byte offset of element (row, col) inside a 16-row x 128-column K-major tile of 16-bit values stored
// as two 64-column atoms with the 128-byte swizzle (the tile's base is 1024-byte aligned).
MACO_DEVICE uint32_t attn_tile_off(int row, int col) {
  return (uint32_t)((col >> 6) * 2048 + (row >> 3) * 1024 + (row & 7) * 128 + ((((col & 63) >> 3) ^ (row & 7)) << 4) + (col & 7) * 2);
}

// Maximum over the warp in one instruction (sm_100a).
MACO_DEVICE float warp_max_redux(float v) {
  float r;
  asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
  return r;
}

// Barrier of the 128 general threads that also ORs a predicate over them.
MACO_DEVICE bool attn_bar_or(bool pred) {
  uint32_t r;
  asm volatile("{\n .reg .pred p, q;\n setp.ne.u32 q, %1, 0;\n bar.red.or.pred p, 1, 128, q;\n selp.u32 %0, 1, 0, p;\n}"
               : "=r"(r) : "r"((uint32_t)pred) : "memory");
  return r != 0;
}

// Softmax side: all 128 general threads; they wait for scores, stage P and post "P staged", and never issue a
// tensor-core product themselves (attn_mma does, on the MMA warp). `ait`: this task's first use of the attention
// ring (kept for symmetry with the other two roles). `chunk_seq` counts the chunks this worker has processed
// (buffer index and parity of the MMA barriers); every thread keeps its own copy.
template <int DTT>
__device__ __noinline__ bool attn_consume_t(const MacoEltArgs& ar, int tid, uint8_t* scratch, const AttnPipe& pp, uint32_t ait,
                                            uint32_t& chunk_seq) {
  const MacoEltArgs a = ar;
  const int G = a.i0 < kAttnMaxG ? a.i0 : kAttnMaxG;
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(scratch) + 1023) & ~uintptr_t(1023));
  uint8_t* q_t = tiles;                                  // Q  [16 heads][128 dims]
  uint8_t* p_t = tiles + kAttnTileBytes;                 // P  [2][16 heads][128 keys]
  float* red_m = reinterpret_cast<float*>(tiles + 3 * kAttnTileBytes);
  const int lane = tid & 31;
  const int quarter = ((tid >> 5) + 2) & 3;              // TMEM lane quarter this warp may read (warp id mod 4)
  const int row = quarter * 32 + lane;                   // key of the chunk, then output dimension, of this thread
  const int wslot = tid >> 5;
  // Q: 16 x 16 vectors of 16 bytes; rows >= G are zero. P: zero everywhere (rows >= G stay zero).
  for (int i = tid; i < 256; i += 128) {
    const int r = i >> 4, v = i & 15;
    uint4 u = make_uint4(0, 0, 0, 0);
    if (r < G) u = reinterpret_cast<const uint4*>(a.in0)[r * 16 + v];
    *reinterpret_cast<uint4*>(q_t + attn_tile_off(r, v * 8)) = u;
    *reinterpret_cast<uint4*>(p_t + i * 16) = make_uint4(0, 0, 0, 0);
    *reinterpret_cast<uint4*>(p_t + kAttnTileBytes + i * 16) = make_uint4(0, 0, 0, 0);
  }
  fence_proxy_async_smem();
  float m_ref[kAttnMaxG], l_thr[kAttnMaxG], o[kAttnMaxG];
#pragma unroll
  for (int g = 0; g < kAttnMaxG; ++g) { m_ref[g] = -INFINITY; l_thr[g] = 0.f; o[g] = 0.f; }
  attn_bar();
  if (tid == 0) mbar_arrive(&pp.p_ready[2]);             // Q and the zeroed P buffers are in place: the MMA warp may start
  bool ok = true;
  bool acc_live = false;                                 // TMEM holds P.V sums not yet drained (same in every thread)
  const uint32_t t_lane = (uint32_t)(quarter * 32) << 16;
  const uint32_t t_o = pp.tmem_base + 32;
  const int chunks = (a.rows + 127) / 128;

  // every thread: waits for the P.V of chunk `seq` (and all before it), then o += accumulator
  auto drain_output = [&](uint32_t seq) {
    if (!mbar_wait(&pp.mma_bars[2 + (seq & 1)], (seq >> 1) & 1, pp.budget_ns, pp.abort_word)) ok = false;
    tc_fence_after();
    uint32_t r[16];
    if (ok) { tmem_ld_32x16(t_o + t_lane, r); tmem_ld_wait(); }
#pragma unroll
    for (int g = 0; g < kAttnMaxG; ++g) o[g] += (ok && g < G) ? __uint_as_float(r[g]) : 0.f;
    tc_fence_before();
  };
  // every thread: P[g][row] = exp(s - m_ref) rounded to the operand type; returns the rounded values
  auto store_p = [&](uint8_t* p_buf, const float (&s)[kAttnMaxG], float (&pr)[kAttnMaxG]) {
#pragma unroll
    for (int g = 0; g < kAttnMaxG; ++g) {
      float pj = (g < G && m_ref[g] != -INFINITY) ? __expf(s[g] - m_ref[g]) : 0.f;
      if (g < G) {
        // the product uses the rounded value; the denominator sums the same one, so the two agree
        if (DTT == MACO_DT_BF16) {
          const __nv_bfloat16 h = __float2bfloat16_rn(pj);
          *reinterpret_cast<__nv_bfloat16*>(p_buf + attn_tile_off(g, row)) = h;
          pj = __bfloat162float(h);
        } else {
          const __half h = __float2half_rn(pj);
          *reinterpret_cast<__half*>(p_buf + attn_tile_off(g, row)) = h;
          pj = __half2float(h);
        }
      }
      pr[g] = pj;
    }
    fence_proxy_async_smem();
  };

  for (int c = 0; c < chunks; ++c, ++chunk_seq) {
    const int nk = min(128, a.rows - c * 128);
    const bool valid = row < nk;
    const uint32_t seq = chunk_seq, buf = seq & 1, par = (seq >> 1) & 1;
    if (!mbar_wait(&pp.mma_bars[buf], par, pp.budget_ns, pp.abort_word)) ok = false;
    tc_fence_after();
    float s[kAttnMaxG], pr[kAttnMaxG];
    {
      uint32_t r[16];
      if (ok) { tmem_ld_32x16(pp.tmem_base + buf * 16 + t_lane, r); tmem_ld_wait(); }
#pragma unroll
      for (int g = 0; g < kAttnMaxG; ++g) s[g] = (ok && valid && g < G) ? __uint_as_float(r[g]) * a.f0 : -INFINITY;
    }
    tc_fence_before();
    // the P buffer is free once the product issued from it two chunks ago has finished
    if (c >= 2 && !mbar_wait(&pp.mma_bars[2 + buf], ((seq - 2) >> 1) & 1, pp.budget_ns, pp.abort_word)) ok = false;
    uint8_t* p_buf = p_t + buf * kAttnTileBytes;
    bool exceed = false;
#pragma unroll
    for (int g = 0; g < kAttnMaxG; ++g) exceed |= s[g] > m_ref[g] + kAttnLazyMargin;
    store_p(p_buf, s, pr);
    if (attn_bar_or(exceed)) {                    // P complete, and: does the reference have to move?
#pragma unroll
      for (int g = 0; g < kAttnMaxG; ++g) {
        const float mx = warp_max_redux(s[g]);
        if (lane == g) red_m[wslot * kAttnMaxG + g] = mx;
      }
      if (acc_live) drain_output(seq - 1);        // sums under the old reference leave TMEM
      attn_bar();
#pragma unroll
      for (int g = 0; g < kAttnMaxG; ++g) {
        const float cm = fmaxf(fmaxf(red_m[g], red_m[kAttnMaxG + g]), fmaxf(red_m[2 * kAttnMaxG + g], red_m[3 * kAttnMaxG + g]));
        const float m_new = fmaxf(m_ref[g], cm);
        const float corr = (m_ref[g] == -INFINITY) ? 0.f : __expf(m_ref[g] - m_new);
        o[g] *= corr;
        l_thr[g] *= corr;
        m_ref[g] = m_new;
      }
      store_p(p_buf, s, pr);
      acc_live = false;
      attn_bar();                                 // P complete under the new reference; red_m free
    }
#pragma unroll
    for (int g = 0; g < kAttnMaxG; ++g) l_thr[g] += pr[g];
    // P of this chunk is staged (the barrier above ordered every thread's stores and proxy fence): hand it to
    // the MMA warp, which issues the P.V product as soon as the chunk's V rows have landed
    if (tid == 0) {
      pp.pv_flags[buf] = acc_live ? 1u : 0u;
      mbar_arrive(&pp.p_ready[buf]);
    }
    acc_live = true;
  }
  drain_output(chunk_seq - 1);
  // softmax denominator: one CTA-wide sum per head
#pragma unroll
  for (int g = 0; g < kAttnMaxG; ++g) {
    const float sm = warp_sum(l_thr[g]);
    if (lane == 0) red_m[wslot * kAttnMaxG + g] = sm;
  }
  attn_bar();
  float* out = reinterpret_cast<float*>(a.out);
  const int S = a.i1;                              // splits of this (sequence, kv head); the last one to finish merges
  uint32_t* counter = reinterpret_cast<uint32_t*>(const_cast<void*>(a.in1));
  if (S <= 1 && counter != nullptr) {
    // a single split: normalise and write the final rows directly
#pragma unroll
    for (int g = 0; g < kAttnMaxG; ++g) {
      if (g < G) {
        const float l = red_m[g] + red_m[kAttnMaxG + g] + red_m[2 * kAttnMaxG + g] + red_m[3 * kAttnMaxG + g];
        store1(const_cast<void*>(a.in2), g * kAttnD + row, DTT, l > 0.f ? o[g] / l : 0.f);
      }
    }
  } else {
#pragma unroll
    for (int g = 0; g < kAttnMaxG; ++g) if (g < G) out[g * kAttnD + row] = o[g];
    if (tid < G) {
      float mg = -INFINITY;
#pragma unroll
      for (int g = 0; g < kAttnMaxG; ++g) if (g == tid) mg = m_ref[g];
      out[G * kAttnD + tid] = mg;
      out[G * kAttnD + G + tid] = red_m[tid] + red_m[kAttnMaxG + tid] + red_m[2 * kAttnMaxG + tid] + red_m[3 * kAttnMaxG + tid];
    }
    if (counter != nullptr) {
      // The split that arrives last at the group's counter combines all S records (no separate merge
      // task, no extra dependency hop). The counter only grows: S arrivals per launch.
      __threadfence();                             // this thread's part of the record is visible GPU-wide
      attn_bar();
      __shared__ uint32_t s_last;
      if (tid == 0) s_last = ((atomicAdd(counter, 1u) + 1u) % (uint32_t)S) == 0u ? 1u : 0u;
      attn_bar();
      if (s_last != 0u) {
        __threadfence();
        const int rec = G * kAttnD + 2 * G;
        const float* part = out - (size_t)(int)a.f1 * rec;      // record of split 0 of this group
        float M[kAttnMaxG], L[kAttnMaxG], acc[kAttnMaxG];
#pragma unroll
        for (int g = 0; g < kAttnMaxG; ++g) { M[g] = -INFINITY; L[g] = 0.f; acc[g] = 0.f; }
        for (int sp = 0; sp < S; ++sp) {
#pragma unroll
          for (int g = 0; g < kAttnMaxG; ++g) if (g < G) M[g] = fmaxf(M[g], __ldcg(part + sp * rec + G * kAttnD + g));
        }
        for (int sp = 0; sp < S; ++sp) {
          float ms[kAttnMaxG], ls[kAttnMaxG], os[kAttnMaxG];
#pragma unroll
          for (int g = 0; g < kAttnMaxG; ++g) {
            ms[g] = g < G ? __ldcg(part + sp * rec + G * kAttnD + g) : -INFINITY;
            ls[g] = g < G ? __ldcg(part + sp * rec + G * kAttnD + G + g) : 0.f;
            os[g] = g < G ? __ldcg(part + sp * rec + g * kAttnD + row) : 0.f;
          }
#pragma unroll
          for (int g = 0; g < kAttnMaxG; ++g) {
            const float w = (ms[g] == -INFINITY) ? 0.f : __expf(ms[g] - M[g]);
            L[g] += ls[g] * w;
            acc[g] += os[g] * w;
          }
        }
#pragma unroll
        for (int g = 0; g < kAttnMaxG; ++g)
          if (g < G) store1(const_cast<void*>(a.in2), g * kAttnD + row, DTT, L[g] > 0.f ? acc[g] / L[g] : 0.f);
      }
    }
  }
  attn_bar();                                     // red_m is free again
  return ok;
}

// MMA side of the task: one thread (the worker's MMA warp, idle during an attention task otherwise) issues every
// tensor-core product, so the softmax warps never issue one. Per chunk c: scores S(c+1) = K(c+1) Q^T as soon as the
// chunk's K rows have landed (into the score buffer the softmax warps left two chunks ago), then, when the softmax
// warps have staged P(c), O (+)= V(c)^T P(c). With the issue inside the softmax loop, one thread's instruction stream
// (two waits, 16 descriptor pairs, 16 MMAs, 4 commits per chunk) sat on the critical path of all 128 threads and
// held a worker at about 23 GB/s of K/V.
// `ait`, `chunk_seq`: this worker's ring uses and chunks before this task (same counts as the consumer's).
MACO_DEVICE bool attn_mma(const MacoEltArgs& ar, uint8_t* scratch, const AttnPipe& pp, uint32_t ait, uint32_t chunk_seq) {
  const MacoEltArgs a = ar;
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(scratch) + 1023) & ~uintptr_t(1023));
  const uint32_t q_addr = smem_u32(tiles), p_addr = smem_u32(tiles + kAttnTileBytes);
  const uint32_t fmt = a.dtype == MACO_DT_BF16 ? 1u : 0u;
  const uint32_t idesc_s = make_idesc(fmt, 128, 16, 0, 0);
  const uint32_t idesc_o = make_idesc(fmt, 128, 16, 1, 0);
  const uint32_t t_o = pp.tmem_base + 32;
  const int chunks = (a.rows + 127) / 128;
  if (!mbar_wait(&pp.p_ready[2], pp.task_idx & 1u, pp.budget_ns, pp.abort_word)) return false;
  auto issue_scores = [&](int c, uint32_t seq) -> bool {
    const uint32_t u = ait + 2u * (uint32_t)c, sk = u % kAttnStages, phk = (u / kAttnStages) & 1;
    if (!mbar_wait(&pp.full[sk], phk, pp.budget_ns, pp.abort_word)) return false;
    tc_fence_after();
    const uint32_t k_addr = smem_u32(pp.ring + (size_t)sk * kAttnStageBytes);
    const uint32_t t_s = pp.tmem_base + (seq & 1) * 16;
#pragma unroll
    for (int k = 0; k < kAttnD / 16; ++k) {
      const uint64_t adesc = make_smem_desc(k_addr + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024, 2);
      const uint64_t bdesc = make_smem_desc(q_addr + (k >> 2) * 2048 + (k & 3) * 32, 16, 1024, 2);
      tc_mma_f16(t_s, adesc, bdesc, idesc_s, k != 0 ? 1u : 0u);
    }
    tc_commit(&pp.empty[sk]);
    tc_commit(&pp.mma_bars[seq & 1]);
    return true;
  };
  if (!issue_scores(0, chunk_seq)) return false;
  for (int c = 0; c < chunks; ++c) {
    const uint32_t seq = chunk_seq + (uint32_t)c, buf = seq & 1, par = (seq >> 1) & 1;
    if (c + 1 < chunks && !issue_scores(c + 1, seq + 1)) return false;
    if (!mbar_wait(&pp.p_ready[buf], par, pp.budget_ns, pp.abort_word)) return false;
    const uint32_t accum = pp.pv_flags[buf];
    const uint32_t u = ait + 2u * (uint32_t)c + 1u, sv = u % kAttnStages, phv = (u / kAttnStages) & 1;
    if (!mbar_wait(&pp.full[sv], phv, pp.budget_ns, pp.abort_word)) return false;
    tc_fence_after();
    const uint32_t v_addr = smem_u32(pp.ring + (size_t)sv * kAttnStageBytes);
    const uint32_t pb = p_addr + buf * kAttnTileBytes;
#pragma unroll
    for (int k = 0; k < 128 / 16; ++k) {
      const uint64_t adesc = make_smem_desc(v_addr + (k >> 2) * 16384 + (k & 3) * 2048, 8192, 1024, 2);
      const uint64_t bdesc = make_smem_desc(pb + (k >> 2) * 2048 + (k & 3) * 32, 16, 1024, 2);
      tc_mma_f16(t_o, adesc, bdesc, idesc_o, (k != 0 || accum != 0) ? 1u : 0u);
    }
    tc_commit(&pp.empty[sv]);
    tc_commit(&pp.mma_bars[2 + buf]);
  }
  return true;
}

MACO_DEVICE bool attn_consume(const MacoEltArgs& a, int tid, uint8_t* scratch, const AttnPipe& pp, uint32_t it, uint32_t& chunk_seq) {
  if (a.dtype == MACO_DT_BF16) return attn_consume_t<MACO_DT_BF16>(a, tid, scratch, pp, it, chunk_seq);
  return attn_consume_t<MACO_DT_F16>(a, tid, scratch, pp, it, chunk_seq);
}

MACO_DEVICE void attn_decode_task(const MacoEltArgs& a, int tid, uint8_t* scratch) {
  if (a.dtype == MACO_DT_BF16) attn_decode_task_t<MACO_DT_BF16>(a, tid, scratch);
  else attn_decode_task_t<MACO_DT_F16>(a, tid, scratch);
}

// Combines the S split records {o[G][128], m[G], l[G]} of one (sequence, kv head): thread `tid` owns output
// dimension `tid` of every head. The loads of one split are independent of each other (8 heads in flight).
MACO_DEVICE void attn_merge_task(const MacoEltArgs& ar, int tid) {
  const MacoEltArgs a = ar;                              // private copy: stores cannot alias it
  const int G = a.i0 < kAttnMaxG ? a.i0 : kAttnMaxG, S = a.i1;
  const int rec = G * kAttnD + 2 * G;
  const float* part = reinterpret_cast<const float*>(a.in0);
  float M[kAttnMaxG], L[kAttnMaxG], acc[kAttnMaxG];
#pragma unroll
  for (int g = 0; g < kAttnMaxG; ++g) { M[g] = -INFINITY; L[g] = 0.f; acc[g] = 0.f; }
  for (int s = 0; s < S; ++s) {
#pragma unroll
    for (int g = 0; g < kAttnMaxG; ++g) if (g < G) M[g] = fmaxf(M[g], part[s * rec + G * kAttnD + g]);
  }
  for (int s = 0; s < S; ++s) {
    float ms[kAttnMaxG], ls[kAttnMaxG], os[kAttnMaxG];
#pragma unroll
    for (int g = 0; g < kAttnMaxG; ++g) {
      ms[g] = g < G ? part[s * rec + G * kAttnD + g] : -INFINITY;
      ls[g] = g < G ? part[s * rec + G * kAttnD + G + g] : 0.f;
      os[g] = g < G ? part[s * rec + g * kAttnD + tid] : 0.f;
    }
#pragma unroll
    for (int g = 0; g < kAttnMaxG; ++g) {
      const float w = (ms[g] == -INFINITY) ? 0.f : __expf(ms[g] - M[g]);
      L[g] += ls[g] * w;
      acc[g] += os[g] * w;
    }
  }
#pragma unroll
  for (int g = 0; g < kAttnMaxG; ++g) if (g < G) store1(a.out, g * kAttnD + tid, a.dtype, L[g] > 0.f ? acc[g] / L[g] : 0.f);
}

MACO_DEVICE void attn_run(uint32_t type, const MacoEltArgs& a, int tid, int nthreads, uint8_t* scratch) {
  (void)nthreads;
  if (type == MACO_TASK_ATTENTION) attn_decode_task(a, tid, scratch); else attn_merge_task(a, tid);
}

}  // namespace maco
