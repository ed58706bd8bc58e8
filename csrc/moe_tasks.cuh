// Mixture-of-experts tasks of the persistent kernel: top-k routing fused with the dispatch
// all-to-all, publication of the per-expert counts, and the weighted return (combine) of expert
// outputs, all over NVLink peer memory from inside the kernel.
//
//   TOPK (dispatch)   per token: softmax top-k over the router logits, a slot in the destination
//                     expert's receive slab (atomic counter), the token row staged in shared memory
//                     once and sent with one bulk copy per chosen expert straight into the slab of the
//                     GPU that owns the expert (the permute IS the store address), plus a 16-byte
//                     {token, k, weight} record beside it.
//   MOE_COUNTS        after the last dispatch task: this rank's counts go to the expert owners.
//   MOE_RETURN        per (expert, source rank, 128-row block): rows below the received count are
//                     scaled by their routing weight and sent back into the source rank's combine
//                     buffer at [token, k]; the source then sums the k rows of every token.
//
// The reference has none of this: its expert-parallel example uses equal splits on one GPU and a
// dummy all_to_all node (examples/benchmark_all_to_all.py:31-127). Receive slabs have a fixed
// capacity per (source, expert); a token that does not fit is dropped for that expert (its combine
// row is zeroed at the source) and counted, never silently lost.
#pragma once
#include "elementwise.cuh"
#include "comm_tasks.cuh"

namespace maco {

struct MoeMeta { int32_t token; int32_t k; float weight; int32_t _pad; };

__device__ __forceinline__ void moe_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// One warp per token. `stage`: 4 x hidden*2 bytes of shared memory (one row per warp).
// Latency plan for a warp: the next token's row and logits are fetched into registers before the
// warp waits for the bulk engine to have read the current row out of shared memory; lane k takes the
// slot for choice k and sends copy k, so the K slot atomics and the K bulk copies of a token are one
// round trip each instead of K.
template <typename Program>
MACO_DEVICE void moe_topk_dispatch(const Program& p, const MacoEltArgs& ar, int tid, uint8_t* stage) {
  // private copies: descriptor and parameter block live in global memory; read in place every use inside the
  // loops would be a fresh load, because the loops' stores could alias them
  const MacoEltArgs a = ar;
  const MacoMoeParams m = *reinterpret_cast<const MacoMoeParams*>(a.in2);
  const int warp = tid >> 5, lane = tid & 31;
  const int E = m.experts, K = m.top_k, H = m.hidden;
  const int row_bytes = H * 2;
  const int nvec = row_bytes >> 4;                    // 16-byte vectors per row (<= 320: 10 per lane)
  uint8_t* srow = stage + (size_t)warp * row_bytes;
  const int per_lane = (E + 31) / 32;                 // logits held by each lane (<= 8: up to 256 experts)
  constexpr int kVecPerLane = 10;                      // 16-byte vectors of a row per lane: hidden <= 2560
  float v[8];
  uint4 xr[kVecPerLane];
  auto fetch = [&](int t) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int e = lane + 32 * i;
      v[i] = (i < per_lane && e < E) ? load1(m.logits, (long long)t * E + e, m.dtype) : -INFINITY;
    }
    const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(m.x) + (size_t)t * row_bytes);
#pragma unroll
    for (int i = 0; i < kVecPerLane; ++i) if (lane + 32 * i < nvec) xr[i] = src[lane + 32 * i];
  };
  const int t_end = a.row0 + a.rows;
  int t = a.row0 + warp;
  if (t < t_end) fetch(t);
  bool stores_pending = false;
  for (; t < t_end; t += 4) {
    // top-k by repeated warp arg-max (registers only)
    int sel_e[8];
    float sel_v[8];
    float vmax = -INFINITY;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      sel_e[k] = 0; sel_v[k] = -INFINITY;
      if (k < K) {
        float best = -INFINITY;
        int best_e = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < 8; ++i) if (v[i] > best) { best = v[i]; best_e = lane + 32 * i; }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const float ob = __shfl_xor_sync(0xffffffffu, best, o);
          const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
          if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
        }
        sel_e[k] = best_e; sel_v[k] = best;
        if (k == 0) vmax = best;
#pragma unroll
        for (int i = 0; i < 8; ++i) if (i == (best_e >> 5) && (best_e & 31) == lane) v[i] = -INFINITY;   // remove the winner
      }
    }
    float denom = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) if (k < K) denom += __expf(sel_v[k] - vmax);
    // lane k owns choice k: its slot atomic is issued now and overlaps the staging below
    int my_e = 0;
    float my_w = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) if (k == lane) { my_e = sel_e[k]; my_w = __expf(sel_v[k] - vmax) / denom; }
    uint32_t slot = 0;
    if (lane < K) slot = atomicAdd(&m.counts[my_e], 1u);
    // the staged row of the previous token must have been read by the bulk engine before it is overwritten
    if (stores_pending && lane < K) tma_store_wait_read<0>();
    __syncwarp();
#pragma unroll
    for (int i = 0; i < kVecPerLane; ++i) if (lane + 32 * i < nvec) reinterpret_cast<uint4*>(srow)[lane + 32 * i] = xr[i];
    const int t_cur = t;
    if (t + 4 < t_end) fetch(t + 4);                  // next token's loads fly while this one is sent
    fence_proxy_async_smem();
    __syncwarp();
    if (lane < K) {
      uint8_t* comb_row = reinterpret_cast<uint8_t*>(m.comb) + ((size_t)t_cur * K + lane) * row_bytes;
      if (slot < (uint32_t)m.capacity) {
        const int dst = my_e / m.experts_per_rank, el = my_e % m.experts_per_rank;
        const size_t cell = ((size_t)el * p.world + p.rank) * m.capacity + slot;
        bulk_store(p.peer_heap[dst] + m.recv_off + cell * row_bytes, srow, row_bytes);
        MoeMeta mm{t_cur, lane, my_w, 0};
        *reinterpret_cast<uint4*>(p.peer_heap[dst] + m.meta_off + cell * sizeof(MoeMeta)) = *reinterpret_cast<uint4*>(&mm);
      } else {
        // dropped for this expert: its combine row contributes nothing
        for (int i = 0; i < row_bytes / 16; ++i) reinterpret_cast<uint4*>(comb_row)[i] = make_uint4(0, 0, 0, 0);
        atomicAdd(&m.counts[E], 1u);                               // counts[E] = dropped (token, expert) pairs
      }
      tma_store_commit();
    }
    stores_pending = true;
  }
  if (lane < K) tma_store_wait<0>();                                // all rows have landed before the task signals
}

// counts[e] of this rank -> cnt[world][experts_per_rank] on the owner of e (slot = this rank).
template <typename Program>
MACO_DEVICE void moe_publish_counts(const Program& p, const MacoEltArgs& a, int tid) {
  const MacoMoeParams m = *reinterpret_cast<const MacoMoeParams*>(a.in2);
  for (int e = tid; e < m.experts; e += 128) {
    const int dst = e / m.experts_per_rank, el = e % m.experts_per_rank;
    uint32_t c = m.counts[e];
    if (c > (uint32_t)m.capacity) c = m.capacity;
    reinterpret_cast<uint32_t*>(p.peer_heap[dst] + m.cnt_off)[p.rank * m.experts_per_rank + el] = c;
  }
}

// rows [row0, row0+rows) of slab (el = i0, source rank = i1): y row * weight -> source's comb[token, k].
// One warp per row; the next row and its record are fetched into registers before the warp waits for
// the bulk engine to have read the current row out of shared memory.
template <typename Program>
MACO_DEVICE void moe_return(const Program& p, const MacoEltArgs& ar, int tid, uint8_t* stage) {
  const MacoEltArgs a = ar;
  const MacoMoeParams m = *reinterpret_cast<const MacoMoeParams*>(a.in2);
  const int warp = tid >> 5, lane = tid & 31;
  const int el = a.i0, src = a.i1, H = m.hidden, K = m.top_k;
  const int row_bytes = H * 2;
  const int nvec = row_bytes >> 4;
  constexpr int kVecPerLane = 10;                      // 16-byte vectors of a row per lane: hidden <= 2560
  const uint32_t count = reinterpret_cast<const uint32_t*>(p.peer_heap[p.rank] + m.cnt_off)[src * m.experts_per_rank + el];
  uint8_t* srow = stage + (size_t)warp * row_bytes;
  const size_t slab = ((size_t)el * p.world + src) * m.capacity;
  const MoeMeta* meta = reinterpret_cast<const MoeMeta*>(p.peer_heap[p.rank] + m.meta_off) + slab;
  const uint8_t* y = reinterpret_cast<const uint8_t*>(m.y) + slab * row_bytes;
  const int r_end = min(a.row0 + a.rows, (int)count);
  uint4 yr[kVecPerLane];
  MoeMeta mm{0, 0, 0.f, 0};
  auto fetch = [&](int r) {
    mm = meta[r];
    const uint4* q = reinterpret_cast<const uint4*>(y + (size_t)r * row_bytes);
#pragma unroll
    for (int i = 0; i < kVecPerLane; ++i) if (lane + 32 * i < nvec) yr[i] = q[lane + 32 * i];
  };
  int r = a.row0 + warp;
  if (r < r_end) fetch(r);
  bool pending = false;
  for (; r < r_end; r += 4) {
    if (pending && lane == 0) tma_store_wait_read<0>();
    __syncwarp();
#pragma unroll
    for (int i = 0; i < kVecPerLane; ++i) {
      if (lane + 32 * i < nvec) {
        uint32_t w[4] = {yr[i].x, yr[i].y, yr[i].z, yr[i].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = m.dtype == MACO_DT_BF16 ? unpack_bf16x2(w[j]) : __half22float2(*reinterpret_cast<__half2*>(&w[j]));
          f.x *= mm.weight; f.y *= mm.weight;
          if (m.dtype == MACO_DT_BF16) w[j] = pack_bf16x2(f.x, f.y);
          else { __half2 h = __floats2half2_rn(f.x, f.y); w[j] = *reinterpret_cast<uint32_t*>(&h); }
        }
        reinterpret_cast<uint4*>(srow)[lane + 32 * i] = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
    const MoeMeta cur = mm;
    if (r + 4 < r_end) fetch(r + 4);
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      bulk_store(p.peer_heap[src] + m.comb_off + ((size_t)cur.token * K + cur.k) * row_bytes, srow, row_bytes);
      tma_store_commit();
    }
    pending = true;
  }
  if (lane == 0) tma_store_wait<0>();
}

// Combine: out[t] = sum over k of comb[t][k] for tokens [row0, row0 + rows). A token's K rows are one
// contiguous block of the combine buffer, so with the operand ring idle (`bc` given) the leader
// streams whole token blocks into shared memory with the bulk-copy engine, half of the slots always
// in flight while the other half is summed; without the ring the rows are read with vector loads.
template <typename Program>
__device__ __noinline__ bool moe_combine(const Program& p, const MacoEltArgs& ar, int tid, BulkCtx* bc) {
  const MacoEltArgs a = ar;
  const MacoMoeParams m = *reinterpret_cast<const MacoMoeParams*>(a.in2);
  const int K = m.top_k, dt = m.dtype;
  const uint32_t row_bytes = (uint32_t)m.hidden * 2, tb = row_bytes * (uint32_t)K, nvec = row_bytes >> 4;
  const uint8_t* comb = p.peer_heap[p.rank] + m.comb_off;
  uint8_t* out = reinterpret_cast<uint8_t*>(a.out);
  const int t_end = a.row0 + a.rows;
  auto bar = [] { asm volatile("bar.sync 1, 128;" ::: "memory"); };
  uint32_t nslot = bc != nullptr ? min(bc->nbuf, (bc->nbuf * bc->buf_bytes) / tb) & ~1u : 0u;
  if (nslot < 2) {
    for (uint32_t i = tid; i < (uint32_t)a.rows * nvec; i += 128) {
      const uint32_t r = i / nvec, v = i - r * nvec;
      const uint8_t* src = comb + (size_t)(a.row0 + r) * tb + ((size_t)v << 4);
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int k = 0; k < K; ++k) add8(acc, *reinterpret_cast<const uint4*>(src + (size_t)k * row_bytes), dt);
      *reinterpret_cast<uint4*>(out + (size_t)(a.row0 + r) * row_bytes + ((size_t)v << 4)) = pack8(acc, 1.f, dt);
    }
    return true;
  }
  const uint32_t half = nslot >> 1;
  bool ok = true;
  auto issue = [&](uint32_t h, int t0) {                 // leader only
    for (uint32_t s = 0; s < half; ++s) {
      const int t = t0 + (int)s;
      if (t >= t_end) break;
      const uint32_t b = h * half + s;
      mbar_arrive_expect_tx(&bc->bars[b], tb);
      bulk_load(bc->buf + (size_t)b * tb, comb + (size_t)t * tb, tb, &bc->bars[b]);
    }
  };
  auto consume = [&](uint32_t h, int t0) {
    const uint32_t phase = *bc->phase;
    uint32_t used = 0;
    for (uint32_t s = 0; s < half; ++s) {
      const int t = t0 + (int)s;
      if (t >= t_end) break;
      const uint32_t b = h * half + s;
      used |= 1u << b;
      const uint64_t w0 = globaltimer_ns();
      while (!mbar_try_wait(&bc->bars[b], (phase >> b) & 1u)) {
        if (globaltimer_ns() - w0 > p.budget_ns) { ok = false; break; }
      }
      const uint8_t* src = bc->buf + (size_t)b * tb;
      for (uint32_t v = tid; v < nvec; v += 128) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int k = 0; k < K; ++k) add8(acc, *reinterpret_cast<const uint4*>(src + (size_t)k * row_bytes + ((size_t)v << 4)), dt);
        *reinterpret_cast<uint4*>(out + (size_t)t * row_bytes + ((size_t)v << 4)) = pack8(acc, 1.f, dt);
      }
    }
    bar();                                               // the half's buffers are consumed by everybody
    if (tid == 0) *bc->phase = phase ^ used;             // read again only after the next barrier
  };
  if (tid == 0) {
    fence_proxy_async_all();
    issue(0, a.row0);
    issue(1, a.row0 + (int)half);
  }
  for (int t0 = a.row0; t0 < t_end; t0 += (int)nslot) {
    consume(0, t0);
    if (tid == 0) issue(0, t0 + (int)nslot);
    consume(1, t0 + (int)half);
    if (tid == 0) issue(1, t0 + (int)half + (int)nslot);
  }
  bar();                                                 // the last phase word is visible before the next task reads it
  return ok;
}

}  // namespace maco
