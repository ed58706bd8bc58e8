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

namespace maco {

struct MoeMeta { int32_t token; int32_t k; float weight; int32_t _pad; };

__device__ __forceinline__ void moe_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// One warp per token. `stage`: 4 x hidden*2 bytes of shared memory (one row per warp).
template <typename Program>
MACO_DEVICE void moe_topk_dispatch(const Program& p, const MacoEltArgs& a, int tid, uint8_t* stage) {
  const MacoMoeParams& m = *reinterpret_cast<const MacoMoeParams*>(a.in2);
  const int warp = tid >> 5, lane = tid & 31;
  const int E = m.experts, K = m.top_k, H = m.hidden;
  const int row_bytes = H * 2;
  uint8_t* srow = stage + (size_t)warp * row_bytes;
  const int per_lane = (E + 31) / 32;                 // logits held by each lane (<= 8: up to 256 experts)
  for (int t = a.row0 + warp; t < a.row0 + a.rows; t += 4) {
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int e = lane + 32 * i;
      v[i] = (i < per_lane && e < E) ? load1(m.logits, (long long)t * E + e, m.dtype) : -INFINITY;
    }
    // stage the token row once (coalesced 16-byte loads)
    const uint4* xr = reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(m.x) + (size_t)t * row_bytes);
    for (int i = lane; i < row_bytes / 16; i += 32) reinterpret_cast<uint4*>(srow)[i] = xr[i];
    // top-k by repeated warp arg-max
    int sel_e[8];
    float sel_v[8];
    float vmax = -INFINITY;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
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
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        if (k >= K) break;
        const int e = sel_e[k];
        const float w = __expf(sel_v[k] - vmax) / denom;
        const uint32_t slot = atomicAdd(&m.counts[e], 1u);
        uint8_t* comb_row = reinterpret_cast<uint8_t*>(m.comb) + ((size_t)t * K + k) * row_bytes;
        if (slot < (uint32_t)m.capacity) {
          const int dst = e / m.experts_per_rank, el = e % m.experts_per_rank;
          const size_t cell = ((size_t)el * p.world + p.rank) * m.capacity + slot;
          bulk_store(p.peer_heap[dst] + m.recv_off + cell * row_bytes, srow, row_bytes);
          MoeMeta mm{t, k, w, 0};
          *reinterpret_cast<uint4*>(p.peer_heap[dst] + m.meta_off + cell * sizeof(MoeMeta)) = *reinterpret_cast<uint4*>(&mm);
        } else {
          // dropped for this expert: its combine row contributes nothing
          for (int i = 0; i < row_bytes / 16; ++i) reinterpret_cast<uint4*>(comb_row)[i] = make_uint4(0, 0, 0, 0);
          atomicAdd(&m.counts[E], 1u);                               // counts[E] = dropped (token, expert) pairs
        }
      }
      tma_store_commit();
      tma_store_wait_read<0>();                                      // the staged row may be overwritten
    }
    __syncwarp();
  }
  if (lane == 0) tma_store_wait<0>();                                // all rows have landed before the task signals
}

// counts[e] of this rank -> cnt[world][experts_per_rank] on the owner of e (slot = this rank).
template <typename Program>
MACO_DEVICE void moe_publish_counts(const Program& p, const MacoEltArgs& a, int tid) {
  const MacoMoeParams& m = *reinterpret_cast<const MacoMoeParams*>(a.in2);
  for (int e = tid; e < m.experts; e += 128) {
    const int dst = e / m.experts_per_rank, el = e % m.experts_per_rank;
    uint32_t c = m.counts[e];
    if (c > (uint32_t)m.capacity) c = m.capacity;
    reinterpret_cast<uint32_t*>(p.peer_heap[dst] + m.cnt_off)[p.rank * m.experts_per_rank + el] = c;
  }
}

// rows [row0, row0+rows) of slab (el = i0, source rank = i1): y row * weight -> source's comb[token, k].
template <typename Program>
MACO_DEVICE void moe_return(const Program& p, const MacoEltArgs& a, int tid, uint8_t* stage) {
  const MacoMoeParams& m = *reinterpret_cast<const MacoMoeParams*>(a.in2);
  const int warp = tid >> 5, lane = tid & 31;
  const int el = a.i0, src = a.i1, H = m.hidden, K = m.top_k;
  const int row_bytes = H * 2;
  const uint32_t count = reinterpret_cast<const uint32_t*>(p.peer_heap[p.rank] + m.cnt_off)[src * m.experts_per_rank + el];
  uint8_t* srow = stage + (size_t)warp * row_bytes;
  const size_t slab = ((size_t)el * p.world + src) * m.capacity;
  const MoeMeta* meta = reinterpret_cast<const MoeMeta*>(p.peer_heap[p.rank] + m.meta_off) + slab;
  const uint8_t* y = reinterpret_cast<const uint8_t*>(m.y) + slab * row_bytes;
  for (int r = a.row0 + warp; r < a.row0 + a.rows && (uint32_t)r < count; r += 4) {
    const MoeMeta mm = meta[r];
    const uint4* yr = reinterpret_cast<const uint4*>(y + (size_t)r * row_bytes);
    for (int i = lane; i < row_bytes / 16; i += 32) {
      uint4 u = yr[i];
      uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = m.dtype == MACO_DT_BF16 ? unpack_bf16x2(w[j]) : __half22float2(*reinterpret_cast<__half2*>(&w[j]));
        f.x *= mm.weight; f.y *= mm.weight;
        if (m.dtype == MACO_DT_BF16) w[j] = pack_bf16x2(f.x, f.y);
        else { __half2 h = __floats2half2_rn(f.x, f.y); w[j] = *reinterpret_cast<uint32_t*>(&h); }
      }
      reinterpret_cast<uint4*>(srow)[i] = make_uint4(w[0], w[1], w[2], w[3]);
    }
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      bulk_store(p.peer_heap[src] + m.comb_off + ((size_t)mm.token * K + mm.k) * row_bytes, srow, row_bytes);
      tma_store_commit();
      tma_store_wait_read<0>();
    }
    __syncwarp();
  }
  if (lane == 0) tma_store_wait<0>();
}

}  // namespace maco
