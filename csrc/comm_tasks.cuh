// Communication tasks of the persistent kernel: copies and reductions over the symmetric heap.
//
// Every rank maps every other rank's heap (peer_heap[r]); a buffer allocated from the heap has
// the same offset on every rank. Tasks move 2-D blocks with 16-byte accesses issued by the
// worker's 128 general threads: stores into a peer's heap (push), loads from it (pull), and
// reductions in fp32. This is the in-kernel replacement for the torch.distributed call sites
// of the reference (all_reduce / all_gather / reduce_scatter / all_to_all, see
// maco/comm/patterns.py and maco/task_graph/runtime.py:211-226) and for its NVSHMEM kernels
// (maco/csrc/nvshmem_ops.cu:219-494), whose cross-CTA ordering relied on __syncthreads().
// Ordering here is carried by the task graph: a consumer task waits on an event that the
// producers bump with red.release.sys after their stores.
#pragma once
#include "elementwise.cuh"

namespace maco {

MACO_DEVICE void add8(float (&acc)[8], uint4 u, int dtype) {
  if (dtype == MACO_DT_F32) {
    acc[0] += __uint_as_float(u.x); acc[1] += __uint_as_float(u.y);
    acc[2] += __uint_as_float(u.z); acc[3] += __uint_as_float(u.w);
  } else if (dtype == MACO_DT_BF16) {
    float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
    acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y; acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
  } else {
    uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __half22float2(*reinterpret_cast<__half2*>(&w[i]));
      acc[2 * i] += f.x; acc[2 * i + 1] += f.y;
    }
  }
}

MACO_DEVICE uint4 pack8(const float (&acc)[8], float scale, int dtype) {
  uint4 o;
  if (dtype == MACO_DT_F32) {
    o.x = __float_as_uint(acc[0] * scale); o.y = __float_as_uint(acc[1] * scale);
    o.z = __float_as_uint(acc[2] * scale); o.w = __float_as_uint(acc[3] * scale);
  } else if (dtype == MACO_DT_BF16) {
    o.x = pack_bf16x2(acc[0] * scale, acc[1] * scale); o.y = pack_bf16x2(acc[2] * scale, acc[3] * scale);
    o.z = pack_bf16x2(acc[4] * scale, acc[5] * scale); o.w = pack_bf16x2(acc[6] * scale, acc[7] * scale);
  } else {
    __half2 h0 = __floats2half2_rn(acc[0] * scale, acc[1] * scale), h1 = __floats2half2_rn(acc[2] * scale, acc[3] * scale);
    __half2 h2 = __floats2half2_rn(acc[4] * scale, acc[5] * scale), h3 = __floats2half2_rn(acc[6] * scale, acc[7] * scale);
    o.x = *reinterpret_cast<uint32_t*>(&h0); o.y = *reinterpret_cast<uint32_t*>(&h1);
    o.z = *reinterpret_cast<uint32_t*>(&h2); o.w = *reinterpret_cast<uint32_t*>(&h3);
  }
  return o;
}

// Block geometry: `rows` rows of `row_bytes` (a multiple of 16) bytes. Every loop keeps kU
// independent 16-byte accesses per thread in flight: with 128 threads per task the copies are
// latency-bound otherwise.
constexpr int kU = 8;

// Data loads are plain (weak) 16-byte loads: ordering against the producer comes from the acquire
// on the task's event followed by the CTA barrier, so the compiler is free to batch them.
MACO_DEVICE uint4 ldv(const uint8_t* p) { return *reinterpret_cast<const uint4*>(p); }
// Explicit shared-memory vector accesses (32-bit shared addresses): no generic-address resolution, and the
// compiler knows they cannot alias global or local memory.
MACO_DEVICE uint4 lds128(uint32_t saddr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(saddr));
  return v;
}
MACO_DEVICE void sts128(uint32_t saddr, uint4 v) {
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" :: "r"(saddr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
MACO_DEVICE void stv(uint8_t* p, uint4 v) { *reinterpret_cast<uint4*>(p) = v; }

// Byte offset of 16-byte vector `i` of a block whose rows are `stride` bytes apart. 32-bit index
// arithmetic (64-bit division is emulated and would dominate the copy loops); rows that are packed
// back to back take the division-free path.
MACO_DEVICE uint64_t blk_off(uint32_t i, uint32_t vpr, uint64_t stride) {
  if (stride == ((uint64_t)vpr << 4)) return (uint64_t)i << 4;
  const uint32_t r = i / vpr;
  return (uint64_t)r * stride + ((uint64_t)(i - r * vpr) << 4);
}

// out = scale * (sum over n sources (+ aux)); kR vectors per thread per pass, loads of kS sources issued together.
template <int DTT, int kR, int kS, typename Program>
__device__ __noinline__ void comm_reduce(const Program& p, const MacoCommArgs& ar, int n, uint32_t total, uint32_t vpr, int tid,
                             int nthreads) {
  const MacoCommArgs a = ar;     // private copy: the descriptor lives in global memory and the loop stores could alias it
  uint8_t* mine = p.peer_heap[p.rank];
  const bool local = a.op == MACO_COMM_REDUCE_LOCAL || a.op == MACO_COMM_REDUCE_LOCAL_BCAST;
  uint8_t* out = a.local_ptr != nullptr ? reinterpret_cast<uint8_t*>(a.local_ptr) : mine + a.dst_off;
  const uint32_t rstep = (uint32_t)nthreads * kR;
  for (uint32_t base = tid; base < total; base += rstep) {
    float acc[kR][8];
#pragma unroll
    for (int u = 0; u < kR; ++u)
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[u][e] = 0.f;
    uint64_t soff[kR];
#pragma unroll
    for (int u = 0; u < kR; ++u) {
      const uint32_t i = base + (uint32_t)u * nthreads;
      soff[u] = blk_off(i < total ? i : 0, vpr, a.src_stride);
    }
    for (int j0 = 0; j0 < n; j0 += kS) {
      uint4 v[kS][kR];
#pragma unroll
      for (int jj = 0; jj < kS; ++jj) {
        const int j = j0 + jj;
        if (j < n) {
          const uint8_t* src = local ? mine + a.src_off + (uint64_t)j * a.slot_stride
                                     : p.peer_heap[(p.rank + j) % p.world] + a.src_off;
#pragma unroll
          for (int u = 0; u < kR; ++u) v[jj][u] = ldv(src + soff[u]);
        }
      }
#pragma unroll
      for (int jj = 0; jj < kS; ++jj) {
        if (j0 + jj < n) {
#pragma unroll
          for (int u = 0; u < kR; ++u) add8(acc[u], v[jj][u], DTT);
        }
      }
    }
    if (a.aux_ptr != nullptr) {
#pragma unroll
      for (int u = 0; u < kR; ++u) {
        const uint32_t i = base + (uint32_t)u * nthreads;
        if (i < total) add8(acc[u], ldv(reinterpret_cast<const uint8_t*>(a.aux_ptr) + blk_off(i, vpr, a.dst_stride)), DTT);
      }
    }
#pragma unroll
    for (int u = 0; u < kR; ++u) {
      const uint32_t i = base + (uint32_t)u * nthreads;
      if (i >= total) continue;
      const uint4 o = pack8(acc[u], a.scale, DTT);
      if (a.op == MACO_COMM_ALLREDUCE || a.op == MACO_COMM_REDUCE_LOCAL_BCAST) {
        for (int j = 0; j < p.world; ++j)
          stv(p.peer_heap[(p.rank + j) % p.world] + a.dst_off + blk_off(i, vpr, a.dst_stride), o);
      } else {
        stv(out + blk_off(i, vpr, a.dst_stride), o);
      }
    }
  }
}

// Shared-memory staging for bulk pushes: only offered on workers whose operand ring is idle
// (communication workers never receive GEMM tasks).
struct BulkCtx {
  uint8_t* buf;            // nbuf buffers of buf_bytes each (1024-byte aligned)
  uint64_t* bars;          // one mbarrier per buffer, initialised with count 1
  uint32_t nbuf, buf_bytes;
  volatile uint32_t* phase;  // shared word: bit b = parity the next wait on bars[b] uses (updated by the leader only)
};

// Contiguous push through the bulk-copy engine: one thread keeps nbuf * buf_bytes in flight
// (load rounds into shared memory, then one bulk store per destination), which is what it takes
// to fill an NVLink from a single SM; 128 threads with 16-byte accesses are latency-bound far below.
template <typename Program>
MACO_DEVICE bool comm_push_bulk(const Program& p, const MacoCommArgs& ar, BulkCtx& bc, uint64_t budget_ns) {
  const MacoCommArgs a = ar;     // private copy (the descriptor is in global memory)
  const uint64_t bytes = (uint64_t)a.rows * a.row_bytes;
  const uint8_t* src = p.peer_heap[p.rank] + a.src_off;
  fence_proxy_async_all();
  bool ok = true;
  // Ring over the staging buffers: the load of chunk i is issued kLead chunks before its store, and a buffer
  // is reloaded once the store that used it last has read it out (stores are committed one group per
  // chunk, so "at most nbuf - kLead - 1 newer groups still reading" is exactly that condition).
  constexpr uint32_t kRing = 12, kLead = 8;
  const uint32_t n_chunks = (uint32_t)((bytes + bc.buf_bytes - 1) / bc.buf_bytes);
  if (bc.nbuf == kRing) {
    for (uint32_t i = 0; i < n_chunks + kLead && ok; ++i) {
      if (i < n_chunks) {
        const uint32_t b = i % kRing;
        if (i >= kRing) tma_store_wait_read<kRing - kLead - 1>();
        const uint64_t off = (uint64_t)i * bc.buf_bytes;
        const uint32_t n = (uint32_t)(bytes - off < bc.buf_bytes ? bytes - off : bc.buf_bytes);
        mbar_arrive_expect_tx(&bc.bars[b], n);
        bulk_load(bc.buf + (size_t)b * bc.buf_bytes, src + off, n, &bc.bars[b]);
      }
      if (i >= kLead) {
        const uint32_t c = i - kLead, b = c % kRing;
        const uint64_t off = (uint64_t)c * bc.buf_bytes;
        const uint32_t n = (uint32_t)(bytes - off < bc.buf_bytes ? bytes - off : bc.buf_bytes);
        const uint32_t parity = (*bc.phase >> b) & 1u;
        const uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(&bc.bars[b], parity)) {
          if (globaltimer_ns() - t0 > budget_ns) { ok = false; break; }
        }
        *bc.phase = *bc.phase ^ (1u << b);
        if (!ok) break;
        const uint8_t* sm = bc.buf + (size_t)b * bc.buf_bytes;
        if (a.peer >= 0) {
          bulk_store(p.peer_heap[a.peer] + a.dst_off + off, sm, n);
        } else {
          for (int k = 0; k < p.world; ++k) {
            const int dr = (p.rank + 1 + k) % p.world;
            if (dr == p.rank && a.peer != -3) continue;
            bulk_store(p.peer_heap[dr] + a.dst_off + off, sm, n);
          }
        }
        tma_store_commit();
      }
    }
    if (!ok) {
      // loads that were issued and never waited for get a bounded time to land (their destination is this CTA's memory)
      for (uint32_t b = 0; b < kRing; ++b) {
        const uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(&bc.bars[b], (*bc.phase >> b) & 1u)) {
          if (globaltimer_ns() - t0 > 2000000ull) break;
        }
      }
    }
    tma_store_wait<0>();               // every store has completed before the task signals
    return ok;
  }
  for (uint64_t pos = 0; pos < bytes && ok; pos += (uint64_t)bc.nbuf * bc.buf_bytes) {
    uint32_t used = 0;
    for (uint32_t b = 0; b < bc.nbuf; ++b) {
      const uint64_t off = pos + (uint64_t)b * bc.buf_bytes;
      if (off >= bytes) break;
      const uint32_t n = (uint32_t)(bytes - off < bc.buf_bytes ? bytes - off : bc.buf_bytes);
      mbar_arrive_expect_tx(&bc.bars[b], n);
      bulk_load(bc.buf + (size_t)b * bc.buf_bytes, src + off, n, &bc.bars[b]);
      ++used;
    }
    for (uint32_t b = 0; b < used; ++b) {
      const uint64_t off = pos + (uint64_t)b * bc.buf_bytes;
      const uint32_t n = (uint32_t)(bytes - off < bc.buf_bytes ? bytes - off : bc.buf_bytes);
      const uint32_t parity = (*bc.phase >> b) & 1u;
      const uint64_t t0 = globaltimer_ns();
      while (!mbar_try_wait(&bc.bars[b], parity)) {
        if (globaltimer_ns() - t0 > budget_ns) { ok = false; break; }
      }
      *bc.phase = *bc.phase ^ (1u << b);
      if (!ok) break;
      const uint8_t* sm = bc.buf + (size_t)b * bc.buf_bytes;
      if (a.peer >= 0) {
        bulk_store(p.peer_heap[a.peer] + a.dst_off + off, sm, n);
      } else {
        for (int k = 0; k < p.world; ++k) {
          const int dr = (p.rank + 1 + k) % p.world;
          if (dr == p.rank && a.peer != -3) continue;
          bulk_store(p.peer_heap[dr] + a.dst_off + off, sm, n);
        }
      }
      tma_store_commit();
    }
    tma_store_wait_read<0>();          // the buffers may be refilled
  }
  tma_store_wait<0>();                 // every store has completed before the task signals
  return ok;
}

// Reduction with the sources staged through shared memory by the bulk-copy engine: the leader
// thread keeps up to nbuf * buf_bytes of loads in flight (local slots or peers' heaps), all
// threads sum the staged vectors in fp32 and write the result (to local memory with vector stores,
// or, for an all-reduce, back into shared memory from where one bulk store per rank sends it).
// `bar_sync` is the barrier of the calling thread group.
template <int DTT, typename Program, typename BarFn>
__device__ __noinline__ bool comm_reduce_bulk(const Program& p, const MacoCommArgs& ar, int n, int tid, int nthreads, BulkCtx& bcr,
                                  BarFn bar_sync) {
  // private copies: the descriptor lives in global memory; read in place, every use inside the summing loop
  // would be a fresh load (the loop's stores could alias it), about 500 cycles per vector
  const MacoCommArgs a = ar;
  const BulkCtx bc = bcr;
  uint8_t* mine = p.peer_heap[p.rank];
  const bool local = a.op == MACO_COMM_REDUCE_LOCAL || a.op == MACO_COMM_REDUCE_LOCAL_BCAST;
  const bool bcast = a.op == MACO_COMM_ALLREDUCE || a.op == MACO_COMM_REDUCE_LOCAL_BCAST;
  uint8_t* out = a.local_ptr != nullptr ? reinterpret_cast<uint8_t*>(a.local_ptr) : mine + a.dst_off;
  const uint64_t bytes = (uint64_t)a.rows * a.row_bytes;
  const uint32_t groups = bc.nbuf / (uint32_t)n;             // chunk positions that fit the staging buffers
  // Every chunk position is a pipeline stage of its own: while the threads sum one position, the loads of all
  // the others (and, for an all-reduce, the stores of earlier results) are in flight, so a round trip to a
  // peer (several microseconds) is covered by `groups - 1` stages of work.
  const uint64_t round_bytes = (uint64_t)groups * bc.buf_bytes;
  bool ok = true;
  bool have_prev = false;                                    // leader only: a position whose refill is still owed
  uint32_t prev_g = 0;
  uint64_t prev_pos = 0;
  // leader: loads of position g for the round that starts at byte `pos`
  auto issue = [&](uint32_t g, uint64_t pos) {
    const uint64_t off = pos + (uint64_t)g * bc.buf_bytes;
    if (off >= bytes) return;
    const uint32_t nb = (uint32_t)(bytes - off < bc.buf_bytes ? bytes - off : bc.buf_bytes);
    for (int j = 0; j < n; ++j) {
      const uint32_t b = g * n + j;
      const uint8_t* src = local ? mine + a.src_off + (uint64_t)j * a.slot_stride
                                 : p.peer_heap[(p.rank + j) % p.world] + a.src_off;
      mbar_arrive_expect_tx(&bc.bars[b], nb);
      bulk_load(bc.buf + (size_t)b * bc.buf_bytes, src + off, nb, &bc.bars[b]);
    }
  };
  // everybody: wait for position g of the round at `pos`, sum, write (or stage) the result; then the leader
  // sends the staged result (all-reduce) and refills the position for the next round
  auto consume = [&](uint32_t g, uint64_t pos) {
    const uint64_t off = pos + (uint64_t)g * bc.buf_bytes;
    if (off >= bytes) return;                                // uniform over the thread group
    const uint32_t nb = (uint32_t)(bytes - off < bc.buf_bytes ? bytes - off : bc.buf_bytes);
    const uint32_t phase = *bc.phase;                        // this position's bits change only after the barrier below
    uint32_t used_mask = 0;
    for (int j = 0; j < n; ++j) {
      const uint32_t b = g * n + j;
      used_mask |= 1u << b;
      const uint64_t t0 = globaltimer_ns();
      while (!mbar_try_wait(&bc.bars[b], (phase >> b) & 1u)) {
        if (globaltimer_ns() - t0 > p.budget_ns) { ok = false; break; }
      }
    }
    // Everything the loop needs sits in plain locals: the lambda reaches `a` and `bc` through its closure, i.e.
    // through memory, and every store of the loop (a generic address) would force them to be read again.
    const uint32_t g0s = smem_u32(bc.buf + (size_t)(g * n) * bc.buf_bytes), bufb = bc.buf_bytes, nvec = nb >> 4;
    const int nn = n;
    const float scale = a.scale;
    const uint8_t* aux = a.aux_ptr != nullptr ? reinterpret_cast<const uint8_t*>(a.aux_ptr) + off : nullptr;
    uint8_t* outp = out + off;
    for (uint32_t v = tid; v < nvec; v += nthreads) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int j = 0; j < nn; ++j) add8(acc, lds128(g0s + (uint32_t)j * bufb + (v << 4)), DTT);
      if (aux != nullptr) add8(acc, ldv(aux + ((uint64_t)v << 4)), DTT);
      const uint4 o = pack8(acc, scale, DTT);
      if (bcast) sts128(g0s + (v << 4), o);                                  // result replaces source 0 in shared memory
      else stv(outp + ((uint64_t)v << 4), o);
    }
    uint8_t* g0 = bc.buf + (size_t)(g * n) * bc.buf_bytes;
    if (bcast) fence_proxy_async_smem();
    bar_sync();                                              // the position is consumed (and its result staged)
    if (tid == 0) {
      // only this position's bits change; the bits of other positions, which threads may be reading, keep their value
      *bc.phase = *bc.phase ^ used_mask;
      if (bcast && groups >= 2) {
        for (int j = 0; j < p.world; ++j)
          bulk_store(p.peer_heap[(p.rank + j) % p.world] + a.dst_off + off, g0, nb);
        tma_store_commit();
        // The stores just issued may still be reading shared memory (a store into a peer is paced by the link):
        // do not wait for them. Wait for the PREVIOUS position's stores instead, which had a whole stage to
        // finish, and refill that position; this one is refilled one stage later.
        tma_store_wait_read<1>();
        if (have_prev) issue(prev_g, prev_pos + round_bytes);
        have_prev = true; prev_g = g; prev_pos = pos;
      } else {
        if (bcast) {
          for (int j = 0; j < p.world; ++j)
            bulk_store(p.peer_heap[(p.rank + j) % p.world] + a.dst_off + off, g0, nb);
          tma_store_commit();
          tma_store_wait_read<0>();                          // the staged result has left shared memory
        }
        issue(g, pos + round_bytes);
      }
    }
    if (groups == 1) bar_sync();                             // a single position: its phase bits are read again right away
  };
  if (tid == 0) {
    fence_proxy_async_all();
    for (uint32_t g = 0; g < groups; ++g) issue(g, 0);
  }
  for (uint64_t pos = 0; pos < bytes; pos += round_bytes)
    for (uint32_t g = 0; g < groups; ++g) consume(g, pos);
  bar_sync();                                                // the last phase word is visible to the next task
  if (tid == 0 && bcast) tma_store_wait<0>();
  return ok;
}

template <typename Program>
MACO_DEVICE bool comm_run(const Program& p, const MacoTaskDesc& d, int tid, int nthreads, BulkCtx* bulk = nullptr) {
  const MacoCommArgs& a = d.u.comm;
  if (bulk != nullptr && a.op == MACO_COMM_PUSH && a.src_stride == a.row_bytes && a.dst_stride == a.row_bytes &&
      (uint64_t)a.rows * a.row_bytes >= 65536) {
    bool ok = true;
    if (tid == 0) ok = comm_push_bulk(p, a, *bulk, p.budget_ns);
    return ok;
  }
  if (bulk != nullptr && (a.op == MACO_COMM_REDUCE_LOCAL || a.op == MACO_COMM_REDUCE_PULL || a.op == MACO_COMM_ALLREDUCE ||
                          a.op == MACO_COMM_REDUCE_LOCAL_BCAST) &&
      a.src_stride == a.row_bytes && a.dst_stride == a.row_bytes && (uint64_t)a.rows * a.row_bytes >= 32768) {
    const int n = (a.op == MACO_COMM_REDUCE_LOCAL || a.op == MACO_COMM_REDUCE_LOCAL_BCAST) ? a.nslots : p.world;
    if (n >= 1 && (uint32_t)n <= bulk->nbuf) {
      auto bar = [] { asm volatile("bar.sync 1, 128;" ::: "memory"); };
      if (a.dtype == MACO_DT_F32) return comm_reduce_bulk<MACO_DT_F32>(p, a, n, tid, nthreads, *bulk, bar);
      if (a.dtype == MACO_DT_F16) return comm_reduce_bulk<MACO_DT_F16>(p, a, n, tid, nthreads, *bulk, bar);
      return comm_reduce_bulk<MACO_DT_BF16>(p, a, n, tid, nthreads, *bulk, bar);
    }
  }
  const uint32_t vpr = a.row_bytes >> 4;                     // 16-byte vectors per row
  const uint32_t total = a.rows * vpr;                      // blocks are far below 2^32 vectors
  uint8_t* mine = p.peer_heap[p.rank];
  const uint32_t step = (uint32_t)nthreads * kU;
  switch (a.op) {
    case MACO_COMM_PUSH:
    case MACO_COMM_PULL: {
      // Read each vector once, store it to every destination: the block leaves this GPU once per peer.
      const uint8_t* src = (a.op == MACO_COMM_PULL ? p.peer_heap[a.peer] : mine) + a.src_off;
      for (uint32_t base = tid; base < total; base += step) {
        uint4 v[kU];
#pragma unroll
        for (int u = 0; u < kU; ++u) {
          const uint32_t i = base + (uint32_t)u * nthreads;
          if (i < total) v[u] = ldv(src + blk_off(i, vpr, a.src_stride));
        }
        if (a.op == MACO_COMM_PULL || a.peer >= 0) {
          uint8_t* dst = (a.op == MACO_COMM_PULL ? mine : p.peer_heap[a.peer]) + a.dst_off;
#pragma unroll
          for (int u = 0; u < kU; ++u) {
            const uint32_t i = base + (uint32_t)u * nthreads;
            if (i < total) stv(dst + blk_off(i, vpr, a.dst_stride), v[u]);
          }
        } else {
          for (int k = 0; k < p.world; ++k) {
            const int dr = (p.rank + 1 + k) % p.world;        // staggered so peers are not hit in lockstep
            if (dr == p.rank && a.peer != -3) continue;
            uint8_t* dst = p.peer_heap[dr] + a.dst_off;
#pragma unroll
            for (int u = 0; u < kU; ++u) {
              const uint32_t i = base + (uint32_t)u * nthreads;
              if (i < total) stv(dst + blk_off(i, vpr, a.dst_stride), v[u]);
            }
          }
        }
      }
      return true;
    }
    case MACO_COMM_REDUCE_LOCAL:
    case MACO_COMM_REDUCE_LOCAL_BCAST:
    case MACO_COMM_REDUCE_PULL:
    case MACO_COMM_ALLREDUCE: {
      const int n = (a.op == MACO_COMM_REDUCE_LOCAL || a.op == MACO_COMM_REDUCE_LOCAL_BCAST) ? a.nslots : p.world;
      // 8 independent 16-byte loads per thread in flight whatever the number of sources (more spills registers)
#define MACO_REDUCE_DT(DT)                                                         \
      if (n <= 2) comm_reduce<DT, 4, 2>(p, a, n, total, vpr, tid, nthreads);       \
      else if (n <= 4) comm_reduce<DT, 2, 4>(p, a, n, total, vpr, tid, nthreads);  \
      else comm_reduce<DT, 2, 8>(p, a, n, total, vpr, tid, nthreads);
      if (a.dtype == MACO_DT_F32) { MACO_REDUCE_DT(MACO_DT_F32) }
      else if (a.dtype == MACO_DT_F16) { MACO_REDUCE_DT(MACO_DT_F16) }
      else { MACO_REDUCE_DT(MACO_DT_BF16) }
#undef MACO_REDUCE_DT
      return true;
    }
    case MACO_COMM_PUSH_MC: {
      // Broadcast: every 16-byte vector is read once from this rank's heap and stored once to the multicast
      // address; the switch delivers it to every rank (this one included), so the block leaves the GPU once
      // whatever the number of peers.
      if (p.mc_heap == nullptr) return false;
      const uint8_t* src = mine + a.src_off;
      uint8_t* dst = p.mc_heap + a.dst_off;
      for (uint32_t base = tid; base < total; base += step) {
        uint4 v[kU];
#pragma unroll
        for (int u = 0; u < kU; ++u) {
          const uint32_t i = base + (uint32_t)u * nthreads;
          if (i < total) v[u] = ldv(src + blk_off(i, vpr, a.src_stride));
        }
#pragma unroll
        for (int u = 0; u < kU; ++u) {
          const uint32_t i = base + (uint32_t)u * nthreads;
          if (i < total) {
            if (a.nslots == 1) multimem_st_v4_weak(dst + blk_off(i, vpr, a.dst_stride), v[u]);
            else multimem_st_v4(dst + blk_off(i, vpr, a.dst_stride), v[u]);
          }
        }
      }
      return true;
    }
    case MACO_COMM_ALLREDUCE_MC: {
      // One-shot all-reduce of a block through the switch: multimem.ld_reduce returns the sum over every rank's
      // copy (accumulated in fp32 inside the switch for 16-bit types), multimem.st writes the result back to
      // every copy. kU loads per thread are in flight together: one round trip through the switch is a few
      // microseconds.
      if (p.mc_heap == nullptr) return false;
      const uint8_t* src = p.mc_heap + a.src_off;
      uint8_t* dst = p.mc_heap + a.dst_off;
      for (uint32_t base = tid; base < total; base += step) {
        uint4 v[kU];
#pragma unroll
        for (int u = 0; u < kU; ++u) {
          const uint32_t i = base + (uint32_t)u * nthreads;
          if (i >= total) continue;
          const uint8_t* q = src + blk_off(i, vpr, a.src_stride);
          if (a.dtype == MACO_DT_F32) {
            const float4 f = multimem_ld_reduce_f32x4(q);
            v[u] = make_uint4(__float_as_uint(f.x), __float_as_uint(f.y), __float_as_uint(f.z), __float_as_uint(f.w));
          } else if (a.dtype == MACO_DT_F16) {
            v[u] = multimem_ld_reduce_f16x8(q);
          } else {
            v[u] = multimem_ld_reduce_bf16x8(q);
          }
        }
#pragma unroll
        for (int u = 0; u < kU; ++u) {
          const uint32_t i = base + (uint32_t)u * nthreads;
          if (i >= total) continue;
          uint4 o = v[u];
          if (a.scale != 1.f) {
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            add8(acc, o, a.dtype);
            o = a.dtype == MACO_DT_F32 ? pack8(acc, a.scale, MACO_DT_F32)
              : a.dtype == MACO_DT_F16 ? pack8(acc, a.scale, MACO_DT_F16) : pack8(acc, a.scale, MACO_DT_BF16);
          }
          multimem_st_v4(dst + blk_off(i, vpr, a.dst_stride), o);
        }
      }
      return true;
    }
    default: return false;
  }
}

}  // namespace maco
