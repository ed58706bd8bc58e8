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

// Block geometry: `rows` rows of `row_bytes` (a multiple of 16) bytes.
template <typename Program>
MACO_DEVICE bool comm_run(const Program& p, const MacoTaskDesc& d, int tid, int nthreads) {
  const MacoCommArgs& a = d.u.comm;
  const uint32_t vpr = a.row_bytes >> 4;                     // 16-byte vectors per row
  const uint64_t total = (uint64_t)a.rows * vpr;
  uint8_t* mine = p.peer_heap[p.rank];
  switch (a.op) {
    case MACO_COMM_PUSH: {
      // Read each vector once, store it to every destination: the block leaves this GPU once per peer.
      for (uint64_t i = tid; i < total; i += nthreads) {
        const uint64_t r = i / vpr, c = (i % vpr) << 4;
        const uint4 v = ld_global_v4(mine + a.src_off + r * a.src_stride + c);
        const uint64_t doff = a.dst_off + r * a.dst_stride + c;
        if (a.peer >= 0) {
          st_global_v4(p.peer_heap[a.peer] + doff, v);
        } else {
          for (int k = 0; k < p.world; ++k) {
            const int dst = (p.rank + 1 + k) % p.world;       // staggered so peers are not hit in lockstep
            if (dst == p.rank && a.peer != -3) continue;
            st_global_v4(p.peer_heap[dst] + doff, v);
          }
        }
      }
      return true;
    }
    case MACO_COMM_PULL: {
      const uint8_t* src = p.peer_heap[a.peer];
      for (uint64_t i = tid; i < total; i += nthreads) {
        const uint64_t r = i / vpr, c = (i % vpr) << 4;
        st_global_v4(mine + a.dst_off + r * a.dst_stride + c, ld_global_v4(src + a.src_off + r * a.src_stride + c));
      }
      return true;
    }
    case MACO_COMM_REDUCE_LOCAL:
    case MACO_COMM_REDUCE_PULL: {
      const bool pull = a.op == MACO_COMM_REDUCE_PULL;
      const int n = pull ? p.world : a.nslots;
      uint8_t* out = a.local_ptr != nullptr ? reinterpret_cast<uint8_t*>(a.local_ptr) : mine + a.dst_off;
      const bool f32 = a.dtype == MACO_DT_F32;
      for (uint64_t i = tid; i < total; i += nthreads) {
        const uint64_t r = i / vpr, c = (i % vpr) << 4;
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int j = 0; j < n; ++j) {
          const uint8_t* src = pull ? p.peer_heap[(p.rank + j) % p.world] + a.src_off
                                    : mine + a.src_off + (uint64_t)j * a.slot_stride;
          add8(acc, ld_global_v4(src + r * a.src_stride + c), a.dtype);
        }
        (void)f32;
        st_global_v4(out + r * a.dst_stride + c, pack8(acc, a.scale, a.dtype));
      }
      return true;
    }
    case MACO_COMM_ALLREDUCE: {
      for (uint64_t i = tid; i < total; i += nthreads) {
        const uint64_t r = i / vpr, c = (i % vpr) << 4;
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int j = 0; j < p.world; ++j)
          add8(acc, ld_global_v4(p.peer_heap[(p.rank + j) % p.world] + a.src_off + r * a.src_stride + c), a.dtype);
        const uint4 o = pack8(acc, a.scale, a.dtype);
        for (int j = 0; j < p.world; ++j)
          st_global_v4(p.peer_heap[(p.rank + j) % p.world] + a.dst_off + r * a.dst_stride + c, o);
      }
      return true;
    }
    case MACO_COMM_ALLREDUCE_MC: {
      if (p.mc_heap == nullptr) return false;
      for (uint64_t i = tid; i < total; i += nthreads) {
        const uint64_t r = i / vpr, c = (i % vpr) << 4;
        const uint8_t* src = p.mc_heap + a.src_off + r * a.src_stride + c;
        uint4 o;
        if (a.dtype == MACO_DT_F32) {
          float4 f = multimem_ld_reduce_f32x4(src);
          o = make_uint4(__float_as_uint(f.x * a.scale), __float_as_uint(f.y * a.scale), __float_as_uint(f.z * a.scale),
                         __float_as_uint(f.w * a.scale));
        } else {
          o = multimem_ld_reduce_bf16x8(src);
          if (a.scale != 1.f) {
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            add8(acc, o, MACO_DT_BF16);
            o = pack8(acc, a.scale, MACO_DT_BF16);
          }
        }
        multimem_st_v4(p.mc_heap + a.dst_off + r * a.dst_stride + c, o);
      }
      return true;
    }
    default: return false;
  }
}

}  // namespace maco
