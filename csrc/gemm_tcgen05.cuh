// Warp-specialised tcgen05 GEMM pipeline for sm_100a.
//
//   D[M,N] = epilogue( A[M,K] · B[N,K]^T )      A, B: bf16 or fp16;  accumulate fp32 in TMEM
//
// This replaces the reference's scalar one-thread-per-output GEMM task
// (maco/csrc/maco_worker.cuh:36-57) and the torch.mm call its live runtime makes
// (maco/task_graph/runtime.py:188-209).
//
// One CTA = 6 warps:
//   warp 0      TMA producer   cp.async.bulk.tensor tiles -> 128B-swizzled smem ring
//   warp 1      MMA issuer     one lane issues tcgen05.mma (128 x BN x 16) into a TMEM accumulator
//   warps 2..5  epilogue       tcgen05.ld the accumulator (one TMEM lane quarter per warp),
//                              apply the fused epilogue, store to global (local or peer memory)
// The accumulator is double buffered in TMEM (2 x BN columns) so the epilogue of tile i runs
// under the main loop of tile i+1. All hand-offs are mbarriers; every wait is bounded and a
// wait that runs out sets a CTA-wide abort word, after which all roles drain and the CTA frees
// its TMEM and returns.
//
// Operands may be K-major (row-major [rows, K]) or MN-major (row-major [K, rows]); the latter is
// what the backward GEMMs need (wgrad = dY^T · X contracts over the token dimension).
#pragma once
#include <cuda.h>
#include "maco_atoms.cuh"
#include "maco_types.h"

namespace maco {

constexpr int kBM = 128;       // tile rows  (UMMA M)
constexpr int kBK = 64;        // k-block: 64 x 2 B = one 128-byte swizzle row
constexpr int kUmmaK = 16;     // K per tcgen05.mma for 16-bit inputs
constexpr int kGemmThreads = 192;

// BN is the tile width a task uses; SBN (>= BN) sizes the ring's stages, so tasks of different
// BN can share one ring with identical stage addresses and barrier phases.
template <int BN, int STAGES, int SBN = BN>
struct GemmSmemLayout {
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = BN * kBK * 2;
  static constexpr int kLoadBytes = kABytes + kBBytes;          // bytes one k-step brings in
  static constexpr int kStageBytes = kABytes + SBN * kBK * 2;   // distance between stages
  static constexpr int kRingBytes = STAGES * kStageBytes;
  // after the ring: full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], tmem slot, abort word
  static constexpr int kCtrlBytes = 256;
  static constexpr int kTotalBytes = kRingBytes + kCtrlBytes + 1024;   // +1024: manual alignment slack
  static_assert(2 * STAGES * 8 + 4 * 8 + 16 <= kCtrlBytes, "control block too small");
};

struct GemmCtrl {
  uint64_t* full;        // [STAGES]  TMA -> MMA
  uint64_t* empty;       // [STAGES]  MMA -> TMA
  uint64_t* tmem_full;   // [2]       MMA -> epilogue
  uint64_t* tmem_empty;  // [2]       epilogue -> MMA
  uint32_t* tmem_slot;
  volatile uint32_t* abort_word;
};

template <int BN, int STAGES, int SBN = BN>
MACO_DEVICE GemmCtrl gemm_ctrl(uint8_t* smem_base) {
  using L = GemmSmemLayout<BN, STAGES, SBN>;
  GemmCtrl c;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_base + L::kRingBytes);
  c.full = bars;
  c.empty = bars + STAGES;
  c.tmem_full = bars + 2 * STAGES;
  c.tmem_empty = bars + 2 * STAGES + 2;
  c.tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  c.abort_word = reinterpret_cast<volatile uint32_t*>(c.tmem_slot + 1);
  return c;
}

// Raster order: groups of 8 tile-rows sweep all tile-columns, so CTAs that run together
// share A row-blocks and B column-blocks in L2.
MACO_DEVICE void gemm_tile_coords(int tile, int m_tiles, int n_tiles, int& m_blk, int& n_blk) {
  const int G = 8;
  int per_group = G * n_tiles;
  int g = tile / per_group;
  int first_m = g * G;
  int gsize = min(G, m_tiles - first_m);
  int r = tile - g * per_group;
  m_blk = first_m + r % gsize;
  n_blk = r / gsize;
}

// ---- producer ------------------------------------------------------------------------------
// Loads one (128 x 64) A block and one (BN x 64) B block per k-step. K-major operands take one
// box; MN-major operands take one 64-wide box per 64 rows (each box is a 64x64 swizzle panel).
template <int BN, int STAGES, bool A_MN, bool B_MN, int SBN = BN>
MACO_DEVICE bool gemm_produce_tile(uint8_t* smem, const GemmCtrl& c, const CUtensorMap* tmA,
                                   const CUtensorMap* tmB, int m0, int n0, int k0, int k_blocks,
                                   uint32_t& it, uint64_t budget_ns, long long* prof = nullptr, int k_step = kBK,
                                   int b_blocked_row0 = -1) {
  // b_blocked_row0 >= 0: B is stored tile by tile ([N / BN][K / 64][BN][64], see ops.block_weight) and its tensor map
  // is the 2-D view [rows, 64]; k-block kb of this tile is the contiguous BN x 64 block at row b_blocked_row0 + kb * BN.
  // (A K-major [N, K] weight read once from HBM comes in as BN separate 128-byte pieces per box, one per DRAM
  // page; the blocked form streams at the rate of a plain copy.)
  // k_step: elements per 128-byte k-block (64 for 16-bit operands, 32 for fp32 operands run as TF32)
  using L = GemmSmemLayout<BN, STAGES, SBN>;
  // stage index and phase advance incrementally: the loop is one thread's instruction stream, and a division
  // per k-block is a measurable part of it
  uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
  uint8_t* sa = smem + s * L::kStageBytes;
  int k = k0;
  for (int kb = 0; kb < k_blocks; ++kb, k += k_step) {
    const long long t0 = prof ? clock64() : 0;
    if (!mbar_wait(&c.empty[s], ph ^ 1, budget_ns, c.abort_word)) { it += kb; return false; }
    if (prof) prof[0] += clock64() - t0;
    uint8_t* sb = sa + L::kABytes;
    mbar_arrive_expect_tx(&c.full[s], L::kLoadBytes);
    if constexpr (!A_MN) {
      tma_load_2d(sa, tmA, &c.full[s], k, m0);
    } else {
#pragma unroll
      for (int j = 0; j < kBM / 64; ++j) tma_load_2d(sa + j * 8192, tmA, &c.full[s], m0 + j * 64, k);
    }
    if constexpr (!B_MN) {
      if (b_blocked_row0 >= 0) tma_load_2d(sb, tmB, &c.full[s], 0, b_blocked_row0 + kb * BN);
      else tma_load_2d(sb, tmB, &c.full[s], k, n0);
    } else {
#pragma unroll
      for (int j = 0; j < BN / 64; ++j) tma_load_2d(sb + j * 8192, tmB, &c.full[s], n0 + j * 64, k);
    }
    if (++s == STAGES) { s = 0; ph ^= 1; sa = smem; } else { sa += L::kStageBytes; }
  }
  it += k_blocks;
  return true;
}

// After an abort: give loads that are still in flight a bounded time to land before the CTA
// leaves (their destination is this CTA's shared memory).
template <int STAGES>
MACO_DEVICE void gemm_drain_loads(const GemmCtrl& c, uint32_t issued) {
  uint32_t first = issued > STAGES ? issued - STAGES : 0;
  for (uint32_t i = first; i < issued; ++i) {
    uint64_t t0 = globaltimer_ns();
    while (!mbar_try_wait(&c.full[i % STAGES], (i / STAGES) & 1)) {
      if (globaltimer_ns() - t0 > 2000000ull) break;
    }
  }
}

// ---- MMA issuer ----------------------------------------------------------------------------
template <int BN, int STAGES, bool A_MN, bool B_MN, int SBN = BN, bool TF32 = false>
MACO_DEVICE bool gemm_mma_tile(uint8_t* smem, const GemmCtrl& c, uint32_t tmem_base, uint32_t idesc,
                               int k_blocks, uint32_t& it, uint32_t tile_seq, uint64_t budget_ns,
                               long long* prof = nullptr) {
  using L = GemmSmemLayout<BN, STAGES, SBN>;
  const uint32_t acc = tile_seq & 1, acc_ph = (tile_seq >> 1) & 1;
  long long t0 = prof ? clock64() : 0;
  if (!mbar_wait(&c.tmem_empty[acc], acc_ph ^ 1, budget_ns, c.abort_word)) return false;
  if (prof) prof[1] += clock64() - t0;
  tc_fence_after();
  const uint32_t d_tmem = tmem_base + acc * SBN;
  // K-major: 8-row groups are 1024 B apart (SBO); a K step of 16 elements is 32 B inside the swizzled row.
  // MN-major: 64-row panels are 8192 B apart (LBO), 8-k groups 1024 B apart (SBO); a K step of 16 is two groups
  // = 2048 B. The descriptors' high words are constant; the low word is the start address in 16-byte units.
  const uint64_t da0 = A_MN ? make_smem_desc(0, 8192, 1024, 2) : make_smem_desc(0, 16, 1024, 2);
  const uint64_t db0 = B_MN ? make_smem_desc(0, 8192, 1024, 2) : make_smem_desc(0, 16, 1024, 2);
  const uint32_t a_hi = (uint32_t)(da0 >> 32), b_hi = (uint32_t)(db0 >> 32);
  const uint32_t a_lbo = (uint32_t)da0, b_lbo = (uint32_t)db0;          // leading-dimension offset field (bits 16-29)
  constexpr uint32_t kStepA = (A_MN ? 2048 : 32) >> 4, kStepB = (B_MN ? 2048 : 32) >> 4;
  constexpr uint32_t kStage16 = L::kStageBytes >> 4, kAB16 = L::kABytes >> 4;
  const uint32_t base_lo = (smem_u32(smem) & 0x3FFFFu) >> 4;
  uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
  uint32_t a_lo = base_lo + s * kStage16;
  uint32_t accum = 0;
  for (int kb = 0; kb < k_blocks; ++kb) {
    if (prof) t0 = clock64();
    if (!mbar_wait(&c.full[s], ph, budget_ns, c.abort_word)) { it += kb; return false; }
    if (prof) prof[2] += clock64() - t0;
    const uint32_t b_lo = a_lo + kAB16;
#pragma unroll
    for (int k = 0; k < kBK / kUmmaK; ++k) {
      // low descriptor words: start address (bits 0-13, never carries: shared memory is below 256 KB) | leading offset
      // fp32 operands (TF32): 8 elements of 4 bytes per MMA, the same 32-byte step inside the swizzled row
      if constexpr (TF32) tc_mma_tf32_lo(d_tmem, (a_lo + k * kStepA) | a_lbo, a_hi, (b_lo + k * kStepB) | b_lbo, b_hi, idesc, accum);
      else tc_mma_f16_lo(d_tmem, (a_lo + k * kStepA) | a_lbo, a_hi, (b_lo + k * kStepB) | b_lbo, b_hi, idesc, accum);
      accum = 1;
    }
    tc_commit(&c.empty[s]);          // frees the smem stage once these MMAs have read it
    if (++s == STAGES) { s = 0; ph ^= 1; a_lo = base_lo; } else { a_lo += kStage16; }
  }
  it += k_blocks;
  tc_commit(&c.tmem_full[acc]);      // accumulator complete -> epilogue
  return true;
}

// ---- epilogue ------------------------------------------------------------------------------
MACO_DEVICE float epi_bias(const GemmEpilogue& e, int col) {
  if (e.bias == nullptr) return 0.f;
  if (e.bias_type == MACO_DT_F32) return reinterpret_cast<const float*>(e.bias)[col];
  if (e.bias_type == MACO_DT_F16) return __half2float(reinterpret_cast<const __half*>(e.bias)[col]);
  return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(e.bias)[col]);
}

MACO_DEVICE uint32_t epi_pack(int out_type, float a, float b) {
  if (out_type == MACO_DT_F16) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  return pack_bf16x2(a, b);
}

// Stores 32 consecutive columns of one row. `v` holds fp32 values already transformed.
MACO_DEVICE void epi_store_row32(const GemmEpilogue& e, void* out_base, long long row, int col0,
                                 int ncols_valid, const float (&v)[32]) {
  if (e.out_type == MACO_DT_F32) {
    float* p = reinterpret_cast<float*>(out_base) + row * e.ld_out + col0;
    if (e.mode == MACO_EPI_F32_ATOMIC || e.mode == MACO_EPI_SPLITK_FUSED) {
      // split-K: several tiles add into the same fp32 block; vector reductions at the L2
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        if (j + 4 <= ncols_valid) {
          asm volatile("red.relaxed.gpu.global.add.v4.f32 [%0], {%1, %2, %3, %4};"
                       :: "l"(p + j), "f"(v[j]), "f"(v[j + 1]), "f"(v[j + 2]), "f"(v[j + 3]) : "memory");
        } else {
          for (int t = j; t < ncols_valid && t < j + 4; ++t) atomicAdd(p + t, v[t]);
        }
      }
    } else if (e.mode == MACO_EPI_F32_ACC) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        if (j + 4 <= ncols_valid) {
          float4 o = *reinterpret_cast<float4*>(p + j);
          o.x += v[j]; o.y += v[j + 1]; o.z += v[j + 2]; o.w += v[j + 3];
          *reinterpret_cast<float4*>(p + j) = o;
        } else {
          for (int t = j; t < ncols_valid && t < j + 4; ++t) p[t] += v[t];
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        if (j + 4 <= ncols_valid) {
          *reinterpret_cast<float4*>(p + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        } else {
          for (int t = j; t < ncols_valid && t < j + 4; ++t) p[t] = v[t];
        }
      }
    }
  } else {
    uint16_t* p = reinterpret_cast<uint16_t*>(out_base) + row * e.ld_out + col0;
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
      if (j + 8 <= ncols_valid) {
        uint4 o;
        o.x = epi_pack(e.out_type, v[j], v[j + 1]);
        o.y = epi_pack(e.out_type, v[j + 2], v[j + 3]);
        o.z = epi_pack(e.out_type, v[j + 4], v[j + 5]);
        o.w = epi_pack(e.out_type, v[j + 6], v[j + 7]);
        *reinterpret_cast<uint4*>(p + j) = o;
      } else {
        for (int t = j; t < ncols_valid && t < j + 8; ++t) {
          uint32_t w = epi_pack(e.out_type, v[t], 0.f);
          p[t] = (uint16_t)(w & 0xffffu);
        }
      }
    }
  }
}

MACO_DEVICE float epi_load_aux(const GemmEpilogue& e, long long row, int col) {
  const uint16_t* p = reinterpret_cast<const uint16_t*>(e.aux) + row * e.ld_aux + col;
  if (e.aux_type == MACO_DT_F16) return __half2float(*reinterpret_cast<const __half*>(p));
  return __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(p));
}

// The 32 aux values beside one row's 32-column chunk: four 16-byte loads issued together when the chunk is
// whole and aligned (one 2-byte load per element otherwise). Values past `valid` are 0.
MACO_DEVICE void epi_load_aux32(const GemmEpilogue& e, long long row, int col0, int valid, float (&a)[32]) {
  const uint16_t* p = reinterpret_cast<const uint16_t*>(e.aux) + row * e.ld_aux + col0;
  if (valid == 32 && (reinterpret_cast<uintptr_t>(p) & 15) == 0) {
    uint4 q[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) q[i] = reinterpret_cast<const uint4*>(p)[i];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t w[4] = {q[i].x, q[i].y, q[i].z, q[i].w};
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float2 f = e.aux_type == MACO_DT_F16 ? __half22float2(*reinterpret_cast<const __half2*>(&w[t])) : unpack_bf16x2(w[t]);
        a[i * 8 + 2 * t] = f.x; a[i * 8 + 2 * t + 1] = f.y;
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) a[j] = j < valid ? epi_load_aux(e, row, col0 + j) : 0.f;
  }
}

// Consumes one finished accumulator. Called by all 32 lanes of each of the 4 epilogue warps.
// `out_base` lets a caller redirect the tile (for example into a peer GPU's buffer);
// `row_off` is added to the tile's row index when storing (for scatter into per-rank slabs).
// Staged stores: tiles that leave the GPU (a peer's heap) are first written to shared memory and
// then sent as one 128-byte bulk copy per row and 64-column group. Per-thread 16-byte stores to
// peer memory reach only a small fraction of NVLink bandwidth; the bulk engine writes full lines.
constexpr int kEpiStageRowBytes = 144;                       // 128 bytes of data + 16 of padding (bank spread)
constexpr int kEpiStageWarpBytes = 32 * kEpiStageRowBytes;   // one epilogue warp: 32 rows
constexpr int kEpiStageBytes = 4 * kEpiStageWarpBytes;

MACO_DEVICE void epi_stage_chunk(uint8_t* srow, int half, int out_type, const float (&v)[32]) {
  uint4* dst = reinterpret_cast<uint4*>(srow + half * 64);
#pragma unroll
  for (int j = 0; j < 32; j += 8) {
    uint4 o;
    o.x = epi_pack(out_type, v[j], v[j + 1]); o.y = epi_pack(out_type, v[j + 2], v[j + 3]);
    o.z = epi_pack(out_type, v[j + 4], v[j + 5]); o.w = epi_pack(out_type, v[j + 6], v[j + 7]);
    dst[j >> 3] = o;
  }
}

MACO_DEVICE void epi_stage_chunk_f32(uint8_t* srow, const float (&v)[32]) {
  uint4* dst = reinterpret_cast<uint4*>(srow);
#pragma unroll
  for (int j = 0; j < 32; j += 4)
    dst[j >> 2] = make_uint4(__float_as_uint(v[j]), __float_as_uint(v[j + 1]), __float_as_uint(v[j + 2]), __float_as_uint(v[j + 3]));
}

// Extra destinations of a tile: the same values are also stored at bases[k] + off for k < n
// (used to broadcast a partial result into every rank's staging slot).
struct EpiBroadcast {
  int n;
  uint8_t* const* bases;
  unsigned long long off;
};

template <int BN, int SBN = BN>
MACO_DEVICE bool gemm_epilogue_tile(const GemmCtrl& c, uint32_t tmem_base, const GemmEpilogue& e_in,
                                    void* out_base, long long row_off, int m0, int n0,
                                    uint32_t tile_seq, uint64_t budget_ns, const EpiBroadcast* bc = nullptr,
                                    uint8_t* stage = nullptr, uint32_t pair_empty_bar = 0, int row_limit = 0x7fffffff) {
  // private copy: the record lives in global memory; read in place, its fields would be loaded again after
  // every store of the tile (the stores could alias it)
  const GemmEpilogue e = e_in;
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t q = warp & 3;     // TMEM lane quarter this warp may read
  const uint32_t acc = tile_seq & 1, acc_ph = (tile_seq >> 1) & 1;
  uint32_t ok = 1;
  if (lane == 0) ok = mbar_wait(&c.tmem_full[acc], acc_ph, budget_ns, c.abort_word) ? 1u : 0u;
  ok = __shfl_sync(0xffffffffu, ok, 0);
  if (!ok) return false;
  tc_fence_after();
  const int row = m0 + q * 32 + lane;
  const bool scatter = e.mode == MACO_EPI_SCATTER_ROWS;
  const bool row_ok = row < e.M && (!scatter || row < row_limit);
  // scatter: this thread's row has its own destination row and weight (one 16-byte record per row)
  long long out_row = row + row_off;
  float row_weight = 1.f;
  if (scatter && row_ok) {
    const int4 rec = reinterpret_cast<const int4*>(e.aux)[row];
    out_row = (long long)rec.x * e.bias_type + rec.y;
    row_weight = __int_as_float(rec.z);
  }
  // staged path: 16-bit output, tile completely inside the output columns (uniform over the CTA)
  const int out_cols = e.mode == MACO_EPI_SWIGLU ? e.N / 2 : e.N;
  const int tile_col0 = e.mode == MACO_EPI_SWIGLU ? n0 / 2 : n0;
  const int tile_cols = e.mode == MACO_EPI_SWIGLU ? BN / 2 : BN;
  // (fp32 tiles that are plain stores take the same path: 32 columns are one 128-byte row chunk)
  const bool f32_out = e.out_type == MACO_DT_F32;
  const bool staged = stage != nullptr && (!f32_out || e.mode == MACO_EPI_F32_STORE) && tile_col0 + tile_cols <= out_cols &&
                      e.mode != MACO_EPI_F32_ACC;
  uint8_t* srow = stage != nullptr ? stage + q * kEpiStageWarpBytes + lane * kEpiStageRowBytes : nullptr;
  auto flush_group = [&](int gcol) {
    fence_proxy_async_smem();
    __syncwarp();
    if (row_ok) {
      const long long eoff = (out_row * e.ld_out + gcol) * (f32_out ? 4 : 2);
      if (bc == nullptr) {
        bulk_store(reinterpret_cast<uint8_t*>(out_base) + eoff, srow, 128);
      } else {
        for (int k = 0; k < bc->n; ++k) bulk_store(bc->bases[k] + bc->off + eoff, srow, 128);
      }
      tma_store_commit();
    }
    tma_store_wait_read<0>();
    __syncwarp();
  };
  const uint32_t t_row = tmem_base + ((q * 32u) << 16) + acc * SBN;
  if (e.mode == MACO_EPI_SWIGLU) {
    // Columns [0, BN/2) of the tile hold the gate projection, [BN/2, BN) the up projection of
    // the same BN/2 output features (weights are interleaved that way when the graph is built).
#pragma unroll 1
    for (int ch = 0; ch < BN / 64; ++ch) {
      uint32_t g[32], u[32];
      tmem_ld_32x32(t_row + ch * 32, g);
      tmem_ld_32x32(t_row + BN / 2 + ch * 32, u);
      tmem_ld_wait();
      float v[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = silu(__uint_as_float(g[j])) * __uint_as_float(u[j]);
      const int col0 = n0 / 2 + ch * 32;
      const int valid = min(32, e.N / 2 - col0);
      if (staged) {
        if (row_ok) epi_stage_chunk(srow, ch & 1, e.out_type, v);
        if (ch & 1) flush_group(col0 - 32);
      } else if (row_ok && valid > 0) {
        if (bc == nullptr) epi_store_row32(e, out_base, out_row, col0, valid, v);
        else for (int k = 0; k < bc->n; ++k) epi_store_row32(e, bc->bases[k] + bc->off, out_row, col0, valid, v);
      }
      __syncwarp();
    }
  } else {
#pragma unroll 1
    for (int ch = 0; ch < BN / 32; ++ch) {
      uint32_t r[32];
      tmem_ld_32x32(t_row + ch * 32, r);
      tmem_ld_wait();
      const int col0 = n0 + ch * 32;
      const int valid = min(32, e.N - col0);
      if (row_ok && valid > 0) {
      float v[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * e.alpha;
      if (scatter) {
        // the expert's output row is rounded to the output type first (what a separate return pass would read)
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          const uint32_t pk = epi_pack(e.out_type, v[j], v[j + 1]);
          const float2 f = e.out_type == MACO_DT_F16 ? __half22float2(*reinterpret_cast<const __half2*>(&pk)) : unpack_bf16x2(pk);
          v[j] = f.x * row_weight; v[j + 1] = f.y * row_weight;
        }
      }
      if (e.bias != nullptr && e.mode != MACO_EPI_SPLITK_FUSED) {     // (that mode keeps its arrival counters there)
#pragma unroll
        for (int j = 0; j < 32; ++j) if (j < valid) v[j] += epi_bias(e, col0 + j);
      }
      if (e.mode == MACO_EPI_GELU) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = gelu_tanh(v[j]);
      } else if (e.mode == MACO_EPI_GELU_BWD) {
        float ax[32];
        epi_load_aux32(e, row, col0, valid, ax);
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] *= gelu_tanh_grad(ax[j]);
      } else if (e.mode == MACO_EPI_SILU) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = silu(v[j]);
      } else if (e.mode == MACO_EPI_RESIDUAL) {
        const int n_aux = e.aux_pack & 15;
        if (n_aux <= 1) {
          float ax[32];
          epi_load_aux32(e, row, col0, valid, ax);
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] += ax[j];
        } else {
          // several blocks (a reduce-scatter's staging slots): the tile sums them all into its accumulator
          const int skip = (e.aux_pack >> 4) & 15;
          const long long slot_rows = e.aux_pack >> 8;
          for (int sl = 0; sl < n_aux; ++sl) {
            if (sl == skip) continue;
            float ax[32];
            epi_load_aux32(e, row + sl * slot_rows, col0, valid, ax);
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] += ax[j];
          }
        }
      }
      if (staged) {
        if (row_ok) {
          if (f32_out) epi_stage_chunk_f32(srow, v);
          else epi_stage_chunk(srow, ch & 1, e.out_type, v);
        }
      } else if (bc == nullptr) epi_store_row32(e, out_base, out_row, col0, valid, v);
      else for (int k = 0; k < bc->n; ++k) epi_store_row32(e, bc->bases[k] + bc->off, out_row, col0, valid, v);
      }
      if (staged && f32_out) flush_group(col0);
      else if (staged && (ch & 1)) flush_group(col0 - 32);
      __syncwarp();
    }
  }
  if (staged) tma_store_wait<0>();     // bulk stores complete before the tile is signalled
  tc_fence_before();
  if (pair_empty_bar == 0) {
    mbar_arrive(&c.tmem_empty[acc]);
  } else {
    // two-CTA tile: the pair leader's barrier collects one arrival per epilogue warp of both CTAs
    __syncwarp();
    if (lane == 0) mbar_arrive_cluster(pair_empty_bar + acc * 8);
  }
  return true;
}

// ---- CTA set-up / tear-down shared by every kernel built on this pipeline ------------------------
template <int BN, int STAGES>
MACO_DEVICE uint8_t* gemm_cta_setup(uint8_t* dyn_smem, GemmCtrl& c, uint32_t& tmem_base, bool alloc_tmem = true) {
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(dyn_smem) + 1023) & ~uintptr_t(1023));
  c = gemm_ctrl<BN, STAGES>(smem);
  const uint32_t warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&c.full[s], 1); mbar_init(&c.empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&c.tmem_full[a], 1); mbar_init(&c.tmem_empty[a], 128); }
    *c.abort_word = 0;
    fence_mbar_init();
  }
  if (threadIdx.x == 32) *c.tmem_slot = 0;
  __syncwarp();
  if (warp == 1 && alloc_tmem) {
    tmem_alloc(c.tmem_slot, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  tmem_base = *c.tmem_slot;
  return smem;
}

template <int BN>
MACO_DEVICE void gemm_cta_teardown(const GemmCtrl& c, uint32_t tmem_base, uint32_t* status, bool had_tmem = true) {
  tc_fence_before();
  __syncthreads();
  if ((threadIdx.x >> 5) == 1 && had_tmem) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
  if (threadIdx.x == 0 && *c.abort_word != 0 && status != nullptr) st_relaxed_sys_u32(status, MACO_STATUS_TIMEOUT);
}

// ---- two-CTA tiles (cta_group::2) -----------------------------------------------------------------
// A pair of CTAs (one cluster) computes a 256 x BN tile: each CTA loads its own 128 rows of A and its own
// half (BN/2 rows) of B, the leader issues tcgen05.mma.cta_group::2 (M = 256), which reads both CTAs' shared
// memory and writes each CTA's 128 accumulator rows into that CTA's TMEM. Per k-step a CTA brings in
// 16 KB + BN/2 * 128 B instead of 16 KB + BN * 128 B: a third less shared-memory and L2 traffic per FLOP at
// BN = 256, and six 32 KB stages where the one-CTA form has four of 48 KB. The two row blocks of a pair
// need not be adjacent. Loads carry no multicast: each CTA fetches what it needs itself.
template <int STAGES>
struct PairSmemLayout {
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytesMax = 128 * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytesMax;
  static constexpr int kRingBytes = STAGES * kStageBytes;
  static constexpr int kCtrlBytes = 256;
  static constexpr int kTotalBytes = kRingBytes + kCtrlBytes + 1024;
  static_assert(2 * STAGES * 8 + 4 * 8 + 16 <= kCtrlBytes, "control block too small");
};

template <int STAGES>
MACO_DEVICE GemmCtrl pair_ctrl(uint8_t* smem_base) {
  using L = PairSmemLayout<STAGES>;
  GemmCtrl c;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_base + L::kRingBytes);
  c.full = bars;
  c.empty = bars + STAGES;
  c.tmem_full = bars + 2 * STAGES;
  c.tmem_empty = bars + 2 * STAGES + 2;
  c.tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  c.abort_word = reinterpret_cast<volatile uint32_t*>(c.tmem_slot + 1);
  return c;
}

// Producer of one CTA of the pair. `n0` is the tile's first column; this CTA loads B rows
// [n0 + rank * BN/2, n0 + (rank + 1) * BN/2). All bytes of both CTAs are credited to the LEADER's full barrier
// by the TMA units themselves. (Measured alternative: loads completing on each CTA's own barrier plus a thread
// of the second CTA that forwards an arrival to the leader took twice as long per k-block.)
template <int BN, int STAGES, bool A_MN, bool B_MN>
MACO_DEVICE bool pair_produce_tile(uint8_t* smem, const GemmCtrl& c, uint32_t rank, const CUtensorMap* tmA,
                                   const CUtensorMap* tmB, int m0, int n0, int k0, int k_blocks, uint32_t& it,
                                   uint64_t budget_ns, long long* prof = nullptr) {
  using L = PairSmemLayout<STAGES>;
  constexpr int kBHalf = BN / 2;
  constexpr uint32_t kPairBytes = 2u * (L::kABytes + kBHalf * kBK * 2);
  const uint32_t full0 = mapa_u32(smem_u32(&c.full[0]), 0);
  const int nb0 = n0 + (int)rank * kBHalf;
  uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
  uint8_t* sa = smem + s * L::kStageBytes;
  int k = k0;
  for (int kb = 0; kb < k_blocks; ++kb, k += kBK) {
    const long long t0 = prof ? clock64() : 0;
    if (!mbar_wait(&c.empty[s], ph ^ 1, budget_ns, c.abort_word)) { it += kb; return false; }
    if (prof) prof[0] += clock64() - t0;
    if (prof && prof[4] && prof[5] < 512) reinterpret_cast<uint64_t*>(prof[4])[2 * prof[5]] = globaltimer_ns();
    uint8_t* sb = sa + L::kABytes;
    if (rank == 0) mbar_arrive_expect_tx(&c.full[s], kPairBytes);
    const uint32_t bar = full0 + s * 8;
    if constexpr (!A_MN) {
      tma_load_2d_pair(sa, tmA, bar, k, m0);
    } else {
#pragma unroll
      for (int j = 0; j < kBM / 64; ++j) tma_load_2d_pair(sa + j * 8192, tmA, bar, m0 + j * 64, k);
    }
    if constexpr (!B_MN) {
      tma_load_2d_pair(sb, tmB, bar, k, nb0);
    } else {
#pragma unroll
      for (int j = 0; j < kBHalf / 64; ++j) tma_load_2d_pair(sb + j * 8192, tmB, bar, nb0 + j * 64, k);
    }
    if (prof && prof[4] && prof[5] < 512) { reinterpret_cast<uint64_t*>(prof[4])[2 * prof[5] + 1] = globaltimer_ns(); ++prof[5]; }
    if (++s == STAGES) { s = 0; ph ^= 1; sa = smem; } else { sa += L::kStageBytes; }
  }
  it += k_blocks;
  return true;
}

// MMA issuer: the pair's leader only. `peer_*` are the shared::cluster addresses of the other CTA's barriers.
template <int BN, int STAGES, bool A_MN, bool B_MN>
MACO_DEVICE bool pair_mma_tile(uint8_t* smem, const GemmCtrl& c, uint32_t tmem_base, uint32_t idesc, int k_blocks,
                               uint32_t& it, uint32_t tile_seq, uint64_t budget_ns, long long* prof = nullptr) {
  using L = PairSmemLayout<STAGES>;
  const uint32_t acc = tile_seq & 1, acc_ph = (tile_seq >> 1) & 1;
  const uint32_t empty0 = smem_u32(&c.empty[0]), tfull0 = smem_u32(&c.tmem_full[0]);
  long long t0 = prof ? clock64() : 0;
  if (!mbar_wait(&c.tmem_empty[acc], acc_ph ^ 1, budget_ns, c.abort_word)) return false;
  if (prof) prof[1] += clock64() - t0;
  tc_fence_after();
  const uint32_t d_tmem = tmem_base + acc * 256;
  const uint64_t da0 = A_MN ? make_smem_desc(0, 8192, 1024, 2) : make_smem_desc(0, 16, 1024, 2);
  const uint64_t db0 = B_MN ? make_smem_desc(0, 8192, 1024, 2) : make_smem_desc(0, 16, 1024, 2);
  const uint32_t a_hi = (uint32_t)(da0 >> 32), b_hi = (uint32_t)(db0 >> 32);
  const uint32_t a_lbo = (uint32_t)da0, b_lbo = (uint32_t)db0;          // leading-dimension offset field (bits 16-29)
  constexpr uint32_t kStepA = (A_MN ? 2048 : 32) >> 4, kStepB = (B_MN ? 2048 : 32) >> 4;
  constexpr uint32_t kStage16 = L::kStageBytes >> 4, kAB16 = L::kABytes >> 4;
  const uint32_t base_lo = (smem_u32(smem) & 0x3FFFFu) >> 4;
  uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
  uint32_t a_lo = base_lo + s * kStage16;
  uint32_t accum = 0;
  for (int kb = 0; kb < k_blocks; ++kb) {
    if (prof) t0 = clock64();
    if (!mbar_wait(&c.full[s], ph, budget_ns, c.abort_word)) { it += kb; return false; }
    if (prof) prof[2] += clock64() - t0;
    if (prof && prof[4] && prof[5] < 512) reinterpret_cast<uint64_t*>(prof[4])[2 * prof[5]] = globaltimer_ns();
    const uint32_t b_lo = a_lo + kAB16;
#pragma unroll
    for (int k = 0; k < kBK / kUmmaK; ++k) {
      tc_mma2_f16_lo(d_tmem, (a_lo + k * kStepA) | a_lbo, a_hi, (b_lo + k * kStepB) | b_lbo, b_hi, idesc, accum);
      accum = 1;
    }
    tc_commit2_both(empty0 + s * 8);   // both CTAs may refill the stage once these MMAs have read it
    if (prof && prof[4] && prof[5] < 512) { reinterpret_cast<uint64_t*>(prof[4])[2 * prof[5] + 1] = globaltimer_ns(); ++prof[5]; }
    if (++s == STAGES) { s = 0; ph ^= 1; a_lo = base_lo; } else { a_lo += kStage16; }
  }
  it += k_blocks;
  tc_commit2_both(tfull0 + acc * 8);   // accumulator complete -> both CTAs' epilogues
  return true;
}

template <int STAGES>
MACO_DEVICE uint8_t* pair_cta_setup(uint8_t* dyn_smem, GemmCtrl& c, uint32_t& tmem_base) {
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(dyn_smem) + 1023) & ~uintptr_t(1023));
  c = pair_ctrl<STAGES>(smem);
  const uint32_t warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&c.full[s], 1); mbar_init(&c.empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&c.tmem_full[a], 1); mbar_init(&c.tmem_empty[a], 8); }   // 4 warps x 2 CTAs
    *c.abort_word = 0;
    fence_mbar_init();
  }
  if (threadIdx.x == 32) *c.tmem_slot = 0;
  __syncwarp();
  if (warp == 1) {
    tmem_alloc2(c.tmem_slot, 512);
    tmem_relinquish2();
  }
  tc_fence_before();
  __syncthreads();
  cluster_arrive();            // the other CTA's barriers are initialised before anything is sent to them
  cluster_wait();
  tc_fence_after();
  tmem_base = *c.tmem_slot;
  return smem;
}

MACO_DEVICE void pair_cta_teardown(const GemmCtrl& c, uint32_t tmem_base, uint32_t* status) {
  tc_fence_before();
  __syncthreads();
  cluster_arrive();            // neither CTA frees TMEM or leaves while the other may still touch its memory
  cluster_wait();
  if ((threadIdx.x >> 5) == 1) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, 512);
  }
  if (threadIdx.x == 0 && *c.abort_word != 0 && status != nullptr) st_relaxed_sys_u32(status, MACO_STATUS_TIMEOUT);
}

constexpr int kPairStages = 6;

// Stand-alone GEMM on two-CTA tiles: grid = 2 x (number of CTA pairs), launched as clusters of two.
template <int BN, bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         GemmEpilogue epi, int K, uint32_t idesc, uint64_t budget_ns, uint32_t* status, long long* dbg) {
  extern __shared__ uint8_t dyn_smem[];
  GemmCtrl c;
  uint32_t tmem_base;
  uint8_t* smem = pair_cta_setup<kPairStages>(dyn_smem, c, tmem_base);
  // optional cycle counters per CTA: [0] producer waiting for a free stage, [1] MMA waiting for a free
  // accumulator, [2] MMA waiting for operands, [3] MMA warp total, [4] producer total
  // [3]: experiment switches, see maco_gemm_set_debug; [4], [5]: optional time-line log (switch 8, first pair only):
  // words 4096 + 2048 * cta + {0: producer, 1024: MMA warp} + 2 * i + {0: wait over, 1: issue done}, %globaltimer ns
  long long prof[6] = {0, 0, 0, dbg != nullptr ? dbg[7] : 0, 0, 0};
  long long* pp = dbg != nullptr ? prof : nullptr;
  const int variant = (int)prof[3];
  if (dbg != nullptr && (variant & 8) && blockIdx.x < 2)
    prof[4] = reinterpret_cast<long long>(dbg + 4096 + 2048 * blockIdx.x + ((threadIdx.x >> 5) == 1 ? 1024 : 0));
  const long long t_begin = clock64();
  const uint32_t rank = cluster_ctarank();
  const int m_pairs = (epi.M + 2 * kBM - 1) / (2 * kBM), n_tiles = (epi.N + BN - 1) / BN;
  const int num_tiles = m_pairs * n_tiles;
  const int k_blocks = (K + kBK - 1) / kBK;
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t tempty_leader = mapa_u32(smem_u32(&c.tmem_empty[0]), 0);

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      uint32_t it = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < num_tiles; tile += num_pairs) {
        int mp, nb;
        gemm_tile_coords(tile, m_pairs, n_tiles, mp, nb);
        ok = pair_produce_tile<BN, kPairStages, A_MN, B_MN>(smem, c, rank, &tmA, &tmB, (mp * 2 + (int)rank) * kBM, nb * BN, 0,
                                                            k_blocks, it, budget_ns, pp);
      }
      // after an abort the leader's barriers count both CTAs' bytes; the other CTA stays until the leader
      // reaches the teardown (cluster barrier)
      if (!ok && rank == 0) gemm_drain_loads<kPairStages>(c, it);
      if (dbg != nullptr) { dbg[blockIdx.x * 8 + 0] = prof[0]; dbg[blockIdx.x * 8 + 4] = clock64() - t_begin; }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      uint32_t it = 0, seq = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < num_tiles; tile += num_pairs, ++seq)
        ok = pair_mma_tile<BN, kPairStages, A_MN, B_MN>(smem, c, tmem_base, idesc, k_blocks, it, seq, budget_ns, pp);
      if (dbg != nullptr) { dbg[blockIdx.x * 8 + 1] = prof[1]; dbg[blockIdx.x * 8 + 2] = prof[2]; dbg[blockIdx.x * 8 + 3] = clock64() - t_begin; }
    }
    __syncwarp();
  } else {
    uint32_t seq = 0;
    bool ok = true;
    for (int tile = pair; ok && tile < num_tiles; tile += num_pairs, ++seq) {
      int mp, nb;
      gemm_tile_coords(tile, m_pairs, n_tiles, mp, nb);
      if (variant & 1) {           // experiment: barrier handshake only
        if (lane == 0) ok = mbar_wait(&c.tmem_full[seq & 1], (seq >> 1) & 1, budget_ns, c.abort_word);
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(tempty_leader + (seq & 1) * 8);
        continue;
      }
      ok = gemm_epilogue_tile<BN, 256>(c, tmem_base, epi, epi.out, 0, (mp * 2 + (int)rank) * kBM, nb * BN, seq, budget_ns,
                                       nullptr, nullptr, tempty_leader);
    }
  }
  pair_cta_teardown(c, tmem_base, status);
}

// ---- stand-alone persistent GEMM kernel ---------------------------------------------------------
template <int BN, int STAGES, bool A_MN, bool B_MN, bool TF32 = false>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    GemmEpilogue epi, int K, uint32_t idesc, uint64_t budget_ns, uint32_t* status, long long* dbg) {
  extern __shared__ uint8_t dyn_smem[];
  GemmCtrl c;
  uint32_t tmem_base;
  uint8_t* smem = gemm_cta_setup<BN, STAGES>(dyn_smem, c, tmem_base);
  long long prof[4] = {0, 0, 0, dbg != nullptr ? dbg[7] : 0};   // see gemm_tcgen05_pair_kernel
  long long* pp = dbg != nullptr ? prof : nullptr;
  const int variant = (int)prof[3];
  const long long t_begin = clock64();

  const int m_tiles = (epi.M + kBM - 1) / kBM, n_tiles = (epi.N + BN - 1) / BN;
  const int num_tiles = m_tiles * n_tiles;
  constexpr int kStepElems = TF32 ? kBK / 2 : kBK;
  const int k_blocks = (K + kStepElems - 1) / kStepElems;
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        int mb, nb;
        gemm_tile_coords(tile, m_tiles, n_tiles, mb, nb);
        ok = gemm_produce_tile<BN, STAGES, A_MN, B_MN>(smem, c, &tmA, &tmB, mb * kBM, nb * BN, 0, k_blocks, it, budget_ns, pp, kStepElems);
      }
      if (!ok) gemm_drain_loads<STAGES>(c, it);
      if (dbg != nullptr) { dbg[blockIdx.x * 8 + 0] = prof[0]; dbg[blockIdx.x * 8 + 4] = clock64() - t_begin; }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      uint32_t it = 0, seq = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++seq)
        ok = gemm_mma_tile<BN, STAGES, A_MN, B_MN, BN, TF32>(smem, c, tmem_base, idesc, k_blocks, it, seq, budget_ns, pp);
      if (dbg != nullptr) { dbg[blockIdx.x * 8 + 1] = prof[1]; dbg[blockIdx.x * 8 + 2] = prof[2]; dbg[blockIdx.x * 8 + 3] = clock64() - t_begin; }
    }
    __syncwarp();
  } else {
    uint32_t seq = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++seq) {
      int mb, nb;
      gemm_tile_coords(tile, m_tiles, n_tiles, mb, nb);
      if (variant & 1) {           // experiment: barrier handshake only
        if (lane == 0) ok = mbar_wait(&c.tmem_full[seq & 1], (seq >> 1) & 1, budget_ns, c.abort_word);
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        mbar_arrive(&c.tmem_empty[seq & 1]);
        continue;
      }
      ok = gemm_epilogue_tile<BN>(c, tmem_base, epi, epi.out, 0, mb * kBM, nb * BN, seq, budget_ns);
    }
  }
  gemm_cta_teardown<BN>(c, tmem_base, status);
}

}  // namespace maco
