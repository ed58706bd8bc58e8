// The persistent task kernel: ONE launch executes a whole compiled task graph.
//
//   CTA 0 .. num_workers-1   worker CTAs (6 warps: TMA producer, MMA issuer, 4 general warps)
//   CTA num_workers          scheduler CTA (dynamic mode only)
//
// What the reference describes and never launches (maco/csrc/maco_kernel.cu:36-44 has no host
// launcher; its live kernel, :58-140, has workers only with queues the CPU fills through three
// host syncs per task) is here the execution path of TaskGraph.execute():
//
//  * Tasks are tile-granular 128-byte descriptors uploaded once at compile time. Each carries up
//    to two wait conditions (event, count) and up to two local signals plus one peer signal.
//  * Events are monotonic 32-bit counters that are never reset: launch number `epoch` waits for
//    events[e] >= epoch * count, so re-executing a graph needs no clearing pass and a peer GPU
//    that runs ahead cannot be lost by a reset.
//  * STATIC mode: every worker walks a queue written at compile time in global topological
//    order (which makes the schedule deadlock-free as long as all CTAs are resident: the
//    earliest unfinished task always sits at the front of its queue) and waits on the events
//    of each task itself: tile-granular, signal-driven, no central hop.
//  * DYNAMIC mode: the scheduler CTA polls the events of dispatch groups (a group = the tiles of
//    one node that become ready together), and when a group's conditions hold pushes its tasks
//    into the per-worker rings: slot written first, then the head published with st.release
//    (the reference advances the head before writing the slot, maco_worker.cuh:342-344). Each
//    ring has one producer (the scheduler) and one consumer CTA; workers publish their tail for
//    back-pressure. A TERMINATE entry ends each ring.
//  * Inside a worker the three roles read the same task sequence independently, so the
//    producer warp prefetches operands of task i+1 while the epilogue of task i drains TMEM.
//  * Every wait (event, ring, mbarrier) is bounded by `budget_ns`; on expiry the CTA records
//    {status, task, event, cta} in the host-mapped status block, raises the launch-wide abort
//    word, and all CTAs drain and return.
#include "elementwise.cuh"
#include "gemm_tcgen05.cuh"
#include "comm_tasks.cuh"
#include "attention_decode.cuh"
#include "moe_tasks.cuh"
#include "splitk_tasks.cuh"
#include "host_common.h"

using namespace maco;

namespace {

constexpr int kMkBN = 256;
constexpr int kMkStages = 4;
using MkLayout = GemmSmemLayout<kMkBN, kMkStages>;
constexpr int kMkExtraSmem = 1024;     // scheduler heads / current-task slots live after the GEMM control block
constexpr int kMkScratchSmem = 28672;  // scratch of non-GEMM tasks (the operand ring is NOT free for them:
                                       // the producer warp may already be filling it for the next GEMM task)
constexpr int kMkSmemBytes = MkLayout::kTotalBytes + kMkExtraSmem + kMkScratchSmem;
static_assert(kMkScratchSmem >= kEpiStageBytes, "epilogue staging must fit the scratch block");
static_assert(kMkScratchSmem >= kAttnScratchBytes && kMkScratchSmem >= kAttnTcScratchBytes, "attention scratch must fit the scratch block");
static_assert(kMkSmemBytes <= 227 * 1024, "persistent kernel exceeds the shared memory of an SM");
constexpr uint32_t kBulkBufBytes = 16384;                                  // staging buffers of bulk pushes
constexpr uint32_t kBulkBuffers = MkLayout::kRingBytes / kBulkBufBytes;    // the whole operand ring
static_assert(kBulkBuffers <= 16, "phase bits / barrier slots");
// Two-CTA programs (cta_group::2) cut the same operand memory into six 32 KB stages; the control block sits at
// the same offset, so everything behind it (task slots, bulk and attention barriers, scratch) is shared code.
using MkPairLayout = PairSmemLayout<kPairStages>;
static_assert(MkPairLayout::kRingBytes == MkLayout::kRingBytes && MkPairLayout::kCtrlBytes == MkLayout::kCtrlBytes,
              "one-CTA and two-CTA programs share one shared-memory map");

__device__ __forceinline__ void general_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

__device__ __forceinline__ bool is_gemm_type(uint32_t type) { return type == MACO_TASK_MATMUL || type == MACO_TASK_LINEAR; }

__device__ __forceinline__ bool aborted(const MacoProgram& p) { return ld_relaxed_gpu_u32(p.abort_word) == p.epoch; }

__device__ void report_failure(const MacoProgram& p, uint32_t status, uint32_t task, uint32_t event,
                               volatile uint32_t* cta_abort) {
  if (cta_abort != nullptr) *cta_abort = 1;
  // The first CTA to fail claims the abort word with one compare-and-swap (it holds the epoch of an aborted
  // launch, anything else otherwise) and is the only one to fill the status block, so {task, event, cta}
  // always describe the same failure.
  const uint32_t seen = ld_relaxed_gpu_u32(p.abort_word);
  if (seen == p.epoch) return;
  if (atomicCAS(p.abort_word, seen, p.epoch) != seen) return;
  if (p.status != nullptr) {
    volatile MacoStatusBlock* s = p.status;
    s->task = task; s->event = event; s->cta = blockIdx.x; s->rank = (uint32_t)p.rank;
    __threadfence_system();
    s->status = s->status | status;
  }
}

// Bounded wait until *flag >= expect (wrap-safe). Leaves early when the launch was aborted.
__device__ bool mk_wait(const MacoProgram& p, const uint32_t* flag, uint32_t expect, bool sys) {
  uint32_t v = sys ? ld_acquire_sys_u32(flag) : ld_acquire_gpu_u32(flag);
  if ((int32_t)(v - expect) >= 0) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (true) {
    v = sys ? ld_acquire_sys_u32(flag) : ld_acquire_gpu_u32(flag);
    if ((int32_t)(v - expect) >= 0) return true;
    if ((++spins & 31u) == 0) {
      if (aborted(p)) return false;
      if (globaltimer_ns() - t0 > p.budget_ns) return false;
    }
    __nanosleep(32);
  }
}

__device__ bool wait_deps(const MacoProgram& p, const MacoTaskDesc& d, uint32_t task, volatile uint32_t* cta_abort,
                          uint64_t* wait_ns) {
  const uint64_t t0 = wait_ns ? globaltimer_ns() : 0;
  {
    // Common case, every condition already holds. Counters bumped by this GPU only are read together with
    // relaxed loads and ordered by ONE .gpu fence. Counters bumped by other GPUs are read with an acquire load
    // at .sys scope instead of a relaxed load plus fence.acq_rel.sys: the full fence at system scope also waits
    // for this GPU's outstanding writes to peers and to the host, and takes tens of microseconds while a
    // host -> device copy is in flight (measured: +300 us per step of the tensor-parallel layer).
    // A condition with count 0 always holds (a block that is already in place) and is not read at all.
    bool sat = true, any_gpu = false;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int e = d.wait_event[j];
      if (e < 0 || d.wait_count[j] == 0) continue;
      const bool sys = (d.flags & (j == 0 ? MACO_TF_WAIT0_SYS : MACO_TF_WAIT1_SYS)) != 0;
      const bool prev = (d.flags & (j == 0 ? MACO_TF_WAIT0_PREV : MACO_TF_WAIT1_PREV)) != 0;
      const uint32_t need = (p.epoch - (prev ? 1u : 0u)) * d.wait_count[j];
      const uint32_t v = sys ? ld_acquire_sys_u32(&p.events[e]) : ld_relaxed_gpu_u32(&p.events[e]);
      any_gpu |= !sys;
      if ((int32_t)(v - need) < 0) sat = false;
    }
    if (sat) {
      if (any_gpu) fence_acq_rel_gpu();
      if (wait_ns) *wait_ns += globaltimer_ns() - t0;
      return true;
    }
  }
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int e = d.wait_event[j];
    if (e < 0 || d.wait_count[j] == 0) continue;
    const bool sys = (d.flags & (j == 0 ? MACO_TF_WAIT0_SYS : MACO_TF_WAIT1_SYS)) != 0;
    const bool prev = (d.flags & (j == 0 ? MACO_TF_WAIT0_PREV : MACO_TF_WAIT1_PREV)) != 0;
    if (!mk_wait(p, &p.events[e], (p.epoch - (prev ? 1u : 0u)) * d.wait_count[j], sys)) {
      report_failure(p, sys ? MACO_STATUS_PEER_TIMEOUT : MACO_STATUS_TIMEOUT, task, (uint32_t)e, cta_abort);
      return false;
    }
  }
  if (wait_ns) *wait_ns += globaltimer_ns() - t0;
  return true;
}

__device__ void signal_done(const MacoProgram& p, const MacoTaskDesc& d) {
  // One release fence for the whole task, then relaxed counter bumps: a release per destination would
  // repeat the fence (a round trip over NVLink once a peer is involved) for every rank that is signalled.
  const bool sys = (d.flags & MACO_TF_SIGNAL_SYS) != 0 || d.signal_peer_event >= 0;
  if (d.signal_peer == -4 && d.signal_peer_event >= 0 && d.signal_event[0] < 0 && d.signal_event[1] < 0 && p.mc_heap != nullptr) {
    // one release-reduction through the NVSwitch bumps the counter in every rank's table (this rank's too)
    uint32_t* mc_events = reinterpret_cast<uint32_t*>(p.mc_heap + (reinterpret_cast<uint8_t*>(p.events) - p.peer_heap[p.rank]));
    multimem_red_add_u32(mc_events + d.signal_peer_event, 1);
    return;
  }
  if (sys) fence_acq_rel_sys(); else fence_acq_rel_gpu();
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int e = d.signal_event[j];
    if (e < 0) continue;
    if (sys) red_add_relaxed_sys_u32(&p.events[e], 1); else red_add_relaxed_gpu_u32(&p.events[e], 1);
  }
  if (d.signal_peer_event >= 0) {
    if (d.signal_peer >= 0) {
      red_add_relaxed_sys_u32(&p.peer_events[d.signal_peer][d.signal_peer_event], 1);
    } else if (d.signal_peer == -2 || d.signal_peer == -4) {
      for (int r = 0; r < p.world; ++r) red_add_relaxed_sys_u32(&p.peer_events[r][d.signal_peer_event], 1);
    }
  }
}

// Debug re-check of a descriptor on the device (MacoProgram.debug): the same conditions the host checks when the
// program is built. A descriptor that fails is not run; the launch reports BAD_TASK.
__device__ bool desc_ok(const MacoProgram& p, const MacoTaskDesc& d) {
  for (int j = 0; j < 2; ++j) {
    if (d.wait_event[j] >= (int)p.num_events || d.signal_event[j] >= (int)p.num_events) return false;
  }
  if (d.signal_peer_event >= (int)p.num_events) return false;
  if (d.signal_peer >= p.world || d.signal_peer < -4) return false;
  if (is_gemm_type(d.type)) {
    const MacoGemmArgs& g = d.u.gemm;
    if (g.tmap_a >= p.num_tmaps || g.tmap_b >= p.num_tmaps || g.epi >= p.num_epis) return false;
    if (g.peer >= p.world || g.peer < -2) return false;
    if (g.peer != -1 && (p.heap_bytes == 0 || g.out_off >= p.heap_bytes)) return false;
    return g.k_blocks >= 0 && (g.bn == 128 || g.bn == 256);
  }
  if (d.type >= 200 && d.type < 300 && d.u.comm.rows != 0) {
    const MacoCommArgs& a = d.u.comm;
    if (a.row_bytes % 16 != 0 || a.peer >= p.world || a.peer < -3) return false;
    const uint64_t ext = (uint64_t)(a.rows - 1) * a.dst_stride + a.row_bytes;
    const bool writes_heap = a.local_ptr == nullptr && a.op != MACO_COMM_REDUCE_LOCAL;
    if (writes_heap && (p.heap_bytes == 0 || a.dst_off + ext > p.heap_bytes)) return false;
    const uint64_t sext = (uint64_t)(a.rows - 1) * a.src_stride + a.row_bytes;
    const bool reads_peer = a.op == MACO_COMM_REDUCE_PULL || a.op == MACO_COMM_ALLREDUCE || a.op == MACO_COMM_PULL ||
                            a.op == MACO_COMM_ALLREDUCE_MC;
    if (reads_peer && (p.heap_bytes == 0 || a.src_off + sext > p.heap_bytes)) return false;
    if ((a.op == MACO_COMM_PUSH_MC || a.op == MACO_COMM_ALLREDUCE_MC) && p.mc_heap == nullptr) return false;
  }
  return true;
}

// Next entry of this worker's queue. false = aborted / timed out.
__device__ bool fetch_task(const MacoProgram& p, uint32_t w, uint32_t i, uint32_t q_base, uint32_t& task,
                           volatile uint32_t* cta_abort) {
  if (p.mode == MACO_MODE_STATIC) {
    const uint32_t n = p.static_count[w];
    const uint32_t* q = p.static_queue + (size_t)w * p.static_stride;
    task = i < n ? q[i] : MACO_QUEUE_TERMINATE;
    if (i + 1 < n) {
      // the next descriptor is on its way while this task runs (the three roles share the L1 line)
      const MacoTaskDesc* nd = p.tasks + (q[i + 1] & MACO_QUEUE_INDEX_MASK);
      asm volatile("prefetch.global.L1 [%0];" :: "l"(nd));
    }
    return true;
  }
  const uint32_t pos = q_base + i;
  if (!mk_wait(p, &p.heads[w], pos + 1, false)) {
    report_failure(p, MACO_STATUS_TIMEOUT, 0xfffffffeu, w, cta_abort);
    return false;
  }
  task = ld_relaxed_gpu_u32(&p.ring[(size_t)w * MACO_WORKER_QUEUE_SIZE + (pos & (MACO_WORKER_QUEUE_SIZE - 1))]);
  return true;
}

__device__ __forceinline__ bool is_gemm(uint32_t type) { return type == MACO_TASK_MATMUL || type == MACO_TASK_LINEAR; }

__device__ __forceinline__ MacoTaskDesc load_desc(const MacoProgram& p, uint32_t task) {
  MacoTaskDesc d;
  const uint4* src = reinterpret_cast<const uint4*>(p.tasks + task);
  uint4* dst = reinterpret_cast<uint4*>(&d);
#pragma unroll
  for (int i = 0; i < 8; ++i) dst[i] = src[i];
  return d;
}

// ---- producer warp (lane 0), two-CTA programs ----------------------------------------------------
// Every GEMM task of such a program is one half (128 rows) of a 256 x BN tile; the two halves sit at the same
// position of the GEMM sequences of workers 2j and 2j+1 (one cluster). Each CTA waits for ITS half's
// conditions and loads its rows of A and its half of B; the leader's MMA warp starts when both have landed.
__device__ void producer_role_pair(const MacoProgram& p, uint32_t w, uint32_t q_base, uint8_t* smem, const GemmCtrl& c) {
  uint32_t it = 0;
  bool ok = true;
  const uint32_t rank = cluster_ctarank();
  const CUtensorMap* tmaps = reinterpret_cast<const CUtensorMap*>(p.tmaps);
  for (uint32_t i = 0; ok; ++i) {
    uint32_t task;
    if (!fetch_task(p, w, i, q_base, task, c.abort_word)) { ok = false; break; }
    if (task == MACO_QUEUE_TERMINATE) break;
    task &= MACO_QUEUE_INDEX_MASK;
    const MacoTaskDesc& d = p.tasks[task];
    if (!is_gemm(d.type)) continue;
    if (p.debug != 0 && !desc_ok(p, d)) { report_failure(p, MACO_STATUS_BAD_TASK, task, d.type, c.abort_word); ok = false; break; }
    if (!wait_deps(p, d, task, c.abort_word, nullptr)) { ok = false; break; }
    const MacoGemmArgs& g = d.u.gemm;
    fence_proxy_async_all();           // operands were written by generic-proxy stores of other CTAs
    const CUtensorMap* ta = tmaps + g.tmap_a;
    const CUtensorMap* tb = tmaps + g.tmap_b;
    const int sel = (g.bn == 128 ? 4 : 0) | (g.a_mn ? 2 : 0) | ((g.b_mn & 1) ? 1 : 0);
    switch (sel) {
      case 0: ok = pair_produce_tile<256, kPairStages, false, false>(smem, c, rank, ta, tb, g.m0, g.n0, g.k0, g.k_blocks, it, p.budget_ns); break;
      case 1: ok = pair_produce_tile<256, kPairStages, false, true>(smem, c, rank, ta, tb, g.m0, g.n0, g.k0, g.k_blocks, it, p.budget_ns); break;
      case 2: ok = pair_produce_tile<256, kPairStages, true, false>(smem, c, rank, ta, tb, g.m0, g.n0, g.k0, g.k_blocks, it, p.budget_ns); break;
      case 3: ok = pair_produce_tile<256, kPairStages, true, true>(smem, c, rank, ta, tb, g.m0, g.n0, g.k0, g.k_blocks, it, p.budget_ns); break;
      case 4: ok = pair_produce_tile<128, kPairStages, false, false>(smem, c, rank, ta, tb, g.m0, g.n0, g.k0, g.k_blocks, it, p.budget_ns); break;
      case 5: ok = pair_produce_tile<128, kPairStages, false, true>(smem, c, rank, ta, tb, g.m0, g.n0, g.k0, g.k_blocks, it, p.budget_ns); break;
      case 6: ok = pair_produce_tile<128, kPairStages, true, false>(smem, c, rank, ta, tb, g.m0, g.n0, g.k0, g.k_blocks, it, p.budget_ns); break;
      default: ok = pair_produce_tile<128, kPairStages, true, true>(smem, c, rank, ta, tb, g.m0, g.n0, g.k0, g.k_blocks, it, p.budget_ns); break;
    }
    if (!ok) report_failure(p, MACO_STATUS_TIMEOUT, task, 0xffffffffu, c.abort_word);
  }
  if (!ok) {
    // loads in flight land in this CTA's memory: the leader's barriers count both CTAs' bytes, the other CTA
    // gives its own loads a fixed grace period
    if (rank == 0) gemm_drain_loads<kPairStages>(c, it);
    else { const uint64_t t0 = globaltimer_ns(); while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000); }
  }
}

// ---- MMA warp (lane 0) of the pair's leader ------------------------------------------------------
__device__ void mma_role_pair(const MacoProgram& p, uint32_t w, uint32_t q_base, uint8_t* smem, const GemmCtrl& c,
                              uint32_t tmem_base) {
  uint32_t it = 0, seq = 0;
  bool ok = true;
  for (uint32_t i = 0; ok; ++i) {
    uint32_t task;
    if (!fetch_task(p, w, i, q_base, task, c.abort_word)) break;
    if (task == MACO_QUEUE_TERMINATE) break;
    task &= MACO_QUEUE_INDEX_MASK;
    const MacoTaskDesc& d = p.tasks[task];
    if (!is_gemm(d.type)) continue;
    const MacoGemmArgs& g = d.u.gemm;
    const int sel = (g.bn == 128 ? 4 : 0) | (g.a_mn ? 2 : 0) | ((g.b_mn & 1) ? 1 : 0);
    switch (sel) {
      case 0: ok = pair_mma_tile<256, kPairStages, false, false>(smem, c, tmem_base, g.idesc, g.k_blocks, it, seq, p.budget_ns); break;
      case 1: ok = pair_mma_tile<256, kPairStages, false, true>(smem, c, tmem_base, g.idesc, g.k_blocks, it, seq, p.budget_ns); break;
      case 2: ok = pair_mma_tile<256, kPairStages, true, false>(smem, c, tmem_base, g.idesc, g.k_blocks, it, seq, p.budget_ns); break;
      case 3: ok = pair_mma_tile<256, kPairStages, true, true>(smem, c, tmem_base, g.idesc, g.k_blocks, it, seq, p.budget_ns); break;
      case 4: ok = pair_mma_tile<128, kPairStages, false, false>(smem, c, tmem_base, g.idesc, g.k_blocks, it, seq, p.budget_ns); break;
      case 5: ok = pair_mma_tile<128, kPairStages, false, true>(smem, c, tmem_base, g.idesc, g.k_blocks, it, seq, p.budget_ns); break;
      case 6: ok = pair_mma_tile<128, kPairStages, true, false>(smem, c, tmem_base, g.idesc, g.k_blocks, it, seq, p.budget_ns); break;
      default: ok = pair_mma_tile<128, kPairStages, true, true>(smem, c, tmem_base, g.idesc, g.k_blocks, it, seq, p.budget_ns); break;
    }
    ++seq;
  }
}

// ---- producer warp ------------------------------------------------------------------------------
// All 32 lanes walk the task sequence together. Lane 0 owns every decision and every side effect (queue reads,
// dependency waits, GEMM loads); its verdicts are broadcast with shuffles. The other lanes exist for one thing:
// the K / V stream of a decode-attention task is six TMA boxes per 64 KB chunk, and one thread issues a few TMA
// operations per microsecond only; lanes 0-5 issue the six boxes with ONE warp instruction.

// One GEMM task on lane 0: 1 = carry on, 0 = stop (failure already reported where it has a reporter).
__device__ int producer_gemm_task(const MacoProgram& p, const MacoTaskDesc& d, uint32_t task, uint8_t* smem, const GemmCtrl& c,
                                  const CUtensorMap* tmaps, const AttnPipe& apipe, uint32_t ait, uint32_t& it, int& owner) {
  if (p.debug != 0 && !desc_ok(p, d)) { report_failure(p, MACO_STATUS_BAD_TASK, task, d.type, c.abort_word); return 0; }
  if (!wait_deps(p, d, task, c.abort_word, nullptr)) return 0;
  const MacoGemmArgs& g = d.u.gemm;
  // run-time guarded tile: every role reads the same (final) count after the task's conditions hold
  if ((d.flags & MACO_TF_COUNTED) && ld_relaxed_gpu_u32(g.count_ptr) <= g.count_base) return 1;
  fence_proxy_async_all();           // operands were written by generic-proxy stores of other CTAs
  if (owner == 2 && !attn_ring_drained(apipe, ait)) return 0;
  owner = 1;
  const CUtensorMap* ta = tmaps + g.tmap_a;
  const CUtensorMap* tb = tmaps + g.tmap_b;
  const int sel = (g.bn == 128 ? 4 : 0) | (g.a_mn ? 2 : 0) | ((g.b_mn & 1) ? 1 : 0);
  bool ok;
  // b_mn bit 1: blocked B (256-column tiles only); count_base then holds the weight's total number of k-blocks
  const int b_row0 = (g.b_mn & 2) ? (int)(((uint32_t)g.n0 / 256u * g.count_base + (uint32_t)g.k0 / (uint32_t)kBK) * 256u) : -1;
  switch (sel) {
    case 0: ok = gemm_produce_tile<256, kMkStages, false, false, kMkBN>(smem, c, ta, tb, g.m0, g.n0, g.k0, g.k_blocks, it, p.budget_ns, nullptr, kBK, b_row0); break;
    case 1: ok = gemm_produce_tile<256, kMkStages, false, true, kMkBN>(smem, c, ta, tb, g.m0, g.n0, g.k0, g.k_blocks, it, p.budget_ns); break;
    case 2: ok = gemm_produce_tile<256, kMkStages, true, false, kMkBN>(smem, c, ta, tb, g.m0, g.n0, g.k0, g.k_blocks, it, p.budget_ns); break;
    case 3: ok = gemm_produce_tile<256, kMkStages, true, true, kMkBN>(smem, c, ta, tb, g.m0, g.n0, g.k0, g.k_blocks, it, p.budget_ns); break;
    case 4: ok = gemm_produce_tile<128, kMkStages, false, false, kMkBN>(smem, c, ta, tb, g.m0, g.n0, g.k0, g.k_blocks, it, p.budget_ns); break;
    case 5: ok = gemm_produce_tile<128, kMkStages, false, true, kMkBN>(smem, c, ta, tb, g.m0, g.n0, g.k0, g.k_blocks, it, p.budget_ns); break;
    case 6: ok = gemm_produce_tile<128, kMkStages, true, false, kMkBN>(smem, c, ta, tb, g.m0, g.n0, g.k0, g.k_blocks, it, p.budget_ns); break;
    default: ok = gemm_produce_tile<128, kMkStages, true, true, kMkBN>(smem, c, ta, tb, g.m0, g.n0, g.k0, g.k_blocks, it, p.budget_ns); break;
  }
  if (!ok) report_failure(p, MACO_STATUS_TIMEOUT, task, 0xffffffffu, c.abort_word);
  return ok ? 1 : 0;
}

__device__ void producer_role(const MacoProgram& p, uint32_t w, uint32_t q_base, uint8_t* smem, const GemmCtrl& c,
                              uint64_t* attn_ring_bars) {
  const uint32_t lane = threadIdx.x & 31;
  uint32_t it = 0;                   // stage uses of the GEMM ring (lane 0)
  uint32_t ait = 0;                  // stage uses of the attention ring (same memory); every lane keeps the same count
  int owner = 0;                     // lane 0: which pipeline used the operand memory last: 1 GEMM, 2 attention
  bool ok = true;                    // uniform over the warp
  const CUtensorMap* tmaps = reinterpret_cast<const CUtensorMap*>(p.tmaps);
  const AttnPipe apipe{smem, attn_ring_bars, attn_ring_bars + kAttnStages, p.budget_ns, c.abort_word, tmaps, nullptr, 0,
                       nullptr, nullptr, 0};
  for (uint32_t i = 0; ok; ++i) {
    uint32_t task = 0, verdict = 0;  // 0 run, 1 end of queue, 2 failure
    if (lane == 0) {
      if (!fetch_task(p, w, i, q_base, task, c.abort_word)) verdict = 2;
      else if (task == MACO_QUEUE_TERMINATE) verdict = 1;
    }
    verdict = __shfl_sync(0xffffffffu, verdict, 0);
    task = __shfl_sync(0xffffffffu, task, 0);
    if (verdict == 2) { ok = false; break; }
    if (verdict == 1) break;
    task &= MACO_QUEUE_INDEX_MASK;
    const MacoTaskDesc& d = p.tasks[task];   // read in place (L1/L2 resident): a register copy would cost 32 registers
    if (d.type == MACO_TASK_ATTENTION && attn_pipelined(d.u.elt)) {
      // K / V rows of the split stream through the operand ring; the general warps consume them
      uint32_t go = 1;               // 1 produce, 0 stop silently (the wait reported), 2 stop and report
      if (lane == 0) {
        if (!wait_deps(p, d, task, c.abort_word, nullptr)) {
          go = 0;
        } else {
          fence_proxy_async_all();
          if (owner == 1) {          // the MMA warp may still be reading the last GEMM stages out of this memory
            bool free_ok = true;
            for (uint32_t u = it > (uint32_t)kMkStages ? it - kMkStages : 0; u < it && free_ok; ++u)
              free_ok = mbar_wait(&c.empty[u % kMkStages], (u / kMkStages) & 1, p.budget_ns, c.abort_word);
            if (!free_ok) go = 2;
          }
          owner = 2;
        }
      }
      go = __shfl_sync(0xffffffffu, go, 0);
      if (go == 1 && !attn_produce(d.u.elt, apipe, ait, lane)) go = 2;
      if (go != 1) {
        if (go == 2 && lane == 0) report_failure(p, MACO_STATUS_TIMEOUT, task, 0xffffffffu, c.abort_word);
        ok = false;
      }
      continue;
    }
    if (!is_gemm(d.type)) continue;
    uint32_t carry_on = 1;
    if (lane == 0) carry_on = (uint32_t)producer_gemm_task(p, d, task, smem, c, tmaps, apipe, ait, it, owner);
    carry_on = __shfl_sync(0xffffffffu, carry_on, 0);
    if (carry_on == 0) ok = false;
  }
  if (!ok && lane == 0) { gemm_drain_loads<kMkStages>(c, it); attn_drain_loads(apipe, ait); }
}

// ---- MMA warp (lane 0) --------------------------------------------------------------------------
__device__ void mma_role(const MacoProgram& p, uint32_t w, uint32_t q_base, uint8_t* smem, const GemmCtrl& c,
                         uint32_t tmem_base, volatile uint32_t* attn_done, uint64_t* attn_bars, uint64_t* p_ready,
                         volatile uint32_t* pv_flags, uint8_t* scratch_smem) {
  uint32_t it = 0, seq = 0, attn_seen = 0;
  uint32_t ait = 0, attn_chunks = 0;   // attention ring uses / chunks so far: the same counts the general warps keep
  bool ok = true;
  for (uint32_t i = 0; ok; ++i) {
    uint32_t task;
    if (!fetch_task(p, w, i, q_base, task, c.abort_word)) break;
    if (task == MACO_QUEUE_TERMINATE) break;
    task &= MACO_QUEUE_INDEX_MASK;
    const MacoTaskDesc& d = p.tasks[task];   // read in place (L1/L2 resident): a register copy would cost 32 registers
    if (d.type == MACO_TASK_ATTENTION && attn_pipelined(d.u.elt)) {
      // The attention task issues its own tensor-core products into the low TMEM columns: this warp must
      // not start the next GEMM tile's accumulator there before the general warps have finished the task
      // (CTA-local counter).
      {
        // this warp issues the task's tensor-core products (scores and P.V), the general warps do the softmax
        const AttnPipe pipe{smem, attn_bars + 4, attn_bars + 4 + kAttnStages, p.budget_ns, c.abort_word, nullptr, attn_bars,
                            tmem_base, p_ready, pv_flags, attn_seen};
        if (!attn_mma(d.u.elt, scratch_smem, pipe, ait, attn_chunks)) {
          report_failure(p, MACO_STATUS_TIMEOUT, task, 0xfffffffeu, c.abort_word);
          ok = false;
          break;
        }
        ait += attn_stage_uses(d.u.elt);
        attn_chunks += (uint32_t)((d.u.elt.rows + 127) / 128);
      }
      ++attn_seen;
      const uint64_t t0 = globaltimer_ns();
      while ((int32_t)(*attn_done - attn_seen) < 0) {
        if (*c.abort_word != 0 || globaltimer_ns() - t0 > p.budget_ns) { ok = false; break; }
        __nanosleep(64);
      }
      continue;
    }
    if (!is_gemm(d.type)) continue;
    const MacoGemmArgs& g = d.u.gemm;
    if (d.flags & MACO_TF_COUNTED) {
      if (!wait_deps(p, d, task, c.abort_word, nullptr)) break;
      if (ld_relaxed_gpu_u32(g.count_ptr) <= g.count_base) continue;
    }
    const int sel = (g.bn == 128 ? 4 : 0) | (g.a_mn ? 2 : 0) | ((g.b_mn & 1) ? 1 : 0);
    switch (sel) {
      case 0: ok = gemm_mma_tile<256, kMkStages, false, false, kMkBN>(smem, c, tmem_base, g.idesc, g.k_blocks, it, seq, p.budget_ns); break;
      case 1: ok = gemm_mma_tile<256, kMkStages, false, true, kMkBN>(smem, c, tmem_base, g.idesc, g.k_blocks, it, seq, p.budget_ns); break;
      case 2: ok = gemm_mma_tile<256, kMkStages, true, false, kMkBN>(smem, c, tmem_base, g.idesc, g.k_blocks, it, seq, p.budget_ns); break;
      case 3: ok = gemm_mma_tile<256, kMkStages, true, true, kMkBN>(smem, c, tmem_base, g.idesc, g.k_blocks, it, seq, p.budget_ns); break;
      case 4: ok = gemm_mma_tile<128, kMkStages, false, false, kMkBN>(smem, c, tmem_base, g.idesc, g.k_blocks, it, seq, p.budget_ns); break;
      case 5: ok = gemm_mma_tile<128, kMkStages, false, true, kMkBN>(smem, c, tmem_base, g.idesc, g.k_blocks, it, seq, p.budget_ns); break;
      case 6: ok = gemm_mma_tile<128, kMkStages, true, false, kMkBN>(smem, c, tmem_base, g.idesc, g.k_blocks, it, seq, p.budget_ns); break;
      default: ok = gemm_mma_tile<128, kMkStages, true, true, kMkBN>(smem, c, tmem_base, g.idesc, g.k_blocks, it, seq, p.budget_ns); break;
    }
    ++seq;
  }
}

// Non-GEMM task bodies are kept out of line: each gets its own register allocation, so the
// unrolled copy / reduce / attention loops cannot push spills into the GEMM epilogue.
__device__ __noinline__ bool run_elt(uint32_t type, const MacoEltArgs& a, int tid) { return elt_run(type, a, tid, 128); }
__device__ __noinline__ bool run_comm(const MacoProgram& p, const MacoTaskDesc& d, int tid, BulkCtx* bulk) {
  return comm_run(p, d, tid, 128, bulk);
}
__device__ __noinline__ void run_attn(uint32_t type, const MacoEltArgs& a, int tid, uint8_t* scratch) {
  attn_run(type, a, tid, 128, scratch);
}
__device__ __noinline__ void run_moe(const MacoProgram& p, uint32_t type, const MacoEltArgs& a, int tid, uint8_t* scratch,
                                    BulkCtx* bulk) {
  if (type == MACO_TASK_SPLITK_FIN) splitk_finalize(p, a, tid);
  else if (type == MACO_TASK_MOE_COMBINE) moe_combine(p, a, tid, bulk);
  else if (type == MACO_TASK_TOPK) moe_topk_dispatch(p, a, tid, scratch);
  else if (type == MACO_TASK_MOE_COUNTS) moe_publish_counts(p, a, tid);
  else moe_return(p, a, tid, scratch);
}

// ---- general warps (128 threads): GEMM epilogues and every non-GEMM task -------------------------
// Control words shared by the 128 threads are double buffered by iteration parity, so the
// leader can prepare iteration i+1 while slower threads still read the words of iteration i.
template <int CG>
__device__ void general_role(const MacoProgram& p, uint32_t w, uint32_t q_base, const GemmCtrl& c, uint32_t tmem_base,
                             volatile uint32_t* slots, uint8_t* scratch_smem, uint8_t* ring_smem, uint64_t* bulk_bars,
                             uint64_t* attn_bars, uint64_t* attn_p_ready) {
  const int tid = threadIdx.x - 64;          // 0..127
  // two-CTA programs: the epilogue warps of both CTAs report "accumulator drained" to the leader's barrier
  uint32_t pair_empty_bar = 0;
  if constexpr (CG == 2) pair_empty_bar = mapa_u32(smem_u32(&c.tmem_empty[0]), 0);
  const bool leader = tid == 0;
  // Communication workers never get GEMM tasks, so their operand ring is free to stage bulk copies.
  const bool comm_worker = p.num_comm_workers > 0 && w >= p.num_workers - p.num_comm_workers;
  BulkCtx bulk{ring_smem, bulk_bars, kBulkBuffers, kBulkBufBytes, slots + 12};   // phase word: zeroed at kernel start
  uint32_t seq = 0, done = 0, it = 0;      // it: ring stages consumed so far (kept in step with the TMA and MMA warps)
  uint32_t attn_chunks = 0, ait = 0;       // attention chunks done (parity of its MMA barriers), uses of its ring
  uint32_t attn_tasks = 0;                 // pipelined attention tasks done (parity of the "Q staged" barrier)
  for (uint32_t i = 0;; ++i) {
    volatile uint32_t* cur = slots + (i & 1u) * 4;     // [0] task, [1] dependencies satisfied, [2] failure
    if (leader) {
      uint32_t task;
      if (!fetch_task(p, w, i, q_base, task, c.abort_word)) task = MACO_QUEUE_TERMINATE - 1;   // abort marker
      cur[0] = task;
      cur[2] = 0;
    }
    general_bar();
    const uint32_t raw_entry = cur[0];
    if (raw_entry >= MACO_QUEUE_TERMINATE - 1) {
      const uint32_t task = raw_entry;
      // consume the TERMINATE entry too, so the next launch starts behind it
      if (leader && task == MACO_QUEUE_TERMINATE && p.mode == MACO_MODE_DYNAMIC) st_release_gpu_u32(&p.tails[w], q_base + i + 1);
      break;
    }
    // bit 31 of a static queue entry: no GEMM task follows in this worker's queue, the operand ring is idle
    const uint32_t task = raw_entry & MACO_QUEUE_INDEX_MASK;
    const bool ring_free = comm_worker || (raw_entry & MACO_QUEUE_RING_FREE) != 0;
    const MacoTaskDesc& d = p.tasks[task];   // read in place (L1/L2 resident): a register copy would cost 32 registers
    uint64_t t_start = 0, wait_ns = 0;
    if (leader && p.trace != nullptr) t_start = globaltimer_ns();
    if (p.debug != 0 && !desc_ok(p, d)) {            // uniform over the 128 threads (same descriptor)
      if (leader) report_failure(p, MACO_STATUS_BAD_TASK, task, d.type, c.abort_word);
      break;
    }
    bool skip_tile = false;
    if (is_gemm(d.type) && (d.flags & MACO_TF_COUNTED)) {
      if (leader) {
        const bool okw = wait_deps(p, d, task, c.abort_word, nullptr);
        cur[1] = !okw ? 0u : (ld_relaxed_gpu_u32(d.u.gemm.count_ptr) <= d.u.gemm.count_base ? 2u : 1u);
      }
      general_bar();
      if (cur[1] == 0) cur[2] = 1;
      skip_tile = cur[1] != 1;
    }
    if (is_gemm(d.type) && skip_tile) {
      // nothing to compute: the tile's rows hold no tokens (it still signals below)
    } else if (is_gemm(d.type)) {
      const MacoGemmArgs& g = d.u.gemm;
      const GemmEpilogue& e = p.epis[g.epi];
      void* out_base = e.out;
      if (g.peer >= 0) out_base = p.peer_heap[g.peer] + g.out_off;
      EpiBroadcast bc{p.world, p.peer_heap, g.out_off};       // peer == -2: the tile goes to every rank's heap
      const EpiBroadcast* bcp = g.peer == -2 ? &bc : nullptr;
      bool ok;
      uint8_t* stage = g.peer != -1 ? scratch_smem : nullptr;  // tiles that leave the GPU go through the bulk engine
      // run-time row count of a counted tile's operand block (rows at or beyond it hold no tokens)
      const int row_limit = (d.flags & MACO_TF_COUNTED) ? (int)ld_relaxed_gpu_u32(g.count_ptr) : 0x7fffffff;
      if (g.bn == 128) ok = gemm_epilogue_tile<128, kMkBN>(c, tmem_base, e, out_base, g.row_off, g.m0, g.n0, seq, p.budget_ns, bcp, stage, pair_empty_bar, row_limit);
      else ok = gemm_epilogue_tile<256, kMkBN>(c, tmem_base, e, out_base, g.row_off, g.m0, g.n0, seq, p.budget_ns, bcp, stage, pair_empty_bar, row_limit);
      if (!ok) cur[2] = 1;
      ++seq;
      it += (uint32_t)g.k_blocks;
      if (e.mode == MACO_EPI_SPLITK_FUSED) {
        // Split-K with the finishing pass folded in: every tile adds its partial sums to the workspace and then
        // arrives at its column tile's counter; whoever arrives last finds all K slices summed and finishes the
        // columns here, while this worker's TMA and MMA warps already stream the next tile. (No separate
        // finishing task, no dependency hop between the two.) The counter only grows: `bias_type` arrivals per launch.
        __threadfence();                               // this thread's reductions are performed before the arrival
        general_bar();
        if (leader) {
          uint32_t* ctr = reinterpret_cast<uint32_t*>(const_cast<void*>(e.bias)) + g.n0 / 256;
          cur[3] = ((atomicAdd(ctr, 1u) + 1u) % (uint32_t)e.bias_type) == 0u ? 1u : 0u;
        }
        general_bar();
        if (cur[3] != 0) {
          __threadfence();
          MacoEltArgs fa = *reinterpret_cast<const MacoEltArgs*>(e.aux);
          const int c0 = fa.i0 == 1 ? g.n0 / 2 : g.n0;    // SwiGLU folds 256 workspace columns into 128 outputs
          fa.in0 = reinterpret_cast<const float*>(fa.in0) + g.n0;
          if (fa.i0 == 3) {
            fa.ld_out = g.n0 / 128;                        // first head of this column block; in1 is the parameter block
            fa.cols = 256;
            splitk_finalize(p, fa, tid);
          } else {
          if (fa.in1 != nullptr) fa.in1 = reinterpret_cast<const uint16_t*>(fa.in1) + c0;
          fa.in2 = reinterpret_cast<const void*>(reinterpret_cast<unsigned long long>(fa.in2) + (unsigned long long)c0 * 2ull);
          if (fa.out != nullptr) fa.out = reinterpret_cast<uint16_t*>(fa.out) + c0;
          fa.cols = fa.i0 == 1 ? 128 : 256;
          splitk_finalize(p, fa, tid);
          }
        }
      }
    } else {
      if (leader) cur[1] = wait_deps(p, d, task, c.abort_word, p.trace ? &wait_ns : nullptr) ? 1u : 0u;
      general_bar();
      if (cur[1] != 0) {
        if (d.type >= 200 && d.type < 300) {
          if (!run_comm(p, d, tid, ring_free ? &bulk : nullptr)) {
            cur[2] = 1;
            if (leader) report_failure(p, MACO_STATUS_BAD_TASK, task, d.u.comm.op, c.abort_word);
          }
        } else if (d.type == MACO_TASK_ATTENTION && attn_pipelined(d.u.elt)) {
          if constexpr (CG == 1) {
            const AttnPipe pipe{ring_smem, attn_bars + 4, attn_bars + 4 + kAttnStages, p.budget_ns, c.abort_word,
                                nullptr, attn_bars, tmem_base, attn_p_ready, slots + 20, attn_tasks};
            if (!attn_consume(d.u.elt, tid, scratch_smem, pipe, ait, attn_chunks)) cur[2] = 1;
            ait += attn_stage_uses(d.u.elt);
            ++attn_tasks;
            general_bar();
            if (leader) slots[13] = slots[13] + 1;                 // lets the MMA warp move past this task
          } else {
            // the tensor-core attention task issues one-CTA MMAs; a kernel has one cta_group (the builder
            // keeps such tasks out of two-CTA programs)
            cur[2] = 1;
            if (leader) report_failure(p, MACO_STATUS_BAD_TASK, task, d.type, c.abort_word);
          }
        } else if (d.type == MACO_TASK_ATTENTION || d.type == MACO_TASK_ATTN_MERGE) {
          run_attn(d.type, d.u.elt, tid, scratch_smem);
        } else if (d.type == MACO_TASK_TOPK || d.type == MACO_TASK_MOE_COUNTS || d.type == MACO_TASK_MOE_RETURN ||
                   d.type == MACO_TASK_SPLITK_FIN || d.type == MACO_TASK_MOE_COMBINE) {
          run_moe(p, d.type, d.u.elt, tid, scratch_smem, ring_free ? &bulk : nullptr);
        } else if (d.type != MACO_TASK_NOP) {
          if (!run_elt(d.type, d.u.elt, tid)) {
            cur[2] = 1;
            if (leader) report_failure(p, MACO_STATUS_BAD_TASK, task, d.type, c.abort_word);
          }
        }
      } else if (leader) {
        cur[2] = 1;
      }
    }
    if (leader && *c.abort_word != 0) cur[2] = 1;
    general_bar();                              // every thread's stores are issued, failure word final
    if (cur[2] != 0) break;
    if (leader) {
      fence_proxy_async_all();                  // later TMA reads of this output by other CTAs
      signal_done(p, d);
      ++done;
      if (p.mode == MACO_MODE_DYNAMIC) st_release_gpu_u32(&p.tails[w], q_base + i + 1);
      if (p.trace != nullptr) {
        MacoTraceRecord r;
        r.task = task; r.type = d.type; r.sm = (uint16_t)smid(); r.t_start_ns = t_start; r.t_end_ns = globaltimer_ns();
        r.wait_ns = wait_ns;
        p.trace[task] = r;
      }
    }
  }
  if (leader && done != 0 && p.counters != nullptr) atomicAdd(&p.counters[0], done);
}

// ---- scheduler CTA (warp 0) ---------------------------------------------------------------------
__device__ bool sched_push(const MacoProgram& p, uint32_t* heads_sm, uint32_t w, uint32_t task) {
  const uint32_t head = heads_sm[w];
  // back-pressure: never run more than a ring ahead of the consumer
  if (!mk_wait(p, &p.tails[w], head + 1 - MACO_WORKER_QUEUE_SIZE, false)) return false;
  st_relaxed_gpu_u32(&p.ring[(size_t)w * MACO_WORKER_QUEUE_SIZE + (head & (MACO_WORKER_QUEUE_SIZE - 1))], task);
  st_release_gpu_u32(&p.heads[w], head + 1);
  heads_sm[w] = head + 1;
  return true;
}

__device__ void scheduler_role(const MacoProgram& p, uint32_t* heads_sm) {
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t W = p.num_workers;
  const uint32_t n_comm = p.num_comm_workers < W ? p.num_comm_workers : 0;
  const uint32_t n_compute = W - n_comm;
  for (uint32_t w = lane; w < W; w += 32) heads_sm[w] = ld_relaxed_gpu_u32(&p.heads[w]);
  __syncwarp();
  uint32_t base = 0;                 // first group not yet dispatched
  uint32_t window_done = 0;          // bit i: group base+i dispatched
  uint32_t rr_compute = 0, rr_comm = 0;
  uint64_t last_progress = globaltimer_ns();
  bool ok = true;
  while (ok && base < p.num_groups) {
    const uint32_t g = base + lane;
    bool ready = false;
    MacoGroupDesc gd;
    if (g < p.num_groups && !((window_done >> lane) & 1u)) {
      gd = p.groups[g];
      ready = true;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int e = gd.wait_event[j];
        if (e < 0) continue;
        const bool sys = (gd.flags & (j == 0 ? MACO_TF_WAIT0_SYS : MACO_TF_WAIT1_SYS)) != 0;
        const bool prev = (gd.flags & (j == 0 ? MACO_TF_WAIT0_PREV : MACO_TF_WAIT1_PREV)) != 0;
        const uint32_t v = sys ? ld_acquire_sys_u32(&p.events[e]) : ld_acquire_gpu_u32(&p.events[e]);
        if ((int32_t)(v - (p.epoch - (prev ? 1u : 0u)) * gd.wait_count[j]) < 0) ready = false;
      }
    }
    uint32_t mask = __ballot_sync(0xffffffffu, ready);
    if (mask == 0) {
      if (lane == 0 && (aborted(p) || globaltimer_ns() - last_progress > p.budget_ns)) {
        report_failure(p, MACO_STATUS_TIMEOUT, 0xfffffffdu, base, nullptr);
        ok = false;
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      __nanosleep(64);
      continue;
    }
    while (mask != 0 && ok) {
      const int b = __ffs(mask) - 1;
      mask &= mask - 1;
      const uint32_t first = __shfl_sync(0xffffffffu, gd.first_task, b);
      const uint32_t count = __shfl_sync(0xffffffffu, gd.num_tasks, b);
      const uint32_t gflags = __shfl_sync(0xffffffffu, gd.flags, b);
      const bool to_comm = (gflags & MACO_TF_COMM_WORKER) != 0 && n_comm > 0;
      const uint32_t n_target = to_comm ? n_comm : n_compute;
      const uint32_t w_off = to_comm ? n_compute : 0;
      uint32_t rr = to_comm ? rr_comm : rr_compute;
      // 32 pushes at a time, one lane per distinct worker (fewer lanes when there are fewer workers)
      const uint32_t par = n_target < 32 ? n_target : 32;
      for (uint32_t t0 = 0; t0 < count && ok; t0 += par) {
        bool lane_ok = true;
        if (lane < par && t0 + lane < count) {
          const uint32_t w = w_off + (rr + t0 + lane) % n_target;
          lane_ok = sched_push(p, heads_sm, w, first + t0 + lane);
        }
        if (!__all_sync(0xffffffffu, lane_ok)) {
          if (lane == 0) report_failure(p, MACO_STATUS_QUEUE_OVERFLOW, first, 0, nullptr);
          ok = false;
        }
        __syncwarp();
      }
      rr = (rr + count) % n_target;
      if (to_comm) rr_comm = rr; else rr_compute = rr;
      window_done |= 1u << b;
    }
    last_progress = globaltimer_ns();
    while (window_done & 1u) { window_done >>= 1; ++base; }
  }
  // End of program (or abort): close every ring so the workers leave.
  for (uint32_t w = lane; w < W; w += 32) sched_push(p, heads_sm, w, MACO_QUEUE_TERMINATE);
}

template <int CG>
__device__ __forceinline__ void persistent_body(const MacoProgram& p) {
  extern __shared__ uint8_t dyn_smem[];
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool is_worker = blockIdx.x < p.num_workers;
  GemmCtrl c;
  uint32_t tmem_base;
  uint8_t* smem;
  if constexpr (CG == 2) smem = pair_cta_setup<kPairStages>(dyn_smem, c, tmem_base);
  else smem = gemm_cta_setup<kMkBN, kMkStages>(dyn_smem, c, tmem_base, is_worker);
  uint32_t* extra = reinterpret_cast<uint32_t*>(smem + MkLayout::kRingBytes + MkLayout::kCtrlBytes);
  if (is_worker) {
    const uint32_t w = blockIdx.x;
    // All roles must start from the same ring position: one thread reads it before anyone can move it.
    uint64_t* bulk_bars = reinterpret_cast<uint64_t*>(extra + 32);          // bytes 128.. of the extra block
    uint64_t* attn_bars = reinterpret_cast<uint64_t*>(extra + 64);          // bytes 256..383: 4 MMA barriers, then full[6], empty[6] of the K/V ring
    uint64_t* attn_p_ready = reinterpret_cast<uint64_t*>(extra + 96);       // bytes 384..407: P staged (two buffers), Q staged; words 20, 21: P.V accumulate flags
    if (threadIdx.x == 0) {
      extra[16] = p.mode == MACO_MODE_DYNAMIC ? ld_relaxed_gpu_u32(&p.tails[w]) : 0;
      extra[12] = 0;                                                     // parity bits of the bulk barriers
      extra[13] = 0;                                                     // pipelined attention tasks finished
      for (uint32_t b = 0; b < kBulkBuffers; ++b) mbar_init(&bulk_bars[b], 1);
      for (int b = 0; b < 4 + 2 * kAttnStages; ++b) mbar_init(&attn_bars[b], 1);   // attention: 4 MMA barriers, ring full / empty
      for (int b = 0; b < 3; ++b) mbar_init(&attn_p_ready[b], 1);
      extra[20] = 0; extra[21] = 0;
      fence_mbar_init();
    }
    __syncthreads();
    const uint32_t q_base = extra[16];
    if (warp == 0) {
      if constexpr (CG == 2) {
        if (lane == 0) producer_role_pair(p, w, q_base, smem, c);
      } else {
        producer_role(p, w, q_base, smem, c, attn_bars + 4);          // all 32 lanes (see the role)
      }
      __syncwarp();
    } else if (warp == 1) {
      if (lane == 0) {
        if constexpr (CG == 2) { if (cluster_ctarank() == 0) mma_role_pair(p, w, q_base, smem, c, tmem_base); }
        else mma_role(p, w, q_base, smem, c, tmem_base, extra + 13, attn_bars, attn_p_ready, extra + 20,
                      reinterpret_cast<uint8_t*>(extra) + kMkExtraSmem);
      }
      __syncwarp();
    } else {
      general_role<CG>(p, w, q_base, c, tmem_base, extra, reinterpret_cast<uint8_t*>(extra) + kMkExtraSmem, smem, bulk_bars, attn_bars,
                       attn_p_ready);
    }
  } else {
    if constexpr (CG == 1) { if (warp == 0) scheduler_role(p, extra); }
  }
  if constexpr (CG == 2) pair_cta_teardown(c, tmem_base, nullptr);
  else gemm_cta_teardown<kMkBN>(c, tmem_base, nullptr, is_worker);
}

__global__ void __launch_bounds__(kGemmThreads, 1) maco_persistent_kernel(const __grid_constant__ MacoProgram p) {
  persistent_body<1>(p);
}

// The same kernel for programs whose GEMM tasks are halves of two-CTA tiles: launched as clusters of two
// CTAs (workers 2j and 2j+1), every tcgen05 instruction in its cta_group::2 form, static queues only.
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
maco_persistent_pair_kernel(const __grid_constant__ MacoProgram p) {
  persistent_body<2>(p);
}

__global__ void maco_grid_barrier_demo_kernel(uint32_t* counter, uint32_t* order, float* data, int n_per_cta,
                                              int num_tasks, uint64_t budget_ns, uint32_t* status) {
  // Self-test of the atoms: every CTA updates its slice, then all CTAs meet at a counter barrier
  // (atom.add.release.gpu + bounded ld.acquire.gpu spin), num_tasks times. The launcher clamps
  // the grid to what is co-resident, which the reference's demo kernel
  // (maco/csrc/maco_kernel.cu:154-198) does not, so that one can deadlock.
  float* mine = data + (size_t)blockIdx.x * n_per_cta;
  for (int t = 0; t < num_tasks; ++t) {
    for (int i = threadIdx.x; i < n_per_cta; i += blockDim.x) mine[i] = mine[i] * 1.5f + 0.1f;
    __syncthreads();
    if (threadIdx.x == 0) {
      const uint32_t ticket = atom_add_release_gpu_u32(counter, 1);
      if (order != nullptr) order[ticket] = blockIdx.x;
      if (!wait_flag_ge_u32<false>(counter, (uint32_t)(t + 1) * gridDim.x, budget_ns)) {
        st_relaxed_sys_u32(status, MACO_STATUS_TIMEOUT);
      }
    }
    __syncthreads();
  }
}

}  // namespace

extern "C" {

int maco_abi_sizes(int* task, int* group, int* program, int* epilogue, int* trace, int* tmap) {
  *task = sizeof(MacoTaskDesc); *group = sizeof(MacoGroupDesc); *program = sizeof(MacoProgram);
  *epilogue = sizeof(GemmEpilogue); *trace = sizeof(MacoTraceRecord); *tmap = sizeof(CUtensorMap);
  return 0;
}

int maco_persistent_smem_bytes() { return kMkSmemBytes; }

// Number of two-CTA clusters of the persistent kernel that can be resident at once on the current device
// (0 = unknown before the first launch; the launcher refuses programs that need more).
int maco_persistent_max_pairs() {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * 74, 1, 1); cfg.blockDim = dim3(kGemmThreads, 1, 1); cfg.dynamicSmemBytes = kMkSmemBytes;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension; at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  if (cudaFuncSetAttribute(maco_persistent_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMkSmemBytes) != cudaSuccess) return -1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, maco_persistent_pair_kernel, &cfg) != cudaSuccess) { (void)cudaGetLastError(); return -1; }
  return n;
}

// Encodes one operand tensor map into `out` (128 bytes, host memory).
int maco_encode_operand_tmap(void* out, const void* base, int rows_or_k, int cols, long long ld_elems, int mn_major,
                             int box_rows) {
  CUtensorMap* tm = reinterpret_cast<CUtensorMap*>(out);
  // K-major operand [rows, K]: box = 64 (K) x box_rows. MN-major operand stored [K, rows]: box = 64 (rows) x 64 (K).
  if (!mn_major) return maco_host::encode_tmap_2d(tm, base, 2, rows_or_k, cols, ld_elems * 2, kBK, box_rows);
  return maco_host::encode_tmap_2d(tm, base, 2, rows_or_k, cols, ld_elems * 2, 64, kBK);
}

int maco_program_launch(const MacoProgram* prog, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  static bool attr_set[64] = {};
  static int max_pairs[64] = {};
  int dev = 0;
  MACO_CHECK_CUDA(cudaGetDevice(&dev));
  if (!attr_set[dev]) {
    MACO_CHECK_CUDA(cudaFuncSetAttribute(maco_persistent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMkSmemBytes));
    MACO_CHECK_CUDA(cudaFuncSetAttribute(maco_persistent_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMkSmemBytes));
    // how many two-CTA clusters can be resident at once (every CTA of a program must be)
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * 74, 1, 1); cfg.blockDim = dim3(kGemmThreads, 1, 1); cfg.dynamicSmemBytes = kMkSmemBytes;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension; at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, maco_persistent_pair_kernel, &cfg) != cudaSuccess) { n = 0; (void)cudaGetLastError(); }
    max_pairs[dev] = n;
    attr_set[dev] = true;
  }
  MacoProgram p = *prog;
  if (p.status == nullptr) p.status = reinterpret_cast<MacoStatusBlock*>(maco_host::status_device_ptr());
  const int sms = maco_host::sm_count();
  const int grid = (int)p.num_workers + (p.mode == MACO_MODE_DYNAMIC ? 1 : 0);
  if (grid > sms) {
    // All CTAs must be resident at once (1 per SM): a queued CTA could hold the task another one waits for.
    maco_host::set_error("persistent kernel: workers + scheduler exceed the number of SMs");
    return -1;
  }
  if (p.num_workers == 0 || p.num_workers > MACO_MAX_WORKERS) { maco_host::set_error("bad worker count"); return -1; }
  if (p.cta_group == 2) {
    if (p.mode != MACO_MODE_STATIC || (p.num_workers & 1u)) {
      maco_host::set_error("two-CTA programs need static queues and an even number of workers");
      return -1;
    }
    if ((int)p.num_workers / 2 > max_pairs[dev]) {
      maco_host::set_error("two-CTA program: more CTA pairs than can be resident at once");
      return -1;
    }
    maco_persistent_pair_kernel<<<grid, kGemmThreads, kMkSmemBytes, stream>>>(p);
    MACO_CHECK_CUDA(cudaGetLastError());
    return 0;
  }
  maco_persistent_kernel<<<grid, kGemmThreads, kMkSmemBytes, stream>>>(p);
  MACO_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// Runs the barrier self-test; returns elapsed milliseconds (device-timed) or a negative error.
float maco_run_sm_scheduling_demo(float* data, int n_total, int num_ctas, int threads, int num_tasks,
                                  uint32_t* order_out_dev, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  int sms = maco_host::sm_count();
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, maco_grid_barrier_demo_kernel, threads, 0) != cudaSuccess) return -1.f;
  if (num_ctas > sms * per_sm) { maco_host::set_error("demo: more CTAs than can be co-resident"); return -2.f; }
  uint32_t* counter = nullptr;
  if (cudaMalloc(&counter, sizeof(uint32_t)) != cudaSuccess) return -1.f;
  cudaMemsetAsync(counter, 0, sizeof(uint32_t), stream);
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0); cudaEventCreate(&e1);
  cudaEventRecord(e0, stream);
  maco_grid_barrier_demo_kernel<<<num_ctas, threads, 0, stream>>>(counter, order_out_dev, data, n_total / num_ctas, num_tasks,
                                                                 2000000000ull, maco_host::status_device_ptr());
  cudaEventRecord(e1, stream);
  cudaError_t err = cudaEventSynchronize(e1);
  float ms = -1.f;
  if (err == cudaSuccess) cudaEventElapsedTime(&ms, e0, e1);
  cudaEventDestroy(e0); cudaEventDestroy(e1);
  cudaFree(counter);
  return ms;
}

}  // extern "C"
