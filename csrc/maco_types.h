// Shared host/device ABI of the persistent task kernel and the stand-alone operators.
//
// Counterpart of the reference's maco/csrc/maco_types.h:19-231, redesigned: tasks are
// tile-granular, carry two wait conditions and a local plus an optional remote (peer GPU)
// signal, and the numeric task-type values are the SAME as the Python TaskType enum
// (the reference's two enums disagree: maco/task_graph/__init__.py:65-89 vs
// maco_types.h:41-68).
#pragma once
#include <stdint.h>

#define MACO_MAX_WORKERS 256
#define MACO_WORKER_QUEUE_SIZE 1024      /* ring entries per worker (power of two) */
#define MACO_MAX_EVENTS 65536
#define MACO_MAX_PEERS 16

/* ---- element types -------------------------------------------------------------------------- */
enum MacoDType { MACO_DT_BF16 = 0, MACO_DT_F16 = 1, MACO_DT_F32 = 2 };

/* ---- task types: values match the Python TaskType enum ------------------------------------ */
enum MacoTaskType {
  MACO_TASK_TERMINATE = 0,
  MACO_TASK_NOP = 1,
  MACO_TASK_MATMUL = 100,        /* one 128 x BN GEMM tile */
  MACO_TASK_LINEAR = 101,
  MACO_TASK_ATTENTION = 102,     /* split-KV decode attention, one (batch, kv-head, split) */
  MACO_TASK_LAYERNORM = 103,
  MACO_TASK_RMSNORM = 104,
  MACO_TASK_GELU = 105,
  MACO_TASK_SILU = 106,
  MACO_TASK_SOFTMAX = 107,
  MACO_TASK_SILU_GATE = 108,
  MACO_TASK_ROPE = 109,
  MACO_TASK_TOPK = 110,
  MACO_TASK_ATTN_MERGE = 111,
  MACO_TASK_SCALE = 112,
  MACO_TASK_ADD = 113,
  MACO_TASK_GELU_BWD = 114,
  MACO_TASK_AXPBY = 115,         /* out = f0 * in0 + f1 * in1 */
  MACO_TASK_MOE_RETURN = 116,    /* expert output rows -> weighted -> back to the source rank's combine buffer */
  MACO_TASK_MOE_COUNTS = 117,    /* publish this rank's per-expert token counts to the expert owners */
  MACO_TASK_MOE_COMBINE = 119,   /* out[token] = sum of the token's k returned rows (bulk-staged when the operand ring is idle) */
  MACO_TASK_SPLITK_FIN = 118,    /* split-K GEMM: fp32 partial-sum buffer -> epilogue op -> 16-bit output (local or every rank) */
  MACO_TASK_CUSTOM_COMPUTE = 150,
  MACO_TASK_ALLREDUCE = 200,     /* reduce one chunk over all peers' buffers, write to all */
  MACO_TASK_ALLGATHER = 201,     /* push one chunk of the local shard to every peer */
  MACO_TASK_REDUCE_SCATTER = 202,/* sum one chunk of this rank's slab over P staged partials */
  MACO_TASK_ALL_TO_ALL = 203,    /* push one chunk to one peer */
  MACO_TASK_BROADCAST = 204,
  MACO_TASK_PEER_BARRIER = 205,
  MACO_TASK_CUSTOM_COMM = 250,
  MACO_TASK_COPY = 300,
  MACO_TASK_FILL = 301           /* out[0 .. rows*cols) 32-bit words = i0 */
};

/* ---- GEMM epilogue ------------------------------------------------------------------------ */
enum MacoEpilogueMode {
  MACO_EPI_STORE = 0,      /* out = alpha * acc (+ bias) */
  MACO_EPI_GELU = 1,       /* out = gelu(alpha * acc + bias) */
  MACO_EPI_SWIGLU = 2,     /* tile = [gate | up]; out[:, n/2] = silu(gate) * up */
  MACO_EPI_F32_STORE = 3,  /* fp32 out = alpha * acc */
  MACO_EPI_F32_ACC = 4,    /* fp32 out += alpha * acc */
  MACO_EPI_GELU_BWD = 5,   /* out = alpha * acc * gelu'(aux) */
  MACO_EPI_SILU = 6,
  MACO_EPI_RESIDUAL = 7,   /* out = alpha * acc + bias + aux */
  MACO_EPI_F32_ATOMIC = 8, /* fp32 out += alpha * acc with atomic adds: split-K partial tiles share one buffer */
  /* As F32_ATOMIC, and the tile that arrives LAST for its 256 columns finishes them (sum -> operator -> 16-bit
     output, workspace zeroed again). The record's other fields change meaning: `bias` = uint32 arrival counters,
     one per 256-column tile, never reset; `bias_type` = arrivals per column tile (the K slices); `aux` = a
     MacoEltArgs in device memory written as for a SPLITK_FIN task over ALL columns (the kernel offsets it to the
     tile's columns). */
  MACO_EPI_SPLITK_FUSED = 9,
  /* Row scatter with a per-row weight (the MoE combine all-to-all fused into the down projection): row r of the
     tile's operand block has a 16-byte record {int32 token, int32 k, float weight, pad} at `aux`[r]; the 16-bit
     output row goes to row token * bias_type + k of the destination (ld_out elements per row), scaled by the weight
     after rounding the product to the output type. Rows at or beyond the task's run-time count are not written. */
  MACO_EPI_SCATTER_ROWS = 10
};

struct GemmEpilogue {
  void* out;
  const void* bias;
  const void* aux;
  long long ld_out;     /* row stride of out, in elements */
  long long ld_aux;
  int mode;             /* MacoEpilogueMode */
  int out_type;         /* MacoDType */
  int bias_type;
  int aux_type;
  int M, N;             /* logical extent of the accumulator grid (rows, columns before any fold) */
  float alpha;
  /* MACO_EPI_RESIDUAL with several aux blocks of the same shape (the staging slots of a reduce-scatter): bits 0-3
     number of blocks (0 or 1: the single `aux`), bits 4-7 index of a block to leave out (15: none), bits 8-31
     rows between consecutive blocks (block s starts `s * rows` rows, of ld_aux elements, behind `aux`). */
  int aux_pack;
};

/* ---- status words written by kernels, read by the host --------------------------------------- */
enum MacoStatus {
  MACO_STATUS_OK = 0,
  MACO_STATUS_TIMEOUT = 1,        /* a bounded wait ran out */
  MACO_STATUS_BAD_TASK = 2,       /* unknown task type / descriptor out of range */
  MACO_STATUS_QUEUE_OVERFLOW = 4,
  MACO_STATUS_PEER_TIMEOUT = 8    /* a wait on another GPU's flag ran out */
};

struct MacoStatusBlock {          /* lives in host-mapped pinned memory */
  uint32_t status;                /* OR of MacoStatus bits */
  uint32_t task;                  /* task index of the first failed wait */
  uint32_t event;                 /* event it waited on */
  uint32_t cta;
  uint32_t rank;
  uint32_t tasks_completed;
  uint32_t _pad[2];
};

/* ---- task descriptor (128 bytes) ---------------------------------------------------------- */
struct MacoGemmArgs {             /* one output tile */
  uint16_t tmap_a, tmap_b;        /* indices into the tensor-map table */
  uint16_t epi;                   /* index into the epilogue table */
  uint8_t a_mn, b_mn;             /* operand majors (bit 0: MN-major). b_mn bit 1: B is stored tile by tile ([N/256][K/64][256][64]); count_base = its total k-blocks */
  int32_t m0, n0, k0, k_blocks;
  uint32_t idesc;
  int32_t peer;                   /* -1: store to the epilogue's out; >= 0: into that rank's heap at out_off; -2: into every rank's heap at out_off */
  long long row_off;              /* added to the row index on store */
  uint64_t out_off;               /* with peer >= 0: byte offset of the destination inside the peer's heap */
  uint32_t bn;                    /* tile width: 128 or 256 */
  uint32_t count_base;            /* MACO_TF_COUNTED: the tile is skipped when *count_ptr <= count_base */
  const uint32_t* count_ptr;
};

struct MacoEltArgs {              /* row-wise / element-wise task over rows [row0, row0+rows) */
  const void* in0;
  const void* in1;
  const void* in2;
  void* out;
  int32_t row0, rows, cols;
  int32_t dtype;
  int32_t ld_in, ld_out;
  float f0, f1;
  int32_t i0, i1;
};

/* Parameter block of the "QK-norm + RoPE + cache scatter" finishing pass of a split-K QKV projection (SPLITK_FIN
   operator 3): column block h of the fp32 sums is head h; heads [0, hq) are queries (per-head RMSNorm with q_norm,
   RoPE, row r -> q_out[r, h, :]), heads [hq, hq + hkv) keys (k_norm, RoPE, -> k_cache[r, h - hq, pos, :]), the last hkv
   heads values (copied -> v_cache[r, j, pos, :]). head_dim 128, 16-bit outputs; cos_sin is [rows, 128] with the
   cosines of a row in its first 64 entries and the sines in the last 64. Strides in elements. */
struct MacoQkRopeParams {
  void* q_out;
  void* k_cache;
  void* v_cache;
  const void* q_norm;
  const void* k_norm;
  const void* cos_sin;
  long long kv_batch_stride, kv_head_stride;
  int32_t hq, hkv, pos, dtype;
  float eps;
  int32_t _pad;
};

struct MacoCommArgs {             /* 2-D block (rows x row_bytes) of a buffer in the symmetric heap */
  uint64_t src_off;               /* byte offset of the source inside a rank's heap */
  uint64_t dst_off;               /* byte offset of the destination inside a rank's heap */
  uint64_t src_stride, dst_stride;/* bytes between rows */
  uint32_t row_bytes, rows;
  int32_t dtype;                  /* element type for reductions */
  int32_t peer;                   /* push: destination rank (-1 = every other rank, -3 = every rank incl. self) */
  int32_t op;                     /* MacoCommOp */
  int32_t nslots;                 /* local reduce: number of slots summed */
  uint64_t slot_stride;           /* local reduce: bytes between slots */
  void* local_ptr;                /* optional destination outside the heap (reductions) */
  float scale;                    /* applied to reduced values (1/world for an average) */
  int32_t _pad;
  const void* aux_ptr;            /* reductions: optional block added to the sum (e.g. a residual), laid out like the destination */
};

enum MacoCommOp {
  MACO_COMM_PUSH = 0,             /* copy my block into peer heap(s) */
  MACO_COMM_REDUCE_LOCAL = 1,     /* out = scale * sum of nslots blocks of my own heap */
  MACO_COMM_REDUCE_PULL = 2,      /* out = scale * sum over ranks of heap[r] + src_off (reads peers) */
  MACO_COMM_ALLREDUCE = 3,        /* pull-reduce one block from every rank, store the result to every rank */
  MACO_COMM_ALLREDUCE_MC = 4,     /* same through the NVSwitch multicast address (multimem) */
  MACO_COMM_PULL = 5,             /* copy a block of peer `peer`'s heap into my heap */
  MACO_COMM_REDUCE_LOCAL_BCAST = 6,/* sum `nslots` local slots (filled by the peers' stores) and write the result to dst_off on EVERY rank */
  MACO_COMM_PUSH_MC = 7           /* copy my block to dst_off of EVERY rank with multimem.st through the NVSwitch multicast address */
};

struct MacoTaskDesc {
  uint16_t type;                  /* MacoTaskType */
  uint16_t flags;                 /* MACO_TF_* */
  uint32_t node_id;
  int32_t wait_event[2];          /* -1: no condition; else wait until events[e] >= epoch * wait_count */
  uint32_t wait_count[2];
  int32_t signal_event[2];        /* local events bumped by 1 at completion, -1 none */
  int32_t signal_peer;            /* rank whose event table is bumped, -1 none, -2 every rank (one red per rank),
                                     -4 every rank with ONE multimem.red on the multicast address of the table */
  int32_t signal_peer_event;
  union {
    MacoGemmArgs gemm;
    MacoEltArgs elt;
    MacoCommArgs comm;
    uint8_t raw[88];
  } u;
};

enum MacoTaskFlags {
  MACO_TF_WAIT0_SYS = 1,          /* wait_event[0] is bumped by other GPUs: poll with .sys scope */
  MACO_TF_WAIT1_SYS = 2,
  MACO_TF_COMM_WORKER = 4,        /* prefers a communication worker */
  MACO_TF_SIGNAL_SYS = 8,         /* local signals use .sys scope (another GPU polls them) */
  MACO_TF_WAIT0_PREV = 16,        /* wait_event[0] refers to the previous launch: (epoch-1) * count */
  MACO_TF_WAIT1_PREV = 32,
  MACO_TF_ANY_WORKER = 64,        /* host-side placement hint only */
  MACO_TF_COUNTED = 128           /* GEMM tile guarded by a row count known only at run time (MoE) */
};

/* A dispatch group for the scheduler CTA: a run of consecutive tasks that becomes ready together. */
struct MacoGroupDesc {
  uint32_t first_task, num_tasks;
  int32_t wait_event[2];
  uint32_t wait_count[2];
  uint32_t flags;                 /* MACO_TF_* */
  uint32_t _pad;
};

#define MACO_QUEUE_TERMINATE 0xffffffffu
#define MACO_QUEUE_RING_FREE 0x80000000u   /* static queue entry: no GEMM task follows in this queue */
#define MACO_QUEUE_INDEX_MASK 0x7fffffffu

enum MacoKernelMode { MACO_MODE_STATIC = 0, MACO_MODE_DYNAMIC = 1 };

/* Everything one launch of the persistent kernel needs; passed by value. */
struct MacoProgram {
  const struct MacoTaskDesc* tasks;
  const void* tmaps;              /* CUtensorMap[ ] (128 bytes each, 64-byte aligned) */
  const struct GemmEpilogue* epis;
  uint32_t* events;               /* monotonic counters, never reset; threshold scales with epoch */
  uint32_t* peer_events[MACO_MAX_PEERS];
  uint8_t* peer_heap[MACO_MAX_PEERS];
  const uint32_t* static_queue;   /* [num_workers][static_stride] task indices */
  const uint32_t* static_count;   /* [num_workers] */
  uint32_t* ring;                 /* [num_workers][MACO_WORKER_QUEUE_SIZE] (dynamic mode) */
  uint32_t* heads;                /* [num_workers] published by the scheduler */
  uint32_t* tails;                /* [num_workers] published by the workers */
  const struct MacoGroupDesc* groups;
  uint32_t* abort_word;           /* == epoch when some wait of this launch gave up */
  uint32_t* counters;             /* [0] tasks completed (all launches); may be null */
  uint8_t* mc_heap;               /* multicast (NVLS) address of the symmetric heap, or null */
  struct MacoStatusBlock* status;
  struct MacoTraceRecord* trace;  /* [num_tasks] or null */
  unsigned long long budget_ns;
  uint32_t num_tasks, num_groups, num_workers, num_comm_workers;
  uint32_t static_stride, mode, epoch;
  int32_t rank, world;
  uint32_t cta_group;             /* 1: one-CTA GEMM tiles; 2: every GEMM task is half of a two-CTA tile (cluster launch) */
  uint32_t debug;                 /* non-zero: workers re-check every descriptor (events, peers, heap extents) before running it */
  uint64_t heap_bytes;            /* size of each rank's symmetric heap (0: no heap) */
  uint32_t num_events, num_tmaps, num_epis, _pad;
};

#ifdef __cplusplus
static_assert(sizeof(MacoTaskDesc) == 128, "task descriptor must stay 128 bytes");
#endif

/* ---- mixture-of-experts layer constants (one per layer, in device memory) --------------------- */
struct MacoMoeParams {
  const void* logits;             /* [tokens, experts] router output (16-bit) */
  const void* x;                  /* [tokens, hidden] */
  uint32_t* counts;               /* [experts] slots handed out by this rank, zero at launch start */
  void* comb;                     /* [tokens, top_k, hidden] combine buffer of this rank (inside the heap) */
  unsigned long long recv_off;    /* heap offset: recv [experts_per_rank][world][capacity][hidden] */
  unsigned long long meta_off;    /* heap offset: meta [experts_per_rank][world][capacity] x {token, k, weight, -} */
  unsigned long long cnt_off;     /* heap offset: received counts [world][experts_per_rank] (uint32) */
  unsigned long long comb_off;    /* heap offset of comb */
  const void* y;                  /* [experts_per_rank][world][capacity][hidden] expert outputs (local) */
  int32_t hidden, experts, top_k, experts_per_rank, capacity, tokens, dtype, _pad;
};

/* ---- device trace ring ----------------------------------------------------------------------- */
struct MacoTraceRecord {
  uint32_t task;
  uint16_t type;
  uint16_t sm;
  uint64_t t_start_ns;            /* %globaltimer */
  uint64_t t_end_ns;
  uint64_t wait_ns;               /* time spent in dependency waits before the task body */
};
