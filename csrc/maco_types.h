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
  MACO_TASK_CUSTOM_COMPUTE = 150,
  MACO_TASK_ALLREDUCE = 200,     /* reduce one chunk over all peers' buffers, write to all */
  MACO_TASK_ALLGATHER = 201,     /* push one chunk of the local shard to every peer */
  MACO_TASK_REDUCE_SCATTER = 202,/* sum one chunk of this rank's slab over P staged partials */
  MACO_TASK_ALL_TO_ALL = 203,    /* push one chunk to one peer */
  MACO_TASK_BROADCAST = 204,
  MACO_TASK_PEER_BARRIER = 205,
  MACO_TASK_CUSTOM_COMM = 250,
  MACO_TASK_COPY = 300
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
  MACO_EPI_RESIDUAL = 7    /* out = alpha * acc + bias + aux */
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
  int _pad;
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
  uint8_t a_mn, b_mn;             /* operand majors */
  int32_t m0, n0, k0, k_blocks;
  uint32_t idesc;
  int32_t peer;                   /* -1: store to epilogue.out; else store into peer_out[peer] */
  long long row_off;              /* added to the row index on store */
  void* out_override;             /* non-null: store here instead of epilogue.out */
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

struct MacoCommArgs {             /* chunk [off, off+bytes) of a symmetric buffer */
  uint64_t sym_off_src;           /* byte offset inside the symmetric heap */
  uint64_t sym_off_dst;
  uint64_t bytes;
  int32_t dtype;
  int32_t peer;                   /* destination / source rank, -1 = all */
  int32_t op;                     /* 0 sum, 1 avg, 2 max, 3 min */
  int32_t flag_event;             /* peer event bumped per chunk, -1 none */
  void* local_out;                /* optional non-symmetric destination */
  float scale;
  int32_t _pad;
};

struct MacoTaskDesc {
  uint32_t type;
  uint32_t node_id;
  int32_t wait_event[2];          /* -1: no condition */
  uint32_t wait_count[2];
  int32_t signal_event;           /* local event bumped by 1 at completion, -1 none */
  int32_t signal_peer;            /* rank whose event table is bumped, -1 none, -2 all ranks */
  int32_t signal_peer_event;
  uint32_t flags;                 /* bit0: waits are on .sys-scope (peer-written) counters */
  union {
    MacoGemmArgs gemm;
    MacoEltArgs elt;
    MacoCommArgs comm;
    uint8_t raw[88];
  } u;
};

#ifdef __cplusplus
static_assert(sizeof(MacoTaskDesc) == 128, "task descriptor must stay 128 bytes");
#endif

/* ---- device trace ring ----------------------------------------------------------------------- */
struct MacoTraceRecord {
  uint32_t task;
  uint16_t type;
  uint16_t sm;
  uint64_t t_start_ns;            /* %globaltimer */
  uint64_t t_end_ns;
  uint64_t wait_ns;               /* time spent in dependency waits before the task body */
};
