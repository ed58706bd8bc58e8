// Host-side helpers: error text, run-time driver entry points, tensor maps, status block.
#include "host_common.h"
#include <mutex>

namespace maco_host {

static thread_local std::string g_err;
void set_error(const std::string& msg) { g_err = msg; }
const char* last_error() { return g_err.c_str(); }

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, []() {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

int encode_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t rows, uint64_t cols,
                   uint64_t row_stride_bytes, uint32_t box_cols, uint32_t box_rows) {
  EncodeTiledFn enc = get_encode();
  if (enc == nullptr) { set_error("cuTensorMapEncodeTiled is not available (no CUDA driver?)"); return -1; }
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (row_stride_bytes & 15) != 0) {
    set_error("tensor map: base address and row stride must be multiples of 16 bytes");
    return -2;
  }
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                         : elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  CUresult r = enc(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[160];
    snprintf(buf, sizeof buf, "cuTensorMapEncodeTiled failed with %d (rows=%llu cols=%llu stride=%llu box=%ux%u)",
             (int)r, (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)row_stride_bytes,
             box_cols, box_rows);
    set_error(buf);
    return -3;
  }
  return 0;
}

// One status block per device, allocated on first use in host-mapped pinned memory so the host
// can read what a kernel reported without a copy.
static MacoStatusBlock* g_status_host[64] = {};
static uint32_t* g_status_dev[64] = {};
static std::mutex g_status_mu;

static int ensure_status(int dev) {
  std::lock_guard<std::mutex> lk(g_status_mu);
  if (g_status_host[dev] != nullptr) return 0;
  void* h = nullptr;
  if (cudaHostAlloc(&h, sizeof(MacoStatusBlock), cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) return -1;
  memset(h, 0, sizeof(MacoStatusBlock));
  void* d = nullptr;
  if (cudaHostGetDevicePointer(&d, h, 0) != cudaSuccess) return -1;
  g_status_host[dev] = reinterpret_cast<MacoStatusBlock*>(h);
  g_status_dev[dev] = reinterpret_cast<uint32_t*>(d);
  return 0;
}

uint32_t* status_device_ptr() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (ensure_status(dev) != 0) return nullptr;
  return g_status_dev[dev];
}
MacoStatusBlock* status_host_ptr() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (ensure_status(dev) != 0) return nullptr;
  return g_status_host[dev];
}

int sm_count() {
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    cached[dev] = n;
  }
  return cached[dev];
}

}  // namespace maco_host

extern "C" {
const char* maco_last_error() { return maco_host::last_error(); }
// Reads and optionally clears the status word kernels OR their failures into.
unsigned maco_status(int clear) {
  MacoStatusBlock* s = maco_host::status_host_ptr();
  if (s == nullptr) return 0xffffffffu;
  unsigned v = s->status;
  if (clear) { s->status = 0; s->task = 0; s->event = 0; s->cta = 0; }
  return v;
}
int maco_status_block(MacoStatusBlock* out) {
  MacoStatusBlock* s = maco_host::status_host_ptr();
  if (s == nullptr) return -1;
  *out = *s;
  return 0;
}
int maco_sm_count() { return maco_host::sm_count(); }
}
