// Symmetric heap: one device allocation per rank, mapped into every other rank's address space, and (when
// the GPUs sit behind an NVSwitch that supports it) bound to one multicast object, so that a kernel can
// broadcast a store to every rank (multimem.st), add into every rank's copy (multimem.red) or load the sum
// over all ranks' copies (multimem.ld_reduce) with ONE instruction on the multicast address.
//
// The role NVSHMEM's symmetric heap plays in the reference (maco/csrc/nvshmem_ops.cu:37-147: MPI bootstrap +
// nvshmem_malloc). Two ways to build the heap:
//
//   * maco_heap_create / open / close / destroy: a plain cudaMalloc block exported with a CUDA IPC handle
//     (64 bytes, exchanged through the process group). Plain peer loads / stores only.
//   * maco_vheap_*: the CUDA virtual-memory API. cuMemCreate gives a physical allocation with a shareable
//     POSIX file descriptor; every rank imports the others' descriptors (the Python side passes them over
//     Unix sockets) and maps them; rank 0 creates the multicast object, every rank adds its device and binds
//     its own allocation at offset 0, then maps the object: that mapping is the heap's multicast address.
//
// The driver entry points are fetched at run time (the library has no link dependency on libcuda and loads on
// a machine without a driver). No NVSHMEM, no MPI.
#include "host_common.h"
#include <string.h>
#include <unistd.h>
#include <mutex>

namespace {

#define MACO_DRV_LIST(X)                                                                                       \
  X(cuMemCreate) X(cuMemRelease) X(cuMemAddressReserve) X(cuMemAddressFree) X(cuMemMap) X(cuMemUnmap)           \
  X(cuMemSetAccess) X(cuMemExportToShareableHandle) X(cuMemImportFromShareableHandle)                           \
  X(cuMemGetAllocationGranularity) X(cuMulticastCreate) X(cuMulticastAddDevice) X(cuMulticastBindMem)           \
  X(cuMulticastGetGranularity) X(cuMulticastUnbind) X(cuDeviceGet) X(cuDeviceGetAttribute) X(cuGetErrorString)

struct Driver {
#define X(name) decltype(&name) name##_ = nullptr;
  MACO_DRV_LIST(X)
#undef X
  bool ok = false;
};

Driver& drv() {
  static Driver d;
  static std::once_flag once;
  std::call_once(once, []() {
    bool all = true;
#define X(name)                                                                                                 \
    {                                                                                                           \
      void* p = nullptr;                                                                                        \
      cudaDriverEntryPointQueryResult q;                                                                        \
      if (cudaGetDriverEntryPoint(#name, &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess) \
        d.name##_ = reinterpret_cast<decltype(&name)>(p);                                                       \
      else all = false;                                                                                         \
    }
    MACO_DRV_LIST(X)
#undef X
    (void)cudaGetLastError();
    d.ok = all;
  });
  return d;
}

int drv_fail(const char* what, CUresult r) {
  const char* msg = nullptr;
  if (drv().cuGetErrorString_ != nullptr) drv().cuGetErrorString_(r, &msg);
  maco_host::set_error(std::string(what) + ": " + (msg ? msg : "unknown driver error") + " (" + std::to_string((int)r) + ")");
  return -1;
}

#define MACO_CHECK_DRV(call, what)                       \
  do {                                                   \
    CUresult _r = (call);                                \
    if (_r != CUDA_SUCCESS) return drv_fail(what, _r);   \
  } while (0)

// One virtual-memory heap per process (one process drives one GPU).
struct VHeap {
  CUmemGenericAllocationHandle own = 0, mc = 0;
  CUmemGenericAllocationHandle peer[MACO_MAX_PEERS] = {};
  CUdeviceptr va[MACO_MAX_PEERS] = {};       // mapping of every rank's allocation (own included)
  CUdeviceptr mc_va = 0;
  size_t size = 0;
  int dev = -1, rank = -1, world = 0;
  bool mc_bound = false, live = false;
} g_vh;

int access_rw(CUdeviceptr va, size_t size, int dev) {
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof acc);
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = dev;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  MACO_CHECK_DRV(drv().cuMemSetAccess_(va, size, &acc, 1), "cuMemSetAccess");
  return 0;
}

}  // namespace

extern "C" {

// ---- cudaMalloc + CUDA IPC form ---------------------------------------------------------------------------
// Allocates `bytes` of device memory, zeroes it and writes the 64-byte IPC handle.
int maco_heap_create(unsigned long long bytes, void** base_out, void* handle_out64) {
  void* p = nullptr;
  MACO_CHECK_CUDA(cudaMalloc(&p, bytes));
  MACO_CHECK_CUDA(cudaMemset(p, 0, bytes));
  cudaIpcMemHandle_t h;
  MACO_CHECK_CUDA(cudaIpcGetMemHandle(&h, p));
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle is 64 bytes");
  memcpy(handle_out64, &h, 64);
  MACO_CHECK_CUDA(cudaDeviceSynchronize());
  *base_out = p;
  return 0;
}

// Maps a peer's heap into this process. Peer access between the two devices is enabled lazily.
int maco_heap_open(const void* handle64, void** peer_base_out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* p = nullptr;
  MACO_CHECK_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  *peer_base_out = p;
  return 0;
}

int maco_heap_close(void* peer_base) {
  MACO_CHECK_CUDA(cudaIpcCloseMemHandle(peer_base));
  return 0;
}

int maco_heap_destroy(void* base) {
  MACO_CHECK_CUDA(cudaFree(base));
  return 0;
}

// ---- virtual-memory form (shareable descriptors, multicast) ------------------------------------------------
// 1 when this device can export allocations as POSIX file descriptors; *multicast_out = 1 when it can also
// join a multicast object (NVSwitch with NVLS).
int maco_vheap_supported(int* multicast_out) {
  *multicast_out = 0;
  if (!drv().ok) return 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  CUdevice cd;
  if (drv().cuDeviceGet_(&cd, dev) != CUDA_SUCCESS) return 0;
  int fd_ok = 0, mc_ok = 0;
  drv().cuDeviceGetAttribute_(&fd_ok, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, cd);
  drv().cuDeviceGetAttribute_(&mc_ok, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, cd);
  *multicast_out = mc_ok;
  return fd_ok;
}

// Creates this rank's allocation (zeroed, mapped read-write for this device). `bytes_inout`: requested size,
// rounded up to what both the allocation and the multicast granularity need (every rank gets the same value).
// `fd_out`: descriptor to hand to the other ranks (closed by maco_vheap_destroy).
int maco_vheap_create(unsigned long long* bytes_inout, int rank, int world, int want_multicast, void** base_out, int* fd_out) {
  if (!drv().ok) { maco_host::set_error("the CUDA driver's virtual-memory entry points are not available"); return -1; }
  if (g_vh.live) { maco_host::set_error("a virtual-memory heap already exists in this process"); return -1; }
  if (world < 1 || world > MACO_MAX_PEERS || rank < 0 || rank >= world) { maco_host::set_error("bad rank / world"); return -1; }
  int dev = 0;
  MACO_CHECK_CUDA(cudaGetDevice(&dev));
  MACO_CHECK_CUDA(cudaFree(0));                       // the primary context exists
  CUmemAllocationProp prop;
  memset(&prop, 0, sizeof prop);
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = dev;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  size_t gran = 0;
  MACO_CHECK_DRV(drv().cuMemGetAllocationGranularity_(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED), "cuMemGetAllocationGranularity");
  if (want_multicast) {
    CUmulticastObjectProp mp;
    memset(&mp, 0, sizeof mp);
    mp.numDevices = (unsigned)world;
    mp.size = (size_t)*bytes_inout;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t mg = 0;
    MACO_CHECK_DRV(drv().cuMulticastGetGranularity_(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED), "cuMulticastGetGranularity");
    if (mg > gran) gran = mg;
  }
  const size_t size = ((size_t)*bytes_inout + gran - 1) / gran * gran;
  g_vh = VHeap();
  g_vh.dev = dev; g_vh.rank = rank; g_vh.world = world; g_vh.size = size;
  MACO_CHECK_DRV(drv().cuMemCreate_(&g_vh.own, size, &prop, 0), "cuMemCreate");
  g_vh.live = true;
  MACO_CHECK_DRV(drv().cuMemAddressReserve_(&g_vh.va[rank], size, gran, 0, 0), "cuMemAddressReserve");
  MACO_CHECK_DRV(drv().cuMemMap_(g_vh.va[rank], size, 0, g_vh.own, 0), "cuMemMap");
  if (access_rw(g_vh.va[rank], size, dev) != 0) return -1;
  MACO_CHECK_CUDA(cudaMemset(reinterpret_cast<void*>(g_vh.va[rank]), 0, size));
  MACO_CHECK_CUDA(cudaDeviceSynchronize());
  int fd = -1;
  MACO_CHECK_DRV(drv().cuMemExportToShareableHandle_(&fd, g_vh.own, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0), "cuMemExportToShareableHandle");
  *bytes_inout = size;
  *base_out = reinterpret_cast<void*>(g_vh.va[rank]);
  *fd_out = fd;
  return 0;
}

// Maps rank `peer`'s allocation from its descriptor (received over a Unix socket; the caller closes it).
int maco_vheap_import(int peer, int fd, void** base_out) {
  if (!g_vh.live || peer < 0 || peer >= g_vh.world || peer == g_vh.rank) { maco_host::set_error("maco_vheap_import: bad peer"); return -1; }
  MACO_CHECK_DRV(drv().cuMemImportFromShareableHandle_(&g_vh.peer[peer], reinterpret_cast<void*>((uintptr_t)fd),
                                                       CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR), "cuMemImportFromShareableHandle");
  MACO_CHECK_DRV(drv().cuMemAddressReserve_(&g_vh.va[peer], g_vh.size, 0, 0, 0), "cuMemAddressReserve(peer)");
  MACO_CHECK_DRV(drv().cuMemMap_(g_vh.va[peer], g_vh.size, 0, g_vh.peer[peer], 0), "cuMemMap(peer)");
  if (access_rw(g_vh.va[peer], g_vh.size, g_vh.dev) != 0) return -1;
  *base_out = reinterpret_cast<void*>(g_vh.va[peer]);
  return 0;
}

// Rank 0: creates the multicast object over `world` devices and returns a descriptor for the other ranks.
int maco_vheap_mc_create(int* fd_out) {
  if (!g_vh.live) { maco_host::set_error("no heap"); return -1; }
  CUmulticastObjectProp mp;
  memset(&mp, 0, sizeof mp);
  mp.numDevices = (unsigned)g_vh.world;
  mp.size = g_vh.size;
  mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  MACO_CHECK_DRV(drv().cuMulticastCreate_(&g_vh.mc, &mp), "cuMulticastCreate");
  int fd = -1;
  MACO_CHECK_DRV(drv().cuMemExportToShareableHandle_(&fd, g_vh.mc, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0), "cuMemExportToShareableHandle(multicast)");
  *fd_out = fd;
  return 0;
}

// Other ranks: open rank 0's multicast object.
int maco_vheap_mc_import(int fd) {
  if (!g_vh.live) { maco_host::set_error("no heap"); return -1; }
  MACO_CHECK_DRV(drv().cuMemImportFromShareableHandle_(&g_vh.mc, reinterpret_cast<void*>((uintptr_t)fd),
                                                       CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR), "cuMemImportFromShareableHandle(multicast)");
  return 0;
}

// Every rank, in this order with a host barrier between the steps: add_device, then bind (all devices must
// have been added before the first binding), then map.
int maco_vheap_mc_add_device() {
  CUdevice cd;
  MACO_CHECK_DRV(drv().cuDeviceGet_(&cd, g_vh.dev), "cuDeviceGet");
  MACO_CHECK_DRV(drv().cuMulticastAddDevice_(g_vh.mc, cd), "cuMulticastAddDevice");
  return 0;
}

int maco_vheap_mc_bind() {
  MACO_CHECK_DRV(drv().cuMulticastBindMem_(g_vh.mc, 0, g_vh.own, 0, g_vh.size, 0), "cuMulticastBindMem");
  g_vh.mc_bound = true;
  return 0;
}

int maco_vheap_mc_map(void** mc_base_out) {
  MACO_CHECK_DRV(drv().cuMemAddressReserve_(&g_vh.mc_va, g_vh.size, 0, 0, 0), "cuMemAddressReserve(multicast)");
  MACO_CHECK_DRV(drv().cuMemMap_(g_vh.mc_va, g_vh.size, 0, g_vh.mc, 0), "cuMemMap(multicast)");
  if (access_rw(g_vh.mc_va, g_vh.size, g_vh.dev) != 0) return -1;
  *mc_base_out = reinterpret_cast<void*>(g_vh.mc_va);
  return 0;
}

// Unmaps and releases everything this process holds of the heap. Call it on every rank with nothing in flight;
// a rank must not disappear while its memory is still bound to the multicast object.
int maco_vheap_destroy() {
  if (!g_vh.live) return 0;
  cudaDeviceSynchronize();
  Driver& d = drv();
  if (g_vh.mc_va) { d.cuMemUnmap_(g_vh.mc_va, g_vh.size); d.cuMemAddressFree_(g_vh.mc_va, g_vh.size); }
  if (g_vh.mc_bound) { CUdevice cd; if (d.cuDeviceGet_(&cd, g_vh.dev) == CUDA_SUCCESS) d.cuMulticastUnbind_(g_vh.mc, cd, 0, g_vh.size); }
  if (g_vh.mc) d.cuMemRelease_(g_vh.mc);
  for (int r = 0; r < g_vh.world; ++r) {
    if (g_vh.va[r]) { d.cuMemUnmap_(g_vh.va[r], g_vh.size); d.cuMemAddressFree_(g_vh.va[r], g_vh.size); }
    if (r != g_vh.rank && g_vh.peer[r]) d.cuMemRelease_(g_vh.peer[r]);
  }
  if (g_vh.own) d.cuMemRelease_(g_vh.own);
  g_vh = VHeap();
  return 0;
}

}  // extern "C"
