// Stand-alone launches of the element-wise / row-wise operators (one CTA per chunk of rows).
#include "elementwise.cuh"
#include "host_common.h"

using namespace maco;

namespace {

__global__ void __launch_bounds__(128, 4) elt_kernel(uint32_t type, MacoEltArgs a, int rows_per_cta) {
  MacoEltArgs mine = a;
  mine.row0 = a.row0 + blockIdx.x * rows_per_cta;
  int left = a.rows - blockIdx.x * rows_per_cta;
  mine.rows = left < rows_per_cta ? left : rows_per_cta;
  if (mine.rows <= 0) return;
  elt_run(type, mine, threadIdx.x, blockDim.x);
}

}  // namespace

extern "C" int maco_elementwise(int type, const void* in0, const void* in1, const void* in2, void* out, int rows,
                                int cols, int dtype, int ld_in, int ld_out, float f0, float f1, int i0, int i1,
                                void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (rows <= 0 || cols <= 0) return 0;
  MacoEltArgs a;
  a.in0 = in0; a.in1 = in1; a.in2 = in2; a.out = out; a.row0 = 0; a.rows = rows; a.cols = cols; a.dtype = dtype;
  a.ld_in = ld_in; a.ld_out = ld_out; a.f0 = f0; a.f1 = f1; a.i0 = i0; a.i1 = i1;
  const int sms = maco_host::sm_count();
  // 128-thread CTAs, four resident per SM; several waves so that the tail is short.
  long long work = (long long)rows * cols;
  int target_ctas = (int)((work + 16383) / 16384);
  if (target_ctas > sms * 16) target_ctas = sms * 16;
  if (target_ctas < 1) target_ctas = 1;
  int rows_per_cta = (rows + target_ctas - 1) / target_ctas;
  if (rows_per_cta < 1) rows_per_cta = 1;
  int grid = (rows + rows_per_cta - 1) / rows_per_cta;
  elt_kernel<<<grid, 128, 0, stream>>>((uint32_t)type, a, rows_per_cta);
  MACO_CHECK_CUDA(cudaGetLastError());
  return 0;
}
