// Explicit instantiation of the fused row kernels for one group size (NCN_NG) and one
// direction (NCN_BWD defined or not).  One translation unit per (direction, group size)
// keeps every nvcc job small enough to build in parallel.
#include "ncn_rows.cuh"
#include "ncn_rows_launch.h"

namespace ncn {

#ifdef NCN_BWD
#define NCN_KERNEL rows_bwd_kernel
#define NCN_MAXT RowsMaxThreads<NCN_NG, true>::value
#else
#define NCN_KERNEL rows_fwd_kernel
#define NCN_MAXT RowsMaxThreads<NCN_NG, false>::value
#endif

template <int ACT, typename T>
static cudaError_t launch_one(const RowsParams& p, int grid, int threads, size_t smem, cudaStream_t st, int* occ) {
  auto k = NCN_KERNEL<NCN_NG, ACT, T, NCN_MAXT>;
  static SmemGrant granted;
  cudaError_t e = grant_smem(granted, k, smem);
  if (e != cudaSuccess) return e;
  if (occ) return cudaOccupancyMaxActiveBlocksPerMultiprocessor(occ, k, threads, smem);
  k<<<grid, threads, smem, st>>>(p);
  return cudaGetLastError();
}

template <typename T>
static cudaError_t launch_act(int act, const RowsParams& p, int grid, int threads, size_t smem, cudaStream_t st,
                              int* occ) {
  if constexpr (sizeof(T) == 2) {  // bf16 storage only
    if (act == ACT_TANH_FAST) return launch_one<ACT_TANH_FAST, T>(p, grid, threads, smem, st, occ);
  }
  switch (act) {
    case ACT_TANH: return launch_one<ACT_TANH, T>(p, grid, threads, smem, st, occ);
    case ACT_RELU: return launch_one<ACT_RELU, T>(p, grid, threads, smem, st, occ);
    case ACT_SIGMOID: return launch_one<ACT_SIGMOID, T>(p, grid, threads, smem, st, occ);
    default: return launch_one<ACT_LINEAR, T>(p, grid, threads, smem, st, occ);
  }
}

#define NCN_CAT2(a, b) a##b
#define NCN_CAT(a, b) NCN_CAT2(a, b)
#ifdef NCN_BWD
#define NCN_FN NCN_CAT(launch_rows_bwd_n, NCN_NG)
#else
#define NCN_FN NCN_CAT(launch_rows_fwd_n, NCN_NG)
#endif

cudaError_t NCN_FN(int act, int dtype, const RowsParams& p, int grid, int threads, size_t smem, cudaStream_t st,
                   int* occ) {
  if (dtype == DT_BF16) return launch_act<__nv_bfloat16>(act, p, grid, threads, smem, st, occ);
  return launch_act<float>(act, p, grid, threads, smem, st, occ);
}

}  // namespace ncn
