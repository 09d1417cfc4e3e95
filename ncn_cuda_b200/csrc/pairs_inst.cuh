// Explicit instantiation of the pair kernels (ncn_pairs.cuh) for one group size (NCN_NG) and
// one direction (NCN_BWD defined or not).
#include "ncn_pairs.cuh"
#include "ncn_rows_launch.h"

namespace ncn {

#ifdef NCN_BWD
#define NCN_KERNEL pair_bwd_kernel
#define NCN_CFG PairLaunch<NCN_NG, true>
#else
#define NCN_KERNEL pair_fwd_kernel
#define NCN_CFG PairLaunch<NCN_NG, false>
#endif

template <int ACT, typename T>
static cudaError_t launch_one(const RowsParams& p, int grid, int threads, size_t smem, cudaStream_t st, int* occ) {
#ifdef NCN_BWD
  if (p.variant == 2) {
    if constexpr (NCN_NG <= 8) {
      auto kd = pair_bwd_dual_kernel<NCN_NG, ACT, T, NCN_CFG::threads / 2>;
      static SmemGrant granted_d;
      cudaError_t ed = grant_smem(granted_d, kd, smem);
      if (ed != cudaSuccess) return ed;
      if (occ) return cudaOccupancyMaxActiveBlocksPerMultiprocessor(occ, kd, threads, smem);
      kd<<<grid, threads, smem, st>>>(p);
      return cudaGetLastError();
    } else {
      return cudaErrorNotSupported;
    }
  }
  if (p.variant == 1) {
    auto kw = pair_bwd_wide_kernel<NCN_NG, ACT, T, NCN_CFG::threads>;
    static SmemGrant granted_w;
    cudaError_t ew = grant_smem(granted_w, kw, smem);
    if (ew != cudaSuccess) return ew;
    if (occ) return cudaOccupancyMaxActiveBlocksPerMultiprocessor(occ, kw, threads, smem);
    kw<<<grid, threads, smem, st>>>(p);
    return cudaGetLastError();
  }
#endif
#ifndef NCN_BWD
  if (p.variant == 2) {
    auto kd = pair_fwd_dual_kernel<NCN_NG, ACT, T, NCN_CFG::threads / 2, (NCN_NG <= 8 ? 4 : 2)>;
    static SmemGrant granted_fd;
    cudaError_t ed = grant_smem(granted_fd, kd, smem);
    if (ed != cudaSuccess) return ed;
    if (occ) return cudaOccupancyMaxActiveBlocksPerMultiprocessor(occ, kd, threads, smem);
    kd<<<grid, threads, smem, st>>>(p);
    return cudaGetLastError();
  }
#endif
  auto k = NCN_KERNEL<NCN_NG, ACT, T, NCN_CFG::threads, NCN_CFG::min_blocks>;
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
#define NCN_FN NCN_CAT(launch_pair_bwd_n, NCN_NG)
#else
#define NCN_FN NCN_CAT(launch_pair_fwd_n, NCN_NG)
#endif

cudaError_t NCN_FN(int act, int dtype, const RowsParams& p, int grid, int threads, size_t smem, cudaStream_t st,
                   int* occ) {
  if (dtype == DT_BF16) return launch_act<__nv_bfloat16>(act, p, grid, threads, smem, st, occ);
  return launch_act<float>(act, p, grid, threads, smem, st, occ);
}

}  // namespace ncn
