// Explicit instantiation of the register-resident row kernels (ncn_lanes.cuh) for one group size
// (NCN_NG) and one direction (NCN_BWD defined or not).
#include "ncn_lanes_pipe.cuh"

namespace ncn {

template <int ACT, typename T>
static cudaError_t launch_one(const LaneParams& p, int grid, int threads, size_t smem, cudaStream_t st, int* occ) {
#ifdef NCN_BWD
#if NCN_NG == 4
  if (p.pipelined) {  // two half-rows per thread, half a stage apart (ncn_lanes_pipe.cuh)
    auto kp = lanep_bwd_kernel<NCN_NG, ACT, T, kLaneThreads, kLaneBwdBlocks>;
    static SmemGrant granted_p;
    cudaError_t ep = grant_smem(granted_p, kp, smem);
    if (ep != cudaSuccess) return ep;
    if (occ) return cudaOccupancyMaxActiveBlocksPerMultiprocessor(occ, kp, threads, smem);
    kp<<<grid, threads, smem, st>>>(p);
    return cudaGetLastError();
  }
#endif
  auto k = lane_bwd_kernel<NCN_NG, ACT, T, kLaneThreads, kLaneBwdBlocks>;
#else
#if NCN_NG == 4
  if (p.pipelined) {  // (A/B runs only: measured slower than lane_fwd_kernel)
    auto kp = lanep_fwd_kernel<NCN_NG, ACT, T, kLaneThreads, kLaneBwdBlocks>;
    static SmemGrant granted_pf;
    cudaError_t ep = grant_smem(granted_pf, kp, smem);
    if (ep != cudaSuccess) return ep;
    if (occ) return cudaOccupancyMaxActiveBlocksPerMultiprocessor(occ, kp, threads, smem);
    kp<<<grid, threads, smem, st>>>(p);
    return cudaGetLastError();
  }
#endif
  auto k = lane_fwd_kernel<NCN_NG, ACT, T, kLaneThreads, kLaneFwdBlocks>;
#endif
  static SmemGrant granted;
  cudaError_t e = grant_smem(granted, k, smem);
  if (e != cudaSuccess) return e;
  if (occ) return cudaOccupancyMaxActiveBlocksPerMultiprocessor(occ, k, threads, smem);
  k<<<grid, threads, smem, st>>>(p);
  return cudaGetLastError();
}

template <typename T>
static cudaError_t launch_act(int act, const LaneParams& p, int grid, int threads, size_t smem, cudaStream_t st,
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
#define NCN_FN NCN_CAT(launch_lane_bwd_n, NCN_NG)
#else
#define NCN_FN NCN_CAT(launch_lane_fwd_n, NCN_NG)
#endif

cudaError_t NCN_FN(int act, int dtype, const LaneParams& p, int grid, int threads, size_t smem, cudaStream_t st,
                   int* occ) {
  if (dtype == DT_BF16) return launch_act<__nv_bfloat16>(act, p, grid, threads, smem, st, occ);
  return launch_act<float>(act, p, grid, threads, smem, st, occ);
}

}  // namespace ncn
