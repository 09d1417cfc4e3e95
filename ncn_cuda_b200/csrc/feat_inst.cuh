// Explicit instantiation of the register-tiled multi-feature stage kernels (ncn_feat.cuh) for one
// n_cache (NCN_NC) and one direction (NCN_BWD defined or not); one translation unit each.
// Head widths d = 2, 4 (one lane per position), 8, 16, 32, 64, 128 (8 features per lane), as far as the
// group tile fits the registers of a warp (n_cache * d <= 1024).  Every other shape, and bf16
// storage with the exact tanh, stays with the shared-memory kernels of ncn_generic.cuh.
#include "ncn_feat.cuh"
#include "ncn_feat_launch.h"

namespace ncn {

// NCN_SAVED (with NCN_BWD): the backward that also takes the saved stage input or the forward's stored states.
// NCN_MID (without NCN_BWD): the forward that stores the state after every 16th step.

template <int LD, int KF, int ACT, typename T>
static cudaError_t launch_one(const FeatParamsX& px, int grid, int threads, cudaStream_t st, int* occ) {
  if constexpr (NCN_NC * LD * KF > 1024) {
    return cudaErrorNotSupported;
  } else {
#if defined(NCN_BWD) && defined(NCN_SAVED)
    auto k = feat_bwd_kernel<NCN_NC, LD, KF, ACT, T, true, FeatParamsX>;
    const FeatParamsX& p = px;
#elif defined(NCN_BWD)
    auto k = feat_bwd_kernel<NCN_NC, LD, KF, ACT, T>;
    const FeatParams p = px;  // the default kernels take the first 128 bytes only
#elif defined(NCN_MID)
    auto k = feat_fwd_kernel<NCN_NC, LD, KF, ACT, T, true, FeatParamsX>;
    const FeatParamsX& p = px;
#else
    auto k = feat_fwd_kernel<NCN_NC, LD, KF, ACT, T>;
    const FeatParams p = px;
#endif
    if (occ) return cudaOccupancyMaxActiveBlocksPerMultiprocessor(occ, k, threads, 0);
    k<<<grid, threads, 0, st>>>(p);
    return cudaGetLastError();
  }
}

template <int LD, int KF>
static cudaError_t launch_geo(int act, int dtype, const FeatParamsX& p, int grid, int threads, cudaStream_t st, int* occ) {
  if (dtype == DT_F32) {
    switch (act) {
      case ACT_TANH: return launch_one<LD, KF, ACT_TANH, float>(p, grid, threads, st, occ);
      case ACT_RELU: return launch_one<LD, KF, ACT_RELU, float>(p, grid, threads, st, occ);
      case ACT_SIGMOID: return launch_one<LD, KF, ACT_SIGMOID, float>(p, grid, threads, st, occ);
      case ACT_LINEAR: return launch_one<LD, KF, ACT_LINEAR, float>(p, grid, threads, st, occ);
      default: return cudaErrorNotSupported;
    }
  }
  switch (act) {  // bf16 storage; the exact tanh (NCN_EXACT_TANH=1) stays with the shared-memory kernels
    case ACT_TANH_FAST: return launch_one<LD, KF, ACT_TANH_FAST, __nv_bfloat16>(p, grid, threads, st, occ);
    case ACT_RELU: return launch_one<LD, KF, ACT_RELU, __nv_bfloat16>(p, grid, threads, st, occ);
    case ACT_SIGMOID: return launch_one<LD, KF, ACT_SIGMOID, __nv_bfloat16>(p, grid, threads, st, occ);
    case ACT_LINEAR: return launch_one<LD, KF, ACT_LINEAR, __nv_bfloat16>(p, grid, threads, st, occ);
    default: return cudaErrorNotSupported;
  }
}

#define NCN_CAT2(a, b) a##b
#define NCN_CAT(a, b) NCN_CAT2(a, b)
#if defined(NCN_BWD) && defined(NCN_SAVED)
#define NCN_FN NCN_CAT(launch_feat_bwds_n, NCN_NC)
#elif defined(NCN_BWD)
#define NCN_FN NCN_CAT(launch_feat_bwd_n, NCN_NC)
#elif defined(NCN_MID)
#define NCN_FN NCN_CAT(launch_feat_fwdm_n, NCN_NC)
#else
#define NCN_FN NCN_CAT(launch_feat_fwd_n, NCN_NC)
#endif

cudaError_t NCN_FN(int d, int act, int dtype, const FeatParamsX& p, int grid, int threads, cudaStream_t st, int* occ) {
  switch (d) {
    case 2: return launch_geo<1, 2>(act, dtype, p, grid, threads, st, occ);
    case 4: return launch_geo<1, 4>(act, dtype, p, grid, threads, st, occ);
    case 8: return launch_geo<1, 8>(act, dtype, p, grid, threads, st, occ);
    case 16: return launch_geo<2, 8>(act, dtype, p, grid, threads, st, occ);
    case 32: return launch_geo<4, 8>(act, dtype, p, grid, threads, st, occ);
    case 64: return launch_geo<8, 8>(act, dtype, p, grid, threads, st, occ);
    case 128: return launch_geo<16, 8>(act, dtype, p, grid, threads, st, occ);
    default: return cudaErrorNotSupported;
  }
}

}  // namespace ncn
