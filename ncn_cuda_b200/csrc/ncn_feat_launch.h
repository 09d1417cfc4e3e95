// Host-side entry points of the register-tiled multi-feature stage kernels (one per direction
// and n_cache).  With occ != nullptr nothing is launched: *occ receives the resident CTAs per SM.
// cudaErrorNotSupported: no kernel for this (n_cache, d, dtype, activation).
#pragma once
#include "ncn_common.cuh"

namespace ncn {

struct FeatParamsX;  // FeatParams plus what the kernels with a saved stage input or stored states take

#define NCN_DECL(n)                                                                                          \
  cudaError_t launch_feat_fwd_n##n(int d, int act, int dtype, const FeatParamsX& p, int grid, int threads,     \
                                   cudaStream_t st, int* occ);                                                                 \
  cudaError_t launch_feat_bwd_n##n(int d, int act, int dtype, const FeatParamsX& p, int grid, int threads,     \
                                   cudaStream_t st, int* occ);
NCN_DECL(2)
NCN_DECL(4)
NCN_DECL(8)
NCN_DECL(16)
NCN_DECL(32)
#undef NCN_DECL
// the backward that also takes the saved stage input (inverse chains of n_cache / 2 steps)
cudaError_t launch_feat_bwds_n16(int d, int act, int dtype, const FeatParamsX& p, int grid, int threads, cudaStream_t st,
                                 int* occ);
cudaError_t launch_feat_bwds_n32(int d, int act, int dtype, const FeatParamsX& p, int grid, int threads, cudaStream_t st,
                                 int* occ);
// the forward that also stores the state after every 16th step
cudaError_t launch_feat_fwdm_n16(int d, int act, int dtype, const FeatParamsX& p, int grid, int threads, cudaStream_t st,
                                 int* occ);
cudaError_t launch_feat_fwdm_n32(int d, int act, int dtype, const FeatParamsX& p, int grid, int threads, cudaStream_t st,
                                 int* occ);

// groups a warp works on side by side for (n_cache, d); 0 if there is no kernel
inline int feat_groups_per_warp(int n, int d) {
  if (n != 2 && n != 4 && n != 8 && n != 16 && n != 32) return 0;
  if (d != 2 && d != 4 && d != 8 && d != 16 && d != 32 && d != 64 && d != 128) return 0;
  if (n * d > 1024) return 0;
  const int ld = d <= 8 ? 1 : d / 8;
  const int slots = 32 / ld;
  return n >= slots ? 1 : slots / n;
}

}  // namespace ncn
