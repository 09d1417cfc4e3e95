// Host-side entry points of the fused row kernels (one per direction and group size).
#pragma once
#include "ncn_common.cuh"

namespace ncn {

// Largest block the kernel is compiled for; it fixes the register budget per thread.
template <int NG, bool BWD>
struct RowsMaxThreads {
  static constexpr int value = BWD ? (NG <= 4 ? 1024 : NG == 8 ? 512 : 256) : (NG <= 4 ? 1024 : NG == 8 ? 512 : 256);
};
inline int rows_max_threads(int n, bool bwd) {
  switch (n) {
    case 2: return RowsMaxThreads<2, false>::value;
    case 4: return bwd ? RowsMaxThreads<4, true>::value : RowsMaxThreads<4, false>::value;
    case 8: return bwd ? RowsMaxThreads<8, true>::value : RowsMaxThreads<8, false>::value;
    case 16: return bwd ? RowsMaxThreads<16, true>::value : RowsMaxThreads<16, false>::value;
    default: return 0;
  }
}

// Pair kernels (two groups per thread): block size they are compiled for and the CTAs per SM the
// register budget is set for.
template <int NG, bool BWD>
struct PairLaunch {
  static constexpr int threads = NG <= 4 ? 512 : 256;
  static constexpr int min_blocks = NG <= 4 ? 2 : 1;
};
inline int pair_max_threads(int n, bool bwd) {
  (void)bwd;
  return n <= 4 ? 512 : 256;
}

// With occ != nullptr nothing is launched: *occ receives the resident CTAs per SM.
#define NCN_DECL(n)                                                                                              \
  cudaError_t launch_rows_fwd_n##n(int act, int dtype, const RowsParams& p, int grid, int threads, size_t smem, \
                                   cudaStream_t st, int* occ);                                                  \
  cudaError_t launch_rows_bwd_n##n(int act, int dtype, const RowsParams& p, int grid, int threads, size_t smem, \
                                   cudaStream_t st, int* occ);
NCN_DECL(2)
NCN_DECL(4)
NCN_DECL(8)
NCN_DECL(16)
#undef NCN_DECL
#define NCN_DECL(n)                                                                                              \
  cudaError_t launch_pair_fwd_n##n(int act, int dtype, const RowsParams& p, int grid, int threads, size_t smem, \
                                   cudaStream_t st, int* occ);                                                  \
  cudaError_t launch_pair_bwd_n##n(int act, int dtype, const RowsParams& p, int grid, int threads, size_t smem, \
                                   cudaStream_t st, int* occ);
NCN_DECL(2)
NCN_DECL(4)
NCN_DECL(8)
NCN_DECL(16)
#undef NCN_DECL

}  // namespace ncn
