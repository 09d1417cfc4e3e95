// Host-side entry points and parameter block of the register-resident row kernels (ncn_lanes.cuh).
#pragma once
#include "ncn_common.cuh"

namespace ncn {

struct LaneParams {
  const void* in[4];   // fwd: x, xa, -, - ; bwd: y, ya, dy, dya
  void* out[4];        // fwd: y, ya, -, - ; bwd: dx, dxa, x_rec (or null), xa_rec (or null)
  float* ckpt;         // [K][B*N] (x, a) pairs in this family's order, or null
  const float* W;      // [L][2]
  float* partials;     // bwd: [gridDim.x][L][2]
  int* status;         // device status word
  long long B;
  long long tiles;
  int N, m, R, L, l0, ckpt_every, flags;
  int tpr;             // threads per row (m / G), a multiple of 32
  int ea_max;          // shifts of up to 2^ea_max blocks per offset use shuffles + halo, longer ones the tile buffer
  float alpha, oma;
  uint32_t off_work, off_res, off_ckpt, off_halo, off_red, off_w, off_bar;
  uint32_t halo_warp_bytes;  // halo bytes per warp and buffer
  uint32_t n_ckpt_slots;
  int test_short_wait;       // forward, tests of the give-up path only: expect 16 bytes that never come, poll 2^10 times
  int pipelined;             // backward, n = 4: the kernel of ncn_lanes_pipe.cuh (halo inside the tile buffer)
};

__host__ __device__ constexpr int lane_groups(int ng) { return ng == 2 ? 8 : ng == 4 ? 4 : 2; }
// largest log2 |stride difference| the shuffle exchange is compiled for
__host__ __device__ constexpr int lane_ea_cap(int ng) { return ng == 2 ? 6 : ng == 4 ? 4 : 2; }
// halo floats per warp and stream for a stride difference of 2^e: sum over offsets o of o 2^e (for e = 0 every
// offset's region is rounded up to whole pairs)
__host__ __device__ constexpr int lane_halo_floats(int ng, int e) {
  return e == 0 ? ng * (ng - 1) / 2 + ng / 2 : (1 << e) * ng * (ng - 1) / 2;
}
// first float of offset o's region when the regions hold whole pairs (e = 0): sum over o' < o of o' rounded up to even
__host__ __device__ constexpr int lane_halo_pair_base(int o) {
  int b = 0;
  for (int q = 1; q < o; ++q) b += (q + 1) & ~1;
  return b;
}

// Pipelined kernels (ncn_lanes_pipe.cuh): bytes between the regions of two (stream, offset) pairs of a warp's halo
// area: 4 (kmax + 2) for the largest shift they take (kmax = 3 * 16 blocks), a multiple of 16.  A compile-time
// constant, so that every halo access is "per-thread base register + immediate".
constexpr unsigned kPipeSo = 208;

// Block size the kernels are compiled for, and the CTAs per SM their register budget allows.
constexpr int kLaneThreads = 256;
constexpr int kLaneFwdBlocks = 4;
constexpr int kLaneBwdBlocks = 2;

// With occ != nullptr nothing is launched: *occ receives the resident CTAs per SM.
#define NCN_DECL(n)                                                                                              \
  cudaError_t launch_lane_fwd_n##n(int act, int dtype, const LaneParams& p, int grid, int threads, size_t smem, \
                                   cudaStream_t st, int* occ);                                                  \
  cudaError_t launch_lane_bwd_n##n(int act, int dtype, const LaneParams& p, int grid, int threads, size_t smem, \
                                   cudaStream_t st, int* occ);
NCN_DECL(2)
NCN_DECL(4)
NCN_DECL(8)
#undef NCN_DECL

}  // namespace ncn
