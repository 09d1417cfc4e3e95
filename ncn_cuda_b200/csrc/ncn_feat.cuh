// Per-stage NCN kernels for several features per position (E > 1, heads of d = E / n_head
// features), with the whole group tile in registers.
//
// Behaviour replaced: ncn_cuda/ncn_fwd_cuda_kernel.cu:28-112 (forward_kernel) and
// ncn_cuda/ncn_bwd_cuda_kernel.cu:27-229 (backward_kernel), at the shapes the reference's own
// benchmark uses (grad_test_bench.py:22-28: E = 128, 4 heads, n_cache = 32); math as
// torch_ref/ncn_pytorch.py:74-94 (step) and torch_ref/ncn_pytorch_invertible.py:97-111, 164-172
// (inverse, gradient).
//
// One warp owns one group (or several small ones) for all its n_cache steps:
//   lane = (slot, sub): LD = d / KF lanes share a position, each holding KF contiguous features;
//   the 32 / LD slots of the warp hold the positions, P = n_cache * LD / 32 per lane (position
//   i = r * SEG + s for slot s, r < P), or several groups side by side when n_cache < 32 / LD.
// Per step the row x_j reaches every lane by KF shuffles, the dot products over the features are
// lane-local sums plus log2(LD) exchanges, and no shared memory or barrier is involved.  The
// kernels are bound by the special-function unit (two instructions per element and step for tanh)
// like the one-feature kernels.
#pragma once
#include "ncn_common.cuh"

// Reciprocals of the tanh / sigmoid taken together over the feature pairs of a position (act_r_all,
// ncn_common.cuh): 0 = one special-function reciprocal per value.
#ifndef NCN_FEAT_FWD_BATCH
#define NCN_FEAT_FWD_BATCH 4
#endif
#ifndef NCN_FEAT_BWD_BATCH
#define NCN_FEAT_BWD_BATCH 0
#endif
#ifndef NCN_FEAT_UNROLL
#define NCN_FEAT_UNROLL 1
#endif

namespace ncn {

struct FeatParams {
  const void* in[4];  // fwd: x, xa ; bwd: y, ya, dy, dya
  void* out[4];       // fwd: y, ya ; bwd: dx, dxa, x_rec|null, xa_rec|null
  const float* W;     // [2E]
  float* partials;    // bwd: [gridDim.x][2E]
  long long B;
  long long units;    // B * mg work units per head
  int N, E, C, m, mg, stride;  // mg = ceil(m / groups per warp)
  float alpha, oma;
};
// Parameters of the kernels with a saved stage input or stored states.  A type of its own: the default kernels
// keep the 128-byte FeatParams (with these fields inside it the default backward, which never reads them, ran
// 4 % slower: the compiler's schedule at 249 registers is that easily disturbed).
struct FeatParamsX : FeatParams {
  const void* xin[2]; // bwd with the stage input saved: x, xa
  float* mid;         // fp32 states after every 16th step: state k, stream s at mid + (2k + s) * bne, in the
                      // element order of the activations (fwd with MID: written; bwd with saved == 3: read)
  long long bne;      // elements per activation tensor
  int saved;          // bwd: 1 = the first half of the steps is replayed from the saved input; 2 = all steps are
                      // (y, ya are not read: bf16 storage); 3 = the states the forward stored in `mid` replace
                      // the rebuilt ones
  int mid_end;        // the state after the LAST step is stored / read as well (bf16 storage: y, ya are not read)
};

template <int NC, int LD, int KF>
struct FeatGeom {
  static_assert(KF % 2 == 0 && 32 % LD == 0, "features are processed in pairs");
  static constexpr int D = LD * KF;
  static constexpr int SLOTS = 32 / LD;
  static constexpr int P = NC >= SLOTS ? NC / SLOTS : 1;  // positions per lane
  static constexpr int SEG = NC >= SLOTS ? SLOTS : NC;    // slots of one group
  static constexpr int GPW = SLOTS / SEG;                 // groups per warp
  static constexpr int KP = KF / 2;
  static_assert(P * SEG == NC, "n_cache must be a power of two");
};
constexpr int kFeatWarps = 8;  // warps per CTA
constexpr int kFeatBwdUnroll = NCN_FEAT_UNROLL;  // backward step loop; 2 measured 10-40 % slower (register spills, code size)
constexpr int ilog2(int v) { return v <= 1 ? 0 : 1 + ilog2(v >> 1); }

__device__ __forceinline__ float2 shfl2(float2 v, int src) {
  return make_float2(__shfl_sync(0xffffffffu, v.x, src), __shfl_sync(0xffffffffu, v.y, src));
}
// sum over the LD lanes that share a position
template <int LD>
__device__ __forceinline__ float red_sub(float v) {
#pragma unroll
  for (int o = 1; o < LD; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
// sum over the SEG slots of a group (lanes LD apart), every lane gets the result
template <int LD, int SEG>
__device__ __forceinline__ float red_slots(float v) {
#pragma unroll
  for (int o = LD; o < LD * SEG; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <int KF, typename T>
__device__ __forceinline__ void ld_feat(const T* p, float2 (&v)[KF / 2]) {
  float t[KF];
  ld_vec<KF>(p, t);
#pragma unroll
  for (int q = 0; q < KF / 2; ++q) v[q] = make_float2(t[2 * q], t[2 * q + 1]);
}
template <int KF, typename T>
__device__ __forceinline__ void st_feat(T* p, const float2 (&v)[KF / 2]) {
  float t[KF];
#pragma unroll
  for (int q = 0; q < KF / 2; ++q) { t[2 * q] = v[q].x; t[2 * q + 1] = v[q].y; }
  st_vec<KF>(p, t);
}

// Work split shared by both directions: warp -> head c (fixed for the whole kernel, so the
// weights and the weight-gradient sums of a lane stay in registers), units of that head.
struct FeatWarp {
  int c;
  long long first, step;
};
__device__ __forceinline__ FeatWarp feat_warp(const FeatParams& p) {
  const long long wg = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long tw = (long long)gridDim.x * (blockDim.x >> 5);  // a multiple of C (launch plan)
  FeatWarp w;
  w.c = (int)(wg % p.C);
  w.first = wg / p.C;
  w.step = tw / p.C;
  return w;
}

// ------------------------------------------------------------------------------------------ forward
// MID: the fp32 state after every 16th step is also written to p.mid, for a backward whose inverse
// chains then never exceed 16 steps.
template <int NC, int LD, int KF, int ACT, typename T, bool MID = false, typename PT = FeatParams>
__global__ void __launch_bounds__(kFeatWarps * 32) feat_fwd_kernel(const PT p) {
  using G = FeatGeom<NC, LD, KF>;
  using F = ActForm<ACT>;
  constexpr int P = G::P, SEG = G::SEG, KP = G::KP;
  constexpr float sT = (float)F::sT;
  constexpr float cf0 = (float)(kCd * F::f0), cf1 = (float)(kCd * F::f1);
  const int lane = threadIdx.x & 31;
  const int sub = lane & (LD - 1), slot = lane / LD;
  const int gw = slot / SEG, s = slot - gw * SEG;
  const FeatWarp fw = feat_warp(p);
  const T* gx = static_cast<const T*>(p.in[0]);
  const T* ga = static_cast<const T*>(p.in[1]);
  T* gy = static_cast<T*>(p.out[0]);
  T* gya = static_cast<T*>(p.out[1]);

  // this lane's weights, with (1 - alpha) and the activation's argument scale folded in
  float2 Wi[KP], Wj[KP];
  {
    const float* wi = p.W + fw.c * G::D + sub * KF;
    const float* wj = wi + p.E;
    const float f = p.oma * sT;
#pragma unroll
    for (int q = 0; q < KP; ++q) {
      Wi[q] = make_float2(wi[2 * q] * f, wi[2 * q + 1] * f);
      Wj[q] = make_float2(wj[2 * q] * f, wj[2 * q + 1] * f);
    }
  }
  const float2 alpha_s = f2(p.alpha * sT);

  for (long long u = fw.first; u < p.units; u += fw.step) {
    const long long b = u / p.mg;
    const int g = (int)(u - b * p.mg) * G::GPW + gw;
    const bool valid = g < p.m;
    float2 X[P][KP], A[P][KP];
    long long off[P];
#pragma unroll
    for (int r = 0; r < P; ++r) {
      const int i = r * SEG + s;
      const int blk = (int)(((long long)g + (long long)i * p.stride) % p.m);
      off[r] = ((b * p.N + (long long)blk * NC + i) * p.E) + fw.c * G::D + sub * KF;
      if (valid) {
        ld_feat<KF, T>(gx + off[r], X[r]);
        ld_feat<KF, T>(ga + off[r], A[r]);
      } else {
#pragma unroll
        for (int q = 0; q < KP; ++q) X[r][q] = A[r][q] = f2(0.0f);
      }
    }
    [[maybe_unused]] auto store_mid = [&](int done) {  // the state after `done` steps, for the backward (MID)
      if constexpr (MID) {
        if (valid) {
          float* mx = p.mid + (long long)(2 * (done / 16 - 1)) * p.bne;
#pragma unroll
          for (int r = 0; r < P; ++r) {
            st_feat<KF, float>(mx + off[r], X[r]);
            st_feat<KF, float>(mx + p.bne + off[r], A[r]);
          }
        }
      }
    };
#pragma unroll
    for (int rj = 0; rj < P; ++rj) {
#pragma unroll 1
      for (int sj = 0; sj < SEG; ++sj) {
        const int src = (gw * SEG + sj) * LD + sub;
        float2 xj[KP];
        float2 accj = f2(0.0f);
#pragma unroll
        for (int q = 0; q < KP; ++q) {
          xj[q] = shfl2(X[rj][q], src);
          accj = __ffma2_rn(xj[q], Wj[q], accj);
        }
        const float cj = accj.x + accj.y;
#pragma unroll
        for (int r = 0; r < P; ++r) {
          float2 acc = f2(0.0f);
#pragma unroll
          for (int q = 0; q < KP; ++q) acc = __ffma2_rn(X[r][q], Wi[q], acc);
          const float2 sim = f2(red_sub<LD>(acc.x + acc.y + cj));  // sT (1-alpha)(x_i.Wi + x_j.Wj)
          // the forward is bound by the special-function unit: the reciprocals of a position's feature
          // pairs come from one reciprocal of their product
          float2 ts[KP], rr[KP];
#pragma unroll
          for (int q = 0; q < KP; ++q) ts[q] = __ffma2_rn(sim, xj[q], __fmul2_rn(X[r][q], alpha_s));
          if constexpr (KP >= 2 && NCN_FEAT_FWD_BATCH > 1) {
            act_r_all<ACT, KP, NCN_FEAT_FWD_BATCH>(ts, rr);
          } else {
#pragma unroll
            for (int q = 0; q < KP; ++q) rr[q] = F::r(ts[q]);
          }
#pragma unroll
          for (int q = 0; q < KP; ++q) {
            A[r][q] = __ffma2_rn(rr[q], f2(cf1), __ffma2_rn(A[r][q], f2(kM), f2(cf0)));
            X[r][q] = __ffma2_rn(A[r][q], f2(kC), __fmul2_rn(X[r][q], f2(kM)));
          }
        }
        if constexpr (MID && SEG > 16) {  // a boundary of 16 steps inside this run of SEG steps
          const int done = rj * SEG + sj + 1;
          if ((done & 15) == 0 && (done < NC || p.mid_end)) store_mid(done);
        }
      }
      if constexpr (MID && SEG <= 16) {  // boundaries of 16 steps fall between two runs (rj is unrolled: known at compile time)
        const int done = (rj + 1) * SEG;
        if ((done & 15) == 0 && (done < NC || p.mid_end)) store_mid(done);
      }
    }
    if (valid) {
#pragma unroll
      for (int r = 0; r < P; ++r) {
        st_feat<KF, T>(gy + off[r], X[r]);
        st_feat<KF, T>(gya + off[r], A[r]);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------ backward
// From the stage OUTPUT (y, ya) and the cotangents (dy, dya): every step first rebuilds its input
// by the reversible inverse, then applies the closed-form vector-Jacobian product.  Per step j and
// position i (features k; sums over k are the dot products):
//     x_i = (y_i - c ya_i) / m ;  sim_i = (1-alpha)(x_i.Wi + x_j.Wj) ;  T = alpha x_i + sim_i x_j
//     a_i = (ya_i - c F(T)) / m
//     gA' = ga + c gy ;  gT = c gA' act'(T) ;  ga <- m gA' ;  gs_i = (1-alpha) gT_i.x_j
//     gx_i = m gy_i + alpha gT_i + gs_i Wi
//     gx_j += Wj sum_i gs_i + sum_i sim_i gT_i          (position j in its role as x_j)
//     dWi += sum_i gs_i x_i ;  dWj += (sum_i gs_i) x_j
// The weight gradient is summed per lane over all its groups, then over the slots of the warp
// (fixed shuffle tree), the warps of the CTA that serve the same head (warp order) and the CTAs
// (dw_reduce_kernel): a fixed order for a given launch shape.
//
// SAVED: the caller also kept the stage INPUT.  Every inverse step grows earlier rounding by 1/m, so
// a chain of NC = 32 steps from the output alone leaves the gradients at 1e-5 of their size; here
// the state half way is rebuilt exactly by running the forward over the first NC/2 steps from the
// input, so that no inverse chain is longer than NC/2 steps.  With bf16 storage (p.saved == 2) the
// end state is replayed too: an inverse started from rounded outputs would amplify their rounding.
template <int NC, int LD, int KF, int ACT, typename T, bool SAVED = false, typename PT = FeatParams>
__global__ void __launch_bounds__(kFeatWarps * 32) feat_bwd_kernel(const PT p) {
  using G = FeatGeom<NC, LD, KF>;
  using F = ActForm<ACT>;
  constexpr int P = G::P, SEG = G::SEG, KP = G::KP, D = G::D;
  constexpr float sT = (float)F::sT;
  constexpr float cds = (float)(kCd * F::ds);                 // gT = cds * gt
  constexpr float af0 = (float)(-kCd * F::f0 / kMd), af1 = (float)(-kCd * F::f1 / kMd);
  constexpr float ff0 = (float)(kCd * F::f0), ff1 = (float)(kCd * F::f1);  // forward replay (SAVED)
  __shared__ float sdw[kFeatWarps][2][D];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane & (LD - 1), slot = lane / LD;
  const int gw = slot / SEG, s = slot - gw * SEG;
  const FeatWarp fw = feat_warp(p);
  const T* g_y = static_cast<const T*>(p.in[0]);
  const T* g_ya = static_cast<const T*>(p.in[1]);
  const T* g_dy = static_cast<const T*>(p.in[2]);
  const T* g_dya = static_cast<const T*>(p.in[3]);
  T* g_dx = static_cast<T*>(p.out[0]);
  T* g_dxa = static_cast<T*>(p.out[1]);
  T* g_xr = static_cast<T*>(p.out[2]);
  T* g_xar = static_cast<T*>(p.out[3]);

  float2 Wi[KP], Wj[KP];  // (1 - alpha) folded in
  {
    const float* wi = p.W + fw.c * D + sub * KF;
    const float* wj = wi + p.E;
#pragma unroll
    for (int q = 0; q < KP; ++q) {
      Wi[q] = make_float2(wi[2 * q] * p.oma, wi[2 * q + 1] * p.oma);
      Wj[q] = make_float2(wj[2 * q] * p.oma, wj[2 * q + 1] * p.oma);
    }
  }
  const float2 alpha_s = f2(p.alpha * sT);
  const float2 alpha_g = f2(p.alpha * cds);
  float2 dwi[KP], dwj[KP];  // without the factor (1 - alpha)
#pragma unroll
  for (int q = 0; q < KP; ++q) dwi[q] = dwj[q] = f2(0.0f);

  for (long long u = fw.first; u < p.units; u += fw.step) {
    const long long b = u / p.mg;
    const int g = (int)(u - b * p.mg) * G::GPW + gw;
    const bool valid = g < p.m;
    float2 X[P][KP], A[P][KP], H[P][KP], Gv[P][KP];
    long long off[P];
#pragma unroll
    for (int r = 0; r < P; ++r) {
      const int i = r * SEG + s;
      const int blk = (int)(((long long)g + (long long)i * p.stride) % p.m);
      off[r] = ((b * p.N + (long long)blk * NC + i) * p.E) + fw.c * D + sub * KF;
      if (valid) {
        bool from_output = true;  // (stored end state or full replay: y, ya are not read)
        if constexpr (SAVED) from_output = !(p.saved == 2 || (p.saved == 3 && p.mid_end));
        if (from_output) {
          ld_feat<KF, T>(g_y + off[r], X[r]);
          ld_feat<KF, T>(g_ya + off[r], A[r]);
        }
        ld_feat<KF, T>(g_dy + off[r], H[r]);
        ld_feat<KF, T>(g_dya + off[r], Gv[r]);
        if constexpr (SAVED) {
          // the stored state is needed half a stage from now: towards L2 already (one lane per 128-byte line)
          if (p.saved == 3 && (sub & (128 / (KF * 4) - 1)) == 0) {
            const float* mx = p.mid + off[r];
            asm volatile("prefetch.global.L2 [%0];" ::"l"(mx));
            asm volatile("prefetch.global.L2 [%0];" ::"l"(mx + p.bne));
          }
        }
      } else {
#pragma unroll
        for (int q = 0; q < KP; ++q) X[r][q] = A[r][q] = H[r][q] = Gv[r][q] = f2(0.0f);
      }
    }
    // SAVED: the steps go in two runs of NC / 2; what replaces the rebuilt state (stored by the forward, or replayed
    // from the saved input) is dealt with between the runs, outside the step loop.  Otherwise one run of NC steps.
    constexpr int RUN = SAVED ? NC / 2 : NC;
#pragma unroll 1
    for (int j0 = NC - 1; j0 >= 0; j0 -= RUN) {
      if constexpr (SAVED) {
        const int j = j0;  // the state wanted is the one after step j0
        if (p.saved == 3) {
          // the state after step j as the forward stored it
          if (((j + 1) & 15) == 0 && (j + 1 < NC || p.mid_end) && valid) {
            const float* mx = p.mid + (long long)(2 * ((j + 1) / 16 - 1)) * p.bne;
#pragma unroll
            for (int r = 0; r < P; ++r) {
              ld_feat<KF, float>(mx + off[r], X[r]);
              ld_feat<KF, float>(mx + p.bne + off[r], A[r]);
            }
          }
        } else if (j == NC / 2 - 1 || (j == NC - 1 && p.saved == 2)) {
          // the state after step j, exactly: the forward over steps 0..j from the saved input
          const T* g_x = static_cast<const T*>(p.xin[0]);
          const T* g_xa = static_cast<const T*>(p.xin[1]);
          if (valid) {
#pragma unroll
            for (int r = 0; r < P; ++r) {
              ld_feat<KF, T>(g_x + off[r], X[r]);
              ld_feat<KF, T>(g_xa + off[r], A[r]);
            }
          }
#pragma unroll 1
          for (int jf = 0; jf <= j; ++jf) {
            const int rf = jf / SEG, sf = jf - rf * SEG;
            const int srcf = (gw * SEG + sf) * LD + sub;
            float2 xf[KP];
            float2 accf = f2(0.0f);
#pragma unroll
            for (int q = 0; q < KP; ++q) {
              float2 v = X[0][q];
#pragma unroll
              for (int r = 1; r < P; ++r)
                if (rf == r) v = X[r][q];
              xf[q] = shfl2(v, srcf);
              accf = __ffma2_rn(xf[q], Wj[q], accf);
            }
            const float cf = accf.x + accf.y;
#pragma unroll
            for (int r = 0; r < P; ++r) {
              float2 acc = f2(0.0f);
#pragma unroll
              for (int q = 0; q < KP; ++q) acc = __ffma2_rn(X[r][q], Wi[q], acc);
              const float2 sim_s = f2(red_sub<LD>(acc.x + acc.y + cf) * sT);
#pragma unroll
              for (int q = 0; q < KP; ++q) {
                const float2 rr = F::r(__ffma2_rn(sim_s, xf[q], __fmul2_rn(X[r][q], alpha_s)));
                A[r][q] = __ffma2_rn(rr, f2(ff1), __ffma2_rn(A[r][q], f2(kM), f2(ff0)));
                X[r][q] = __ffma2_rn(A[r][q], f2(kC), __fmul2_rn(X[r][q], f2(kM)));
              }
            }
          }
        }
      }
#pragma unroll kFeatBwdUnroll
    for (int j = j0; j > j0 - RUN; --j) {
      // one body for every step: the row index of x_j inside a lane (rj) is a run-time value,
      // resolved by selects, so that the code stays small enough for the instruction cache
      const int rj = j / SEG, sj = j - rj * SEG;
      const int src = (gw * SEG + sj) * LD + sub;
      const bool is_j = (s == sj);
      // the step's input x for every position, then the row x_j
#pragma unroll
      for (int r = 0; r < P; ++r)
#pragma unroll
        for (int q = 0; q < KP; ++q) X[r][q] = __ffma2_rn(A[r][q], f2(-kCoverM), __fmul2_rn(X[r][q], f2(kInvM)));
      float2 xj[KP];
      float2 accj = f2(0.0f);
#pragma unroll
      for (int q = 0; q < KP; ++q) {
        float2 v = X[0][q];
#pragma unroll
        for (int r = 1; r < P; ++r)
          if (rj == r) v = X[r][q];
        xj[q] = shfl2(v, src);
        accj = __ffma2_rn(xj[q], Wj[q], accj);
      }
      const float cj = accj.x + accj.y;
      float gs[P];
      float u[KF];  // sum_i sim_i gT_i of this lane's positions, per feature
#pragma unroll
      for (int k = 0; k < KF; ++k) u[k] = 0.0f;
#pragma unroll
      for (int r = 0; r < P; ++r) {
        float2 acc = f2(0.0f);
#pragma unroll
        for (int q = 0; q < KP; ++q) acc = __ffma2_rn(X[r][q], Wi[q], acc);
        const float sim = red_sub<LD>(acc.x + acc.y + cj);
        const float2 sim_s = f2(sim * sT), simg = f2(sim * cds);
        float2 gacc = f2(0.0f);
        float2 tsv[KP], rrv[KP];
#pragma unroll
        for (int q = 0; q < KP; ++q) tsv[q] = __ffma2_rn(sim_s, xj[q], __fmul2_rn(X[r][q], alpha_s));
        if constexpr (KP >= 2 && NCN_FEAT_BWD_BATCH > 1) {
          act_r_all<ACT, KP, NCN_FEAT_BWD_BATCH>(tsv, rrv);
        } else {
#pragma unroll
          for (int q = 0; q < KP; ++q) rrv[q] = F::r(tsv[q]);
        }
#pragma unroll
        for (int q = 0; q < KP; ++q) {
          const float2 ts = tsv[q];
          const float2 rr = rrv[q];
          A[r][q] = __ffma2_rn(rr, f2(af1), __ffma2_rn(A[r][q], f2(kInvM), f2(af0)));
          const float2 gap = __ffma2_rn(f2(kC), H[r][q], Gv[r][q]);
          const float2 gt = F::gt(gap, ts, rr);
          Gv[r][q] = __fmul2_rn(gap, f2(kM));
          H[r][q] = __ffma2_rn(gt, alpha_g, __fmul2_rn(H[r][q], f2(kM)));  // gs_i Wi is added below
          gacc = __ffma2_rn(gt, xj[q], gacc);
          const float2 uu = __ffma2_rn(simg, gt, make_float2(u[2 * q], u[2 * q + 1]));
          u[2 * q] = uu.x; u[2 * q + 1] = uu.y;
        }
        gs[r] = red_sub<LD>(gacc.x + gacc.y) * cds;  // gT_i . x_j
      }
      float sl = 0.0f;
#pragma unroll
      for (int r = 0; r < P; ++r) {
        const float2 gsv = f2(gs[r]);
        sl += gs[r];
#pragma unroll
        for (int q = 0; q < KP; ++q) {
          H[r][q] = __ffma2_rn(gsv, Wi[q], H[r][q]);
          dwi[q] = __ffma2_rn(gsv, X[r][q], dwi[q]);
        }
      }
      const float S = red_slots<LD, SEG>(sl);
      // column sums over the group's slots: halving exchange (each round a lane keeps one half of
      // its values and receives the partner's sums for that half), then the owners hand every
      // feature's total to the lanes of position j
      constexpr int ROUNDS = (KF < SEG) ? ilog2(KF) : ilog2(SEG);
      constexpr int LEFT = KF >> ROUNDS;  // values a lane still holds
#pragma unroll
      for (int t = 0; t < ROUNDS; ++t) {
        const int half = KF >> (t + 1);
        const bool up = ((s >> t) & 1) != 0;
#pragma unroll
        for (int i = 0; i < half; ++i) {
          const float keep = up ? u[i + half] : u[i];
          const float send = up ? u[i] : u[i + half];
          u[i] = keep + __shfl_xor_sync(0xffffffffu, send, LD << t);
        }
      }
      if constexpr (LEFT == 1) {
#pragma unroll
        for (int o = LD << ROUNDS; o < LD * SEG; o <<= 1) u[0] += __shfl_xor_sync(0xffffffffu, u[0], o);
      }
      const int base = lane - ((s & ((1 << ROUNDS) - 1)) * LD);
      float col[KF];
#pragma unroll
      for (int f = 0; f < KF; ++f) {
        int owner = 0;  // slot bits of the lane that ends up with feature f
#pragma unroll
        for (int t = 0; t < ROUNDS; ++t) owner |= ((f / (KF >> (t + 1))) & 1) << t;
        col[f] = __shfl_sync(0xffffffffu, u[f % LEFT], base + owner * LD);
      }
#pragma unroll
      for (int q = 0; q < KP; ++q) {
        const float2 add = __ffma2_rn(f2(S), Wj[q], make_float2(col[2 * q], col[2 * q + 1]));
#pragma unroll
        for (int r = 0; r < P; ++r)
          if (is_j && rj == r) H[r][q] = __fadd2_rn(H[r][q], add);
        if (is_j) dwj[q] = __ffma2_rn(f2(S), xj[q], dwj[q]);
      }
    }
    }  // runs
    if (valid) {
#pragma unroll
      for (int r = 0; r < P; ++r) {
        st_feat<KF, T>(g_dx + off[r], H[r]);
        st_feat<KF, T>(g_dxa + off[r], Gv[r]);
        if (g_xr) {
          st_feat<KF, T>(g_xr + off[r], X[r]);
          st_feat<KF, T>(g_xar + off[r], A[r]);
        }
      }
    }
  }

  // ---- weight gradient: slots of the warp, warps of the same head, then the CTA's partial
#pragma unroll
  for (int q = 0; q < KP; ++q) {
#pragma unroll
    for (int o = LD; o < 32; o <<= 1) {
      dwi[q].x += __shfl_xor_sync(0xffffffffu, dwi[q].x, o);
      dwi[q].y += __shfl_xor_sync(0xffffffffu, dwi[q].y, o);
      dwj[q].x += __shfl_xor_sync(0xffffffffu, dwj[q].x, o);
      dwj[q].y += __shfl_xor_sync(0xffffffffu, dwj[q].y, o);
    }
  }
  if (slot == 0) {
#pragma unroll
    for (int q = 0; q < KP; ++q) {
      sdw[warp][0][sub * KF + 2 * q] = dwi[q].x * p.oma;
      sdw[warp][0][sub * KF + 2 * q + 1] = dwi[q].y * p.oma;
      sdw[warp][1][sub * KF + 2 * q] = dwj[q].x * p.oma;
      sdw[warp][1][sub * KF + 2 * q + 1] = dwj[q].y * p.oma;
    }
  }
  __syncthreads();
  const int nwarp = blockDim.x >> 5;
  for (int idx = threadIdx.x; idx < 2 * p.E; idx += blockDim.x) {
    const int which = idx / p.E, f = idx - which * p.E;
    const int c = f / D, k = f - c * D;
    float acc = 0.0f;
    for (int w = 0; w < nwarp; ++w) {
      const long long wg = (long long)blockIdx.x * nwarp + w;
      if ((int)(wg % p.C) == c) acc += sdw[w][which][k];
    }
    p.partials[(long long)blockIdx.x * 2 * p.E + idx] = acc;
  }
}

}  // namespace ncn
