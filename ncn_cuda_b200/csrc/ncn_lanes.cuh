// Register-resident fused row kernels (one feature per position, power-of-two block count).
//
// The kernels of ncn_pairs.cuh send every stream of every position through shared memory at every
// stage boundary.  Here a thread keeps its share of the row in registers for the whole stack:
//
//   * A thread owns G CONSECUTIVE groups g = G t .. G t + G-1 of its row, packed two groups per
//     fp32x2 instruction.  For offset o the values D_o[blk] of a row form an array over the m blocks;
//     a stage with block stride s lets group g work on D_o[(g + o s) mod m]
//     (torch_ref/ncn_pytorch.py:12-41).  Offset 0 therefore never moves, and going from stride s to
//     stride s' shifts the array of offset o by o (s' - s) blocks against the threads.
//   * Such a shift is a warp shuffle for all but the first (last) few lanes of a warp; those take
//     their values from the neighbouring warp through a small halo in shared memory (one CTA
//     barrier per stage, two halo buffers used alternately).  Shifts too long for that go through
//     the tile buffer (write, barrier, read at the shifted index).
//   * Rows arrive and leave by 1-D TMA bulk copies through ONE tile buffer in native layout, which
//     is idle while the stages run; a thread's G groups are G n contiguous positions at stride 0.
//   * tanh / sigmoid need r = 1 / (1 + 2^t) per position and step.  The n reciprocals of a group are
//     taken four at a time from ONE special-function reciprocal of their product (Montgomery's
//     trick): 1.25 instead of 2 special-function instructions per position and step.
//
// Stored states (checkpoints) are written straight from registers, in the order [stream][offset][pair of
// groups of the stage]; that order differs from the one of ncn_pairs.cuh / ncn_rows.cuh, so a forward
// of this family (this file and ncn_lanes_pipe.cuh) must be paired with a backward of this family
// (the launch plan sees to it).
#pragma once
#include "ncn_pairs.cuh"
#include "ncn_lanes_launch.h"

namespace ncn {

__device__ __forceinline__ float lds32(uint32_t a) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a) : "memory");
  return v;
}
__device__ __forceinline__ void sts32(uint32_t a, float v) {
  asm volatile("st.shared.f32 [%0], %1;" ::"r"(a), "f"(v) : "memory");
}
// Asks for `bytes` (a multiple of 16) at `src` to be brought into L2; no completion to wait for.
__device__ __forceinline__ void l2_prefetch(const void* src, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}
// Predicated forms: ONE instruction under a predicate instead of a branch around the access, so
// that a halo access of a few lanes does not split the basic block it sits in.
__device__ __forceinline__ void sts64_if(bool on, uint32_t a, float x, float y) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.s32 p, %3, 0;\n\t@p st.shared.v2.f32 [%0], {%1, %2};\n\t}" ::"r"(a), "f"(x), "f"(y), "r"((int)on)
               : "memory");
}
__device__ __forceinline__ void sts32_if(bool on, uint32_t a, float v) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.s32 p, %2, 0;\n\t@p st.shared.f32 [%0], %1;\n\t}" ::"r"(a), "f"(v), "r"((int)on) : "memory");
}
__device__ __forceinline__ void lds64_if(bool on, uint32_t a, float2& v) {  // v keeps its value where !on
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.s32 p, %3, 0;\n\t@p ld.shared.v2.f32 {%0, %1}, [%2];\n\t}" : "+f"(v.x), "+f"(v.y) : "r"(a), "r"((int)on)
               : "memory");
}
__device__ __forceinline__ void lds32_if(bool on, uint32_t a, float& v) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.s32 p, %2, 0;\n\t@p ld.shared.f32 %0, [%1];\n\t}" : "+f"(v) : "r"(a), "r"((int)on) : "memory");
}

// ------------------------------------------------------------------ activation, all positions of a group at once
// Measured on the arithmetic alone (microbench.cu): the forward is bound by the special-function pipe
// and wants the largest batch; the backward is bound by the FMA pipe, where groups of 8 do better
// with batches of two (17.3 against 18.5 cycles per warp.position.step), groups of 4 with four.
template <int NG>
struct LaneBatch {
  static constexpr int fwd = 4;
  static constexpr int bwd = NG >= 8 ? 2 : 4;
};

// ------------------------------------------------------------------ step math (scaled variables of ncn_common.cuh)
template <int NG, int ACT, int J>
struct LFwdSteps {
  static __device__ __forceinline__ void run(float2 (&X)[NG], float2 (&A)[NG], const PairW& w) {
    using F = ActForm<ACT>;
    constexpr float mk = (float)cpow(kMd, J);
    constexpr float mkDk = (float)(cpow(kMd, J) * fwd_D(J, F::f0));
    constexpr float cA = (float)(kCd * F::f1 / cpow(kMd, J + 1));
    float2 xj, P, Q;
    if constexpr (J == 0) {
      xj = X[0];
      P = ffma2(w.owi, xj, w.alpha);
      Q = fmul2(fmul2(w.owj, xj), xj);
    } else {
      xj = ffma2(X[J], f2(mk), f2(mkDk));
      const float2 pp = ffma2(w.owi, xj, w.alpha);
      P = fmul2(pp, f2(mk));
      const float2 q0 = fmul2(fmul2(w.owj, xj), xj);
      if constexpr (mkDk != 0.0f) Q = ffma2(pp, f2(mkDk), q0); else Q = q0;
    }
    float2 ts[NG], r[NG];
#pragma unroll
    for (int i = 0; i < NG; ++i) ts[i] = ffma2(X[i], P, Q);
    act_r_all<ACT, NG, LaneBatch<NG>::fwd>(ts, r);
#pragma unroll
    for (int i = 0; i < NG; ++i) {
      A[i] = ffma2(r[i], f2(cA), A[i]);
      X[i] = ffma2(A[i], f2(kC), X[i]);
    }
    LFwdSteps<NG, ACT, J + 1>::run(X, A, w);
  }
};
template <int NG, int ACT>
struct LFwdSteps<NG, ACT, NG> {
  static __device__ __forceinline__ void run(float2 (&)[NG], float2 (&)[NG], const PairW&) {}
};

template <int NG, int ACT>
__device__ __forceinline__ void lane_forward(float2 (&X)[NG], float2 (&A)[NG], const PairW& w) {
  using F = ActForm<ACT>;
  LFwdSteps<NG, ACT, 0>::run(X, A, w);
  constexpr float mN = (float)cpow(kMd, NG);
  constexpr float mNC = (float)(cpow(kMd, NG) * fwd_C(NG, F::f0));
  constexpr float mND = (float)(cpow(kMd, NG) * fwd_D(NG, F::f0));
#pragma unroll
  for (int i = 0; i < NG; ++i) {
    if constexpr (mND != 0.0f) X[i] = ffma2(X[i], f2(mN), f2(mND)); else X[i] = fmul2(X[i], f2(mN));
    if constexpr (mNC != 0.0f) A[i] = ffma2(A[i], f2(mN), f2(mNC)); else A[i] = fmul2(A[i], f2(mN));
  }
}

// Reverse sweep as PBwdSteps (ncn_pairs.cuh) with the per-step scalars cut down: the sums for gx_j
// and the weight gradients stay in raw units (dwi_raw = sum xj (aI + DX aS), dwj_raw = sum m^k xj^2 aS)
// and take their constant factors once per stage.
template <int NG, int ACT, int J>
struct LBwdSteps {
  static __device__ __forceinline__ void run(float2 (&X)[NG], float2 (&A)[NG], float2 (&H)[NG], float2 (&G)[NG],
                                             const PairWB& w, float2& dwi, float2& dwj) {
    using F = ActForm<ACT>;
    constexpr int k = NG - 1 - J;
    constexpr double mkd = cpow(kMd, k);
    constexpr float imk1 = (float)(1.0 / cpow(kMd, k + 1));
    constexpr float DX1 = (float)bwd_DX(k + 1, F::f0);
    constexpr float imk1DX1 = (float)(bwd_DX(k + 1, F::f0) / cpow(kMd, k + 1));
    constexpr float cAr = (float)(-kCd * F::f1 * mkd);
    constexpr float sTimk1 = (float)(F::sT / cpow(kMd, k + 1));
    constexpr float cdsm = (float)(kCd * F::ds / kMd);
    constexpr float K1 = (float)(kCd * F::ds / kMd / cpow(kMd, k + 1));  // c ds / m^(k+2)
    constexpr float twomk1 = (float)(2.0 * cpow(kMd, k + 1));
    constexpr float mk = (float)mkd;
#pragma unroll
    for (int i = 0; i < NG; ++i) X[i] = ffma2(f2(-kC), A[i], X[i]);
    float2 xj;
    if constexpr (imk1DX1 != 0.0f) xj = ffma2(X[J], f2(imk1), f2(imk1DX1)); else xj = fmul2(X[J], f2(imk1));
    const float2 pp = ffma2(w.owi, xj, w.alpha);  // p = alpha + (1-alpha) wi xj
    const float2 Ps = fmul2(pp, f2(sTimk1));
    const float2 q0 = fmul2(fmul2(w.owjs, xj), xj);
    float2 Qs;
    if constexpr (DX1 != 0.0f) Qs = ffma2(Ps, f2(DX1), q0); else Qs = q0;
    const float2 PH = fmul2(pp, f2(cdsm));
    float2 ts[NG], r[NG];
#pragma unroll
    for (int i = 0; i < NG; ++i) ts[i] = ffma2(X[i], Ps, Qs);
    act_r_all<ACT, NG, LaneBatch<NG>::bwd>(ts, r);
    float2 aI, aS;  // sums over the group's positions; the first term starts them (no zeroing, no add to zero)
#pragma unroll
    for (int i = 0; i < NG; ++i) {
      A[i] = ffma2(r[i], f2(cAr), A[i]);
      G[i] = ffma2(f2(kC), H[i], G[i]);
      const float2 gt = F::gt(G[i], ts[i], r[i]);
      H[i] = ffma2(gt, PH, H[i]);
      if (i == 0) {
        aI = fmul2(gt, X[0]);
        aS = gt;
      } else {
        aI = ffma2(gt, X[i], aI);
        aS = fadd2(aS, gt);
      }
    }
    float2 u;
    if constexpr (DX1 != 0.0f) u = ffma2(f2(DX1), aS, aI); else u = aI;  // sum gT x_i = (c ds / m) u
    const float2 v = fmul2(xj, aS);                                       // xj sum gT = c ds m^k v
    // gx_j += (1-alpha) (wi sum gT x + 2 wj xj sum gT), in units of m^(k+1)
    const float2 t3 = ffma2(fmul2(w.owj, v), f2(twomk1), fmul2(w.owi, u));
    H[J] = ffma2(t3, f2(K1), H[J]);
    dwi = ffma2(xj, u, dwi);
    dwj = ffma2(fmul2(xj, v), f2(mk), dwj);
    LBwdSteps<NG, ACT, J - 1>::run(X, A, H, G, w, dwi, dwj);
  }
};
template <int NG, int ACT>
struct LBwdSteps<NG, ACT, -1> {
  static __device__ __forceinline__ void run(float2 (&)[NG], float2 (&)[NG], float2 (&)[NG], float2 (&)[NG],
                                             const PairWB&, float2&, float2&) {}
};

// dwi / dwj gain the RAW sums; their factors are lane_dw_scale_i/j below.
template <int NG, int ACT>
__device__ __forceinline__ void lane_backward(float2 (&X)[NG], float2 (&A)[NG], float2 (&H)[NG], float2 (&G)[NG],
                                              const PairWB& w, float2& dwi, float2& dwj) {
  using F = ActForm<ACT>;
  LBwdSteps<NG, ACT, NG - 1>::run(X, A, H, G, w, dwi, dwj);
  constexpr float imN = (float)(1.0 / cpow(kMd, NG));
  constexpr float imNDX = (float)(bwd_DX(NG, F::f0) / cpow(kMd, NG));
  constexpr float imNCA = (float)(bwd_CA(NG, F::f0) / cpow(kMd, NG));
  constexpr float mN = (float)cpow(kMd, NG);
#pragma unroll
  for (int i = 0; i < NG; ++i) {
    if constexpr (imNDX != 0.0f) X[i] = ffma2(X[i], f2(imN), f2(imNDX)); else X[i] = fmul2(X[i], f2(imN));
    if constexpr (imNCA != 0.0f) A[i] = ffma2(A[i], f2(imN), f2(imNCA)); else A[i] = fmul2(A[i], f2(imN));
    H[i] = fmul2(H[i], f2(mN));
    G[i] = fmul2(G[i], f2(mN));
  }
}
template <int ACT>
__device__ __forceinline__ float lane_dw_scale_i(float oma) {  // (1-alpha) c ds / m
  return oma * (float)(kCd * ActForm<ACT>::ds / kMd);
}
template <int ACT>
__device__ __forceinline__ float lane_dw_scale_j(float oma) {  // (1-alpha) c ds
  return oma * (float)(kCd * ActForm<ACT>::ds);
}

// ------------------------------------------------------------------ exchanges
// V[s][p][o]: stream s, pair p = groups (G t + 2p, G t + 2p + 1), offset o.
template <int NG, int G>
__device__ __forceinline__ float lane_get(const float2 (&S)[G / 2][NG], int o, int j) {
  return (j & 1) ? S[j >> 1][o].y : S[j >> 1][o].x;
}
template <int NG, int G>
__device__ __forceinline__ void lane_set(float2 (&S)[G / 2][NG], int o, int j, float v) {
  if (j & 1) S[j >> 1][o].y = v; else S[j >> 1][o].x = v;
}

__device__ __forceinline__ void cta_sync() { __syncthreads(); }

// Shift of offset o by k = o 2^E blocks: the value of group j comes from D_o index + k (UP = false:
// from higher threads) or - k (UP = true).  halo_pub / halo_nbr: this warp's and the source
// neighbour's halo area of the current buffer (shared-window byte addresses).
template <int NG, int G, int NS, int E, bool UP>
__device__ __forceinline__ void exchange_shfl(float2 (&V)[NS][G / 2][NG], uint32_t halo_pub, uint32_t halo_nbr, int lane) {
  constexpr int D = 1 << E;
  constexpr int HS = lane_halo_floats(NG, E);  // floats per stream
  constexpr int CH = 32 * G;                   // blocks per warp
  if constexpr (E == 0 && G == 2) {
    // One pair per thread and shifts by k = o blocks.  The pair is published whole (for odd k one value more than
    // the neighbour reads); odd shifts swap the halves of a pair: x <- y of lane +- (k-1)/2, y <- x of lane +- (k+1)/2.
#pragma unroll
    for (int s = 0; s < NS; ++s) {
#pragma unroll
      for (int o = 1; o < NG; ++o) {
        const uint32_t reg = halo_pub + 4u * (uint32_t)(s * HS + lane_halo_pair_base(o));
        if (!UP) {
          sts64_if(2 * lane < o, reg + 8u * (uint32_t)lane, V[s][0][o].x, V[s][0][o].y);
        } else {
          const int kb = (CH - o) & ~1;  // first published block, rounded down to a pair
          sts64_if(2 * lane >= kb, reg + 4u * (uint32_t)(2 * lane - kb), V[s][0][o].x, V[s][0][o].y);
        }
      }
    }
    cta_sync();
#pragma unroll
    for (int s = 0; s < NS; ++s) {
#pragma unroll
      for (int o = 1; o < NG; ++o) {
        const uint32_t reg = halo_nbr + 4u * (uint32_t)(s * HS + lane_halo_pair_base(o));
        const float2 v = V[s][0][o];
        float2 n;
        if (o & 1) {
          const int qa = o >> 1, qb = (o + 1) >> 1;
          if (!UP) {
            n.x = qa > 0 ? __shfl_down_sync(0xffffffffu, v.y, qa) : v.y;
            n.y = __shfl_down_sync(0xffffffffu, v.x, qb);
            lds32_if(lane + qa >= 32, reg + 4u * (uint32_t)(2 * lane + o - CH), n.x);
            lds32_if(lane + qb >= 32, reg + 4u * (uint32_t)(2 * lane + o + 1 - CH), n.y);
          } else {
            n.x = __shfl_up_sync(0xffffffffu, v.y, qb);
            n.y = qa > 0 ? __shfl_up_sync(0xffffffffu, v.x, qa) : v.x;
            lds32_if(lane < qb, reg + 4u * (uint32_t)(2 * lane + 1), n.x);  // the lower warp's area starts at block CH - 1 - o
            lds32_if(lane < qa, reg + 4u * (uint32_t)(2 * lane + 2), n.y);
          }
        } else {
          const int q = o >> 1;
          if (!UP) {
            n.x = __shfl_down_sync(0xffffffffu, v.x, q);
            n.y = __shfl_down_sync(0xffffffffu, v.y, q);
            lds64_if(lane + q >= 32, reg + 8u * (uint32_t)(lane + q - 32), n);
          } else {
            n.x = __shfl_up_sync(0xffffffffu, v.x, q);
            n.y = __shfl_up_sync(0xffffffffu, v.y, q);
            lds64_if(lane < q, reg + 8u * (uint32_t)lane, n);
          }
        }
        V[s][0][o] = n;
      }
    }
    return;
  }
  const int c0 = G * lane;
  // ---- publish what the neighbouring warp will want
#pragma unroll
  for (int s = 0; s < NS; ++s) {
#pragma unroll
    for (int o = 1; o < NG; ++o) {
      const int k = o * D;
      const int base = s * HS + D * o * (o - 1) / 2;
      if constexpr (E >= 1) {
#pragma unroll
        for (int p = 0; p < G / 2; ++p) {
          const int c = c0 + 2 * p;
          if (!UP) {
            sts64_if(c < k, halo_pub + 4u * (uint32_t)(base + c), V[s][p][o].x, V[s][p][o].y);
          } else {
            sts64_if(c >= CH - k, halo_pub + 4u * (uint32_t)(base + c - (CH - k)), V[s][p][o].x, V[s][p][o].y);
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < G; ++j) {
          const int c = c0 + j;
          if (!UP) {
            sts32_if(c < k, halo_pub + 4u * (uint32_t)(base + c), lane_get<NG, G>(V[s], o, j));
          } else {
            sts32_if(c >= CH - k, halo_pub + 4u * (uint32_t)(base + c - (CH - k)), lane_get<NG, G>(V[s], o, j));
          }
        }
      }
    }
  }
  cta_sync();
  // ---- fetch
#pragma unroll
  for (int s = 0; s < NS; ++s) {
#pragma unroll
    for (int o = 1; o < NG; ++o) {
      const int k = o * D;
      const int base = s * HS + D * o * (o - 1) / 2;
      float nv[G];
#pragma unroll
      for (int j = 0; j < G; ++j) {
        if (!UP) {
          const int c = j + k, js = c % G, q = c / G;
          float v = lane_get<NG, G>(V[s], o, js);
          if (q > 0) v = __shfl_down_sync(0xffffffffu, v, q);
          nv[j] = v;
        } else {
          const int c = j - k;
          const int js = ((c % G) + G) % G, q = (js - c) / G;
          float v = lane_get<NG, G>(V[s], o, js);
          if (q > 0) v = __shfl_up_sync(0xffffffffu, v, q);
          nv[j] = v;
        }
      }
      if constexpr (E >= 1) {
#pragma unroll
        for (int p = 0; p < G / 2; ++p) {
          const int j = 2 * p;
          if (!UP) {
            const int c = j + k, js = c % G, q = c / G;
            float2 h = make_float2(nv[j], nv[j + 1]);
            lds64_if(lane + q >= 32, halo_nbr + 4u * (uint32_t)(base + G * (lane + q - 32) + js), h);
            nv[j] = h.x; nv[j + 1] = h.y;
          } else {
            const int c = j - k;
            const int js = ((c % G) + G) % G, q = (js - c) / G;
            float2 h = make_float2(nv[j], nv[j + 1]);
            lds64_if(lane < q, halo_nbr + 4u * (uint32_t)(base + G * (lane - q) + js + k), h);
            nv[j] = h.x; nv[j + 1] = h.y;
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < G; ++j) {
          if (!UP) {
            const int c = j + k, js = c % G, q = c / G;
            lds32_if(lane + q >= 32, halo_nbr + 4u * (uint32_t)(base + G * (lane + q - 32) + js), nv[j]);
          } else {
            const int c = j - k;
            const int js = ((c % G) + G) % G, q = (js - c) / G;
            lds32_if(lane < q, halo_nbr + 4u * (uint32_t)(base + G * (lane - q) + js + k), nv[j]);
          }
        }
      }
#pragma unroll
      for (int j = 0; j < G; ++j) lane_set<NG, G>(V[s], o, j, nv[j]);
    }
  }
}

// Shift by any multiple of G blocks per offset through the tile buffer, viewed as fp32 arrays
// [stream][offset][m] of the row (row_addr: shared-window byte address of the row's part of it).
template <int NG, int G, int NS>
__device__ __forceinline__ void exchange_smem(float2 (&V)[NS][G / 2][NG], uint32_t row_addr, int t, int m, int delta) {
  const int mmask = m - 1;
#pragma unroll
  for (int s = 0; s < NS; ++s) {
#pragma unroll
    for (int o = 1; o < NG; ++o) {
      const uint32_t arr = row_addr + 4u * (uint32_t)((s * NG + o) * m);
#pragma unroll
      for (int p = 0; p < G / 2; ++p) sts64(arr + 4u * (uint32_t)(G * t + 2 * p), V[s][p][o].x, V[s][p][o].y);
    }
  }
  cta_sync();
#pragma unroll
  for (int s = 0; s < NS; ++s) {
#pragma unroll
    for (int o = 1; o < NG; ++o) {
      const uint32_t arr = row_addr + 4u * (uint32_t)((s * NG + o) * m);
      const int src = (G * t + o * delta) & mmask;  // multiple of G: the G values stay contiguous
#pragma unroll
      for (int p = 0; p < G / 2; ++p) V[s][p][o] = lds64(arr + 4u * (uint32_t)(src + 2 * p));
    }
  }
  cta_sync();
}

// halo addressing of one thread
struct LaneHalo {
  uint32_t base;        // shared-window address of the halo area (two buffers)
  uint32_t buf_bytes;   // bytes of one buffer = warps per CTA * warp_bytes
  uint32_t warp_bytes;
  int warp, warp_up, warp_dn;  // this warp, and the warps holding the next higher / lower blocks of the row (cyclic)
  int parity;
};

// delta = s_new - s_old (0, or +-2^e).  Shuffle exchange up to 2^ea_max, tile buffer beyond.
template <int NG, int G, int NS>
__device__ __forceinline__ void lane_exchange(float2 (&V)[NS][G / 2][NG], int delta, int ea_max, LaneHalo& h, int lane,
                                              uint32_t row_addr, int t, int m) {
  if (delta == 0) return;
  const bool up = delta < 0;
  const int ad = up ? -delta : delta;
  const int e = 31 - __clz(ad);
  if (e > ea_max) {
    exchange_smem<NG, G, NS>(V, row_addr, t, m, delta);
    return;
  }
  const uint32_t bufa = h.base + (uint32_t)h.parity * h.buf_bytes;
  h.parity ^= 1;
  const uint32_t pub = bufa + (uint32_t)h.warp * h.warp_bytes;
  const uint32_t nbr = bufa + (uint32_t)(up ? h.warp_dn : h.warp_up) * h.warp_bytes;
  constexpr int CAP = lane_ea_cap(NG);
  // one dense switch over (e, direction): a jump table instead of a chain of compares, each of which would be a
  // possibly divergent branch with its own reconvergence point
#define NCN_LANE_CASE(EE)                                                                                   \
  case 2 * EE: if constexpr (CAP >= EE) exchange_shfl<NG, G, NS, EE, false>(V, pub, nbr, lane); break;      \
  case 2 * EE + 1: if constexpr (CAP >= EE) exchange_shfl<NG, G, NS, EE, true>(V, pub, nbr, lane); break;
  switch (2 * e + (up ? 1 : 0)) {
    NCN_LANE_CASE(0)
    NCN_LANE_CASE(1)
    NCN_LANE_CASE(2)
    NCN_LANE_CASE(3)
    NCN_LANE_CASE(4)
    NCN_LANE_CASE(5)
    NCN_LANE_CASE(6)
    default: break;
  }
#undef NCN_LANE_CASE
}

// a thread's G*NG contiguous positions of one stream <-> its registers (stride-0 arrangement).
//
// The chunk is S = G*NG*sizeof(T)/16 sixteen-byte slots, and consecutive lanes are a whole chunk
// apart, so a 128-bit access at the same slot number in every lane would hit the same banks S
// times over.  Lane t therefore starts at slot rot = (t / (8/S)) mod S: instruction i moves slot
// (i + rot) mod S, which spreads the eight lanes of a quarter warp over all 32 banks.  The
// registers then hold the slots in an order that depends on the lane; log2(S) rounds of selects
// put them right.  Those selects double as the copies between the two register orders in play (a
// 128-bit access wants the values of ONE slot in consecutive registers, the packed arithmetic
// wants the values of TWO groups at one offset in a register pair): done here, once per tile and
// on the integer pipe; left to the register allocator such copies ended up inside the step loop.
template <int NG, int G, typename T>
struct LaneChunk {
  static constexpr int EPS = 16 / (int)sizeof(T);   // elements per slot
  static constexpr int S = G * NG / EPS;            // slots per chunk (a power of two)
  static constexpr int LPL = 8 / S > 0 ? 8 / S : 1;  // lanes per 128 bytes
  static __device__ __forceinline__ int rot(int t) { return (t / LPL) & (S - 1); }
};

template <int NG, int G, typename T>
__device__ __forceinline__ void lane_ld_native(const T* chunk, float2 (&Sv)[G / 2][NG], int t) {
  using C = LaneChunk<NG, G, T>;
  constexpr int S = C::S, EPS = C::EPS;
  static_assert(S >= 1 && (S & (S - 1)) == 0, "a whole, power-of-two number of 16-byte slots");
  const int r = C::rot(t);
  float q[S][EPS];
#pragma unroll
  for (int i = 0; i < S; ++i) ld_vec<EPS>(chunk + ((i + r) & (S - 1)) * EPS, q[i]);  // q[i] = slot (i + r) mod S
#pragma unroll
  for (int b = 1; b < S; b <<= 1) {  // q[i] <- q[(i - b) mod S] where bit b of r is set
    const bool on = (r & b) != 0;
    float n[S][EPS];
#pragma unroll
    for (int i = 0; i < S; ++i)
#pragma unroll
      for (int e = 0; e < EPS; ++e) n[i][e] = on ? q[(i - b) & (S - 1)][e] : q[i][e];
#pragma unroll
    for (int i = 0; i < S; ++i)
#pragma unroll
      for (int e = 0; e < EPS; ++e) q[i][e] = n[i][e];
  }
  // q[i][e] is now element i*EPS + e of the chunk = (group, offset) = ((i*EPS + e) / NG, (i*EPS + e) % NG)
#pragma unroll
  for (int p = 0; p < G / 2; ++p)
#pragma unroll
    for (int o = 0; o < NG; ++o) {
      const int ea = (2 * p) * NG + o, eb = (2 * p + 1) * NG + o;
      Sv[p][o] = make_float2(q[ea / EPS][ea % EPS], q[eb / EPS][eb % EPS]);
    }
}
template <int NG, int G, typename T>
__device__ __forceinline__ void lane_st_native(T* chunk, const float2 (&Sv)[G / 2][NG], int t) {
  using C = LaneChunk<NG, G, T>;
  constexpr int S = C::S, EPS = C::EPS;
  const int r = C::rot(t);
  float q[S][EPS];
#pragma unroll
  for (int p = 0; p < G / 2; ++p)
#pragma unroll
    for (int o = 0; o < NG; ++o) {
      const int ea = (2 * p) * NG + o, eb = (2 * p + 1) * NG + o;
      q[ea / EPS][ea % EPS] = Sv[p][o].x;
      q[eb / EPS][eb % EPS] = Sv[p][o].y;
    }
#pragma unroll
  for (int b = 1; b < S; b <<= 1) {  // q[i] <- q[(i + b) mod S] where bit b of r is set
    const bool on = (r & b) != 0;
    float n[S][EPS];
#pragma unroll
    for (int i = 0; i < S; ++i)
#pragma unroll
      for (int e = 0; e < EPS; ++e) n[i][e] = on ? q[(i + b) & (S - 1)][e] : q[i][e];
#pragma unroll
    for (int i = 0; i < S; ++i)
#pragma unroll
      for (int e = 0; e < EPS; ++e) q[i][e] = n[i][e];
  }
#pragma unroll
  for (int i = 0; i < S; ++i) st_vec<EPS>(chunk + ((i + r) & (S - 1)) * EPS, q[i]);  // q[i] = slot (i + r) mod S
}

// ------------------------------------------------------------------------------------------ forward
template <int NG, int ACT, typename T, int MAXT, int MINB>
__global__ void __launch_bounds__(MAXT, MINB) lane_fwd_kernel(const LaneParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  using F = ActForm<ACT>;
  constexpr int G = lane_groups(NG);
  const int tid = threadIdx.x, nthr = blockDim.x;
  const int lane = tid & 31;
  const int N = p.N, m = p.m, R = p.R, L = p.L, TPR = p.tpr;
  const int RN = R * N;
  T* win = reinterpret_cast<T*>(smem + p.off_work);  // native x at win, xa at win + RN
  T* sres = reinterpret_cast<T*>(smem + p.off_res);  // F_RESIDUAL: native x of the tile
  StageRec* recs = reinterpret_cast<StageRec*>(smem + p.off_w);
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem + p.off_bar);
  int* abort_flag = reinterpret_cast<int*>(bar + 2);
  const T* gx_in = static_cast<const T*>(p.in[0]);
  const T* ga_in = static_cast<const T*>(p.in[1]);
  T* gy_out = static_cast<T*>(p.out[0]);
  T* gya_out = static_cast<T*>(p.out[1]);
  float2* ckpt = reinterpret_cast<float2*>(p.ckpt);
  const bool residual = (p.flags & F_RESIDUAL) != 0;
  const long long BN = p.B * (long long)N;

  if (tid == 0) {
    mbar_init(&bar[0], 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  fill_stage_table(recs, p.W, p.oma, p.l0, p.m, p.L, p.ckpt_every, p.flags, ckpt != nullptr, tid, nthr);
  __syncthreads();

  auto issue_load = [&](long long tl) {
    const long long row0 = tl * R;
    const int rows = (int)min((long long)R, p.B - row0);
    const uint32_t bytes = (uint32_t)(rows * N * sizeof(T));
    // (test_short_wait, set by tests of the give-up path only: the barrier expects 16 bytes more than are sent,
    //  so its phase never completes; every copy that IS issued completes as usual)
    mbar_expect_tx(&bar[0], (residual ? 3 : 2) * bytes + (p.test_short_wait ? 16u : 0u));
    bulk_g2s(win, gx_in + row0 * N, bytes, &bar[0]);
    bulk_g2s(win + RN, ga_in + row0 * N, bytes, &bar[0]);
    if (residual) bulk_g2s(sres, gx_in + row0 * N, bytes, &bar[0]);
  };

  const int r = tid / TPR, t = tid - r * TPR;  // row of the tile, thread of the row
  const int wpr = TPR >> 5, wr = t >> 5;
  LaneHalo halo;
  halo.base = smem_u32(smem + p.off_halo);
  halo.warp_bytes = p.halo_warp_bytes;
  halo.buf_bytes = p.halo_warp_bytes * (uint32_t)(nthr >> 5);
  halo.warp = tid >> 5;
  halo.warp_up = r * wpr + (wr + 1 == wpr ? 0 : wr + 1);
  halo.warp_dn = r * wpr + (wr == 0 ? wpr - 1 : wr - 1);
  halo.parity = 0;
  const uint32_t xrow = smem_u32(smem + p.off_work) + (uint32_t)r * (uint32_t)(2 * N) * 4u;  // fp32 [2][NG][m] per row
  const int chunk = r * N + t * (G * NG);  // this thread's positions of the tile
  constexpr float sT = (float)F::sT;
  PairW w;
  w.alpha = f2(p.alpha * sT);
  uint32_t phase = 0;

  for (long long tile = blockIdx.x; tile < p.tiles; tile += gridDim.x) {
    if (tid == 0) {
      bulk_wait_read0();  // the previous tile's stores have left the buffer
      issue_load(tile);
    }
    if (!mbar_wait_bounded(&bar[0], phase, p.test_short_wait ? (1u << 10) : (1u << 22))) *abort_flag = 1;
    phase ^= 1;
    __syncthreads();
    if (*abort_flag) break;

    const long long row0 = tile * R;
    const int rows = (int)min((long long)R, p.B - row0);
    const bool active = r < rows;

    float2 V[2][G / 2][NG];  // x, xa
    if (active) {
      lane_ld_native<NG, G, T>(win + chunk, V[0], t);
      lane_ld_native<NG, G, T>(win + RN + chunk, V[1], t);
    } else {
#pragma unroll
      for (int s = 0; s < 2; ++s)
#pragma unroll
        for (int pp = 0; pp < G / 2; ++pp)
#pragma unroll
          for (int o = 0; o < NG; ++o) V[s][pp][o] = f2(0.0f);
    }
    __syncthreads();  // native inputs are in registers; the buffer is free for long shifts
    if (tid == 0 && tile + gridDim.x < p.tiles) {  // next tile towards L2 while this one is worked on
      const long long nrow0 = (tile + gridDim.x) * R;
      const int nrows = (int)min((long long)R, p.B - nrow0);
      const uint32_t bytes = (uint32_t)(nrows * N * sizeof(T));
      l2_prefetch(gx_in + nrow0 * N, bytes);
      l2_prefetch(ga_in + nrow0 * N, bytes);
    }

    int s_cur = 0;
    StageRec rec_next = recs[0];
    for (int l = 0; l < L; ++l) {
      const StageRec rec = rec_next;
      if (l + 1 < L) rec_next = recs[l + 1];
      lane_exchange<NG, G, 2>(V, rec.s - s_cur, p.ea_max, halo, lane, xrow, t, m);
      s_cur = rec.s;
      w.owi = f2(rec.owi * sT);
      w.owj = f2(rec.owj * sT);
#pragma unroll
      for (int pp = 0; pp < G / 2; ++pp) lane_forward<NG, ACT>(V[0][pp], V[1][pp], w);
      if (rec.ck >= 0 && active) {
        // order of a stored state: [stream][offset][pair of groups], a pair = groups 2q, 2q+1 of the stage
        float2* ck = ckpt + (long long)rec.ck * BN + (row0 + r) * N + (G / 2) * t;
#pragma unroll
        for (int s = 0; s < 2; ++s)
#pragma unroll
          for (int o = 0; o < NG; ++o) {
            if constexpr (G >= 4) {  // a thread's pairs are neighbours in memory: whole 16-byte stores
#pragma unroll
              for (int pp = 0; pp < G / 2; pp += 2)
                *reinterpret_cast<float4*>(ck + (s * NG + o) * (m >> 1) + pp) =
                    make_float4(V[s][pp][o].x, V[s][pp][o].y, V[s][pp + 1][o].x, V[s][pp + 1][o].y);
            } else {
              ck[(s * NG + o) * (m >> 1)] = V[s][0][o];
            }
          }
      }
    }
    lane_exchange<NG, G, 2>(V, -s_cur, p.ea_max, halo, lane, xrow, t, m);  // back to stride 0 = native order
    if (active) {
      if (residual) {
        float2 xin[G / 2][NG];
        lane_ld_native<NG, G, T>(sres + chunk, xin, t);
#pragma unroll
        for (int pp = 0; pp < G / 2; ++pp)
#pragma unroll
          for (int o = 0; o < NG; ++o) V[0][pp][o] = fadd2(V[0][pp][o], xin[pp][o]);
      }
      lane_st_native<NG, G, T>(win + chunk, V[0], t);
      lane_st_native<NG, G, T>(win + RN + chunk, V[1], t);
    }
    fence_proxy_async();
    __syncthreads();
    if (tid == 0) {
      const uint32_t bytes = (uint32_t)(rows * N * sizeof(T));
      bulk_s2g(gy_out + row0 * N, win, bytes);
      bulk_s2g(gya_out + row0 * N, win + RN, bytes);
      bulk_commit();
    }
  }
  if (tid == 0) {
    bulk_wait_all0();
    if (*abort_flag) atomicExch(p.status, DEV_WAIT_TIMEOUT);
  }
}

// ------------------------------------------------------------------------------------------ backward
// From the net output (reversible inverse), from stored states (checkpoints, F_TAPE), F_RESIDUAL; no
// forward replay.
template <int NG, int ACT, typename T, int MAXT, int MINB>
__global__ void __launch_bounds__(MAXT, MINB) lane_bwd_kernel(const LaneParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  using F = ActForm<ACT>;
  constexpr int G = lane_groups(NG);
  const int tid = threadIdx.x, nthr = blockDim.x;
  const int lane = tid & 31, warp = tid >> 5, nwarp = (nthr + 31) >> 5;
  const int N = p.N, m = p.m, R = p.R, L = p.L, TPR = p.tpr;
  const int RN = R * N;
  T* win = reinterpret_cast<T*>(smem + p.off_work);  // native streams q at win + q*RN
  const float2* sck = reinterpret_cast<const float2*>(smem + p.off_ckpt);
  T* sdy = reinterpret_cast<T*>(smem + p.off_res);  // F_RESIDUAL: native dy of the tile
  float* red = reinterpret_cast<float*>(smem + p.off_red);  // [L][nwarp][2]
  StageRec* recs = reinterpret_cast<StageRec*>(smem + p.off_w);
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem + p.off_bar);
  int* abort_flag = reinterpret_cast<int*>(bar + 2);
  const T* g_in[4] = {static_cast<const T*>(p.in[0]), static_cast<const T*>(p.in[1]), static_cast<const T*>(p.in[2]),
                      static_cast<const T*>(p.in[3])};
  const float2* ckpt = reinterpret_cast<const float2*>(p.ckpt);
  const bool want_rec = p.out[2] != nullptr;
  const bool residual = (p.flags & F_RESIDUAL) != 0;
  const bool tape = (p.flags & F_TAPE) != 0;  // the last stage's output state comes from its checkpoint
  const long long BN = p.B * (long long)N;
  const uint32_t n_ck = p.n_ckpt_slots;

  if (tid == 0) {
    mbar_init(&bar[0], 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  fill_stage_table(recs, p.W, p.oma, p.l0, p.m, p.L, p.ckpt_every, p.flags, ckpt != nullptr, tid, nthr);
  for (int i = tid; i < 2 * L * nwarp; i += nthr) red[i] = 0.0f;
  __syncthreads();

  auto issue_load = [&](long long tl) {
    const long long row0 = tl * R;
    const int rows = (int)min((long long)R, p.B - row0);
    const uint32_t bytes = (uint32_t)(rows * N * sizeof(T));
    const uint32_t cbytes = (uint32_t)(rows * N * sizeof(float2));
    mbar_expect_tx(&bar[0], (tape ? 2 : 4) * bytes + n_ck * cbytes + (residual ? bytes : 0));
#pragma unroll
    for (int q = 0; q < 4; ++q)
      if (q >= 2 || !tape) bulk_g2s(win + q * RN, g_in[q] + row0 * N, bytes, &bar[0]);
    for (uint32_t k = 0; k < n_ck; ++k)
      bulk_g2s(const_cast<float2*>(sck) + k * RN, ckpt + (long long)k * BN + row0 * N, cbytes, &bar[0]);
    if (residual) bulk_g2s(sdy, g_in[2] + row0 * N, bytes, &bar[0]);
  };

  const int r = tid / TPR, t = tid - r * TPR;
  const int wpr = TPR >> 5, wr = t >> 5;
  LaneHalo halo;
  halo.base = smem_u32(smem + p.off_halo);
  halo.warp_bytes = p.halo_warp_bytes;
  halo.buf_bytes = p.halo_warp_bytes * (uint32_t)(nthr >> 5);
  halo.warp = warp;
  halo.warp_up = r * wpr + (wr + 1 == wpr ? 0 : wr + 1);
  halo.warp_dn = r * wpr + (wr == 0 ? wpr - 1 : wr - 1);
  halo.parity = 0;
  const uint32_t xrow = smem_u32(smem + p.off_work) + (uint32_t)r * (uint32_t)(4 * N) * 4u;  // fp32 [4][NG][m] per row
  const int chunk = r * N + t * (G * NG);
  constexpr float sT = (float)F::sT;
  PairWB w;
  w.alpha = f2(p.alpha);
  w.oma = f2(p.oma);
  const float dsi = lane_dw_scale_i<ACT>(p.oma), dsj = lane_dw_scale_j<ACT>(p.oma);
  uint32_t phase = 0;

  for (long long tile = blockIdx.x; tile < p.tiles; tile += gridDim.x) {
    if (tid == 0) {
      bulk_wait_read0();  // the previous tile's stores have left the buffer
      issue_load(tile);
    }
    if (!mbar_wait_bounded(&bar[0], phase)) *abort_flag = 1;
    phase ^= 1;
    __syncthreads();
    if (*abort_flag) break;

    const long long row0 = tile * R;
    const int rows = (int)min((long long)R, p.B - row0);
    const bool active = r < rows;

    float2 V[4][G / 2][NG];  // x, xa, gx, ga
#pragma unroll
    for (int s = 0; s < 4; ++s)
#pragma unroll
      for (int pp = 0; pp < G / 2; ++pp)
#pragma unroll
        for (int o = 0; o < NG; ++o) V[s][pp][o] = f2(0.0f);
    if (active) {
      if (!tape) {
        lane_ld_native<NG, G, T>(win + chunk, V[0], t);
        lane_ld_native<NG, G, T>(win + RN + chunk, V[1], t);
      }
      lane_ld_native<NG, G, T>(win + 2 * RN + chunk, V[2], t);
      lane_ld_native<NG, G, T>(win + 3 * RN + chunk, V[3], t);
    }
    __syncthreads();  // native inputs are in registers; the buffer is free for long shifts
    if (tid == 0 && tile + gridDim.x < p.tiles) {  // next tile towards L2 while this one is worked on
      const long long nrow0 = (tile + gridDim.x) * R;
      const int nrows = (int)min((long long)R, p.B - nrow0);
      const uint32_t bytes = (uint32_t)(nrows * N * sizeof(T));
#pragma unroll
      for (int q = 0; q < 4; ++q)
        if (q >= 2 || !tape) l2_prefetch(g_in[q] + nrow0 * N, bytes);
      for (uint32_t k = 0; k < n_ck; ++k) l2_prefetch(ckpt + (long long)k * BN + nrow0 * N, (uint32_t)(nrows * N * sizeof(float2)));
    }

    int s_cur = 0;
    StageRec rec_next = recs[L - 1];
    for (int l = L - 1; l >= 0; --l) {
      const StageRec rec = rec_next;
      if (l > 0) rec_next = recs[l - 1];
      lane_exchange<NG, G, 4>(V, rec.s - s_cur, p.ea_max, halo, lane, xrow, t, m);
      s_cur = rec.s;
      w.owi = f2(rec.owi);
      w.owj = f2(rec.owj);
      w.owjs = f2(rec.owj * sT);
      if (rec.ck >= 0) {  // a state saved after stage l replaces the rebuilt one
        const float2* c = sck + rec.ck * RN + r * N + (G / 2) * t;
#pragma unroll
        for (int s = 0; s < 2; ++s)
#pragma unroll
          for (int o = 0; o < NG; ++o)
#pragma unroll
            for (int pp = 0; pp < G / 2; ++pp) V[s][pp][o] = c[(s * NG + o) * (m >> 1) + pp];
      }
      float2 dwi = f2(0.0f), dwj = f2(0.0f);
#pragma unroll
      for (int pp = 0; pp < G / 2; ++pp) lane_backward<NG, ACT>(V[0][pp], V[1][pp], V[2][pp], V[3][pp], w, dwi, dwj);
      // ---- weight-gradient partial of this stage: fixed-order warp tree, one slot per warp
      {
        const float di = (dwi.x + dwi.y) * dsi, dj = (dwj.x + dwj.y) * dsj;
        const bool hi = (lane & 16) != 0;
        const float give = hi ? di : dj;
        float keep = hi ? dj : di;
        keep += __shfl_xor_sync(0xffffffffu, give, 16);
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) keep += __shfl_xor_sync(0xffffffffu, keep, o);
        if ((lane & 15) == 0 && active) red[(l * nwarp + warp) * 2 + (hi ? 1 : 0)] += keep;
      }
    }
    lane_exchange<NG, G, 4>(V, -s_cur, p.ea_max, halo, lane, xrow, t, m);  // back to stride 0 = native order
    if (active) {
      if (residual) {
        float2 gin[G / 2][NG];
        lane_ld_native<NG, G, T>(sdy + chunk, gin, t);
#pragma unroll
        for (int pp = 0; pp < G / 2; ++pp)
#pragma unroll
          for (int o = 0; o < NG; ++o) V[2][pp][o] = fadd2(V[2][pp][o], gin[pp][o]);
      }
      lane_st_native<NG, G, T>(win + chunk, V[2], t);
      lane_st_native<NG, G, T>(win + RN + chunk, V[3], t);
      if (want_rec) {
        lane_st_native<NG, G, T>(win + 2 * RN + chunk, V[0], t);
        lane_st_native<NG, G, T>(win + 3 * RN + chunk, V[1], t);
      }
    }
    fence_proxy_async();
    __syncthreads();
    if (tid == 0) {
      const uint32_t bytes = (uint32_t)(rows * N * sizeof(T));
      bulk_s2g(static_cast<T*>(p.out[0]) + row0 * N, win, bytes);
      bulk_s2g(static_cast<T*>(p.out[1]) + row0 * N, win + RN, bytes);
      if (want_rec) {
        bulk_s2g(static_cast<T*>(p.out[2]) + row0 * N, win + 2 * RN, bytes);
        bulk_s2g(static_cast<T*>(p.out[3]) + row0 * N, win + 3 * RN, bytes);
      }
      bulk_commit();
    }
  }
  // ---- per-CTA partial: sum the warp slots in warp order
  __syncthreads();
  for (int i = tid; i < 2 * L; i += nthr) {
    const int l = i >> 1, c = i & 1;
    float acc = 0.0f;
    for (int w2 = 0; w2 < nwarp; ++w2) acc += red[(l * nwarp + w2) * 2 + c];
    p.partials[(long long)blockIdx.x * 2 * L + i] = acc;
  }
  if (tid == 0) {
    bulk_wait_all0();
    if (*abort_flag) atomicExch(p.status, DEV_WAIT_TIMEOUT);
  }
}

}  // namespace ncn
