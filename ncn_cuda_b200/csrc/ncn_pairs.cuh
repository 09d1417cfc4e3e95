// Fast path of the fused row kernels: one thread owns TWO groups of a row, g and g + m/2, for the
// whole tile, and every arithmetic instruction is a packed fp32 pair (fma.rn.f32x2 & co.) whose
// two lanes are the two groups.  Compared with ncn_rows.cuh (any m, any number of groups per
// thread) this halves the issue slots of the per-step scalar work as well (xj, P, Q, the
// weight-gradient sums are per-group values, so they pack too), and the packed accumulators need
// no horizontal adds.  Requires m even and one pair per thread per tile (R * m/2 <= blockDim.x).
//
// Shared-memory layouts are those of ncn_rows.cuh: native in/out buffers moved by TMA bulk
// copies, stage-local slots o*m + blk in between, rewritten in place by the thread that read them.
#pragma once
#include "ncn_rows.cuh"

#ifndef NCN_FWD_NEWTON_EVERY
#define NCN_FWD_NEWTON_EVERY 2
#endif

namespace ncn {

__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ float2 fmul2(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float2 fadd2(float2 a, float2 b) { return __fadd2_rn(a, b); }

// per-stage weights, one lane per group (both lanes equal), pre-scaled
struct PairW {
  float2 owi, owj, alpha;  // forward: sT (1-alpha) wi, sT (1-alpha) wj, sT alpha
};

// Forward steps in the scaled variables of ncn_common.cuh; X[i], A[i] = member i of (group a, group b).
template <int NG, int ACT, int J>
struct PFwdSteps {
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
#pragma unroll
    for (int i = 0; i < NG; ++i) {
      float2 r;
      if constexpr (ACT == ACT_TANH && NCN_FWD_NEWTON_EVERY > 0) {
        // the forward is bound by the special-function unit while the FMA pipe idles: one position
        // in NCN_FWD_NEWTON_EVERY takes its reciprocal there
        if ((i % NCN_FWD_NEWTON_EVERY) == NCN_FWD_NEWTON_EVERY - 1) r = F::r_fma(ffma2(X[i], P, Q)); else r = F::r(ffma2(X[i], P, Q));
      } else {
        r = F::r(ffma2(X[i], P, Q));
      }
      A[i] = ffma2(r, f2(cA), A[i]);
      X[i] = ffma2(A[i], f2(kC), X[i]);
    }
    PFwdSteps<NG, ACT, J + 1>::run(X, A, w);
  }
};
template <int NG, int ACT>
struct PFwdSteps<NG, ACT, NG> {
  static __device__ __forceinline__ void run(float2 (&)[NG], float2 (&)[NG], const PairW&) {}
};

template <int NG, int ACT>
__device__ __forceinline__ void pair_forward(float2 (&X)[NG], float2 (&A)[NG], const PairW& w) {
  using F = ActForm<ACT>;
  PFwdSteps<NG, ACT, 0>::run(X, A, w);
  constexpr float mN = (float)cpow(kMd, NG);
  constexpr float mNC = (float)(cpow(kMd, NG) * fwd_C(NG, F::f0));
  constexpr float mND = (float)(cpow(kMd, NG) * fwd_D(NG, F::f0));
#pragma unroll
  for (int i = 0; i < NG; ++i) {
    if constexpr (mND != 0.0f) X[i] = ffma2(X[i], f2(mN), f2(mND)); else X[i] = fmul2(X[i], f2(mN));
    if constexpr (mNC != 0.0f) A[i] = ffma2(A[i], f2(mN), f2(mNC)); else A[i] = fmul2(A[i], f2(mN));
  }
}

// Reverse sweep, same scaled variables as BwdSteps (ncn_common.cuh), two groups per instruction.
struct PairWB {
  float2 owi, owj, owjs, alpha, oma;  // (1-alpha) wi, (1-alpha) wj, sT (1-alpha) wj, alpha, 1-alpha
};
template <int NG, int ACT, int J>
struct PBwdSteps {
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
    constexpr float cdsmk = (float)(kCd * F::ds * mkd);
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
    float2 aI = f2(0.0f), aS = f2(0.0f);
#pragma unroll
    for (int i = 0; i < NG; ++i) {
      const float2 ts = ffma2(X[i], Ps, Qs);
      const float2 r = F::r(ts);
      A[i] = ffma2(r, f2(cAr), A[i]);
      G[i] = ffma2(f2(kC), H[i], G[i]);
      const float2 gt = F::gt(G[i], ts, r);
      H[i] = ffma2(gt, PH, H[i]);
      aI = ffma2(gt, X[i], aI);
      aS = fadd2(aS, gt);
    }
    float2 tI;
    if constexpr (DX1 != 0.0f) tI = fmul2(ffma2(f2(DX1), aS, aI), f2(cdsm)); else tI = fmul2(aI, f2(cdsm));
    const float2 tS = fmul2(aS, f2(cdsmk));
    // gx_j += (1-alpha) (wi sum gT x + 2 wj xj sum gT), in units of m^(k+1)
    const float2 wx = fmul2(fmul2(w.owj, xj), tS);
    const float2 add = ffma2(w.owi, tI, fadd2(wx, wx));
    H[J] = ffma2(add, f2(imk1), H[J]);
    const float2 oxj = fmul2(w.oma, xj);
    dwi = ffma2(oxj, tI, dwi);
    dwj = ffma2(fmul2(oxj, xj), tS, dwj);
    PBwdSteps<NG, ACT, J - 1>::run(X, A, H, G, w, dwi, dwj);
  }
};
template <int NG, int ACT>
struct PBwdSteps<NG, ACT, -1> {
  static __device__ __forceinline__ void run(float2 (&)[NG], float2 (&)[NG], float2 (&)[NG], float2 (&)[NG],
                                             const PairWB&, float2&, float2&) {}
};

template <int NG, int ACT>
__device__ __forceinline__ void pair_backward(float2 (&X)[NG], float2 (&A)[NG], float2 (&H)[NG], float2 (&G)[NG],
                                              const PairWB& w, float2& dwi, float2& dwj) {
  using F = ActForm<ACT>;
  PBwdSteps<NG, ACT, NG - 1>::run(X, A, H, G, w, dwi, dwj);
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

// slot addresses of the pair: group a = t, group b = t + m/2 (always half a row apart)
template <int NG, int SHIFT>
__device__ __forceinline__ void pair_addrs(uint32_t row_addr, int t, int s, int m, uint32_t (&aa)[NG], uint32_t (&ab)[NG]) {
  int blk = t;
  uint32_t ro = row_addr;
  const uint32_t mstep = (uint32_t)m << SHIFT;
  const int mh = m >> 1;
  const uint32_t hstep = (uint32_t)mh << SHIFT;
#pragma unroll
  for (int o = 0; o < NG; ++o) {
    aa[o] = ro + ((uint32_t)blk << SHIFT);
    ab[o] = blk < mh ? aa[o] + hstep : aa[o] - hstep;
    ro += mstep;
    blk = wrap_add(blk, s, m);
  }
}

template <int NG, typename T>
__device__ __forceinline__ void ld_native_pair(const T* row, int t, int s, int m, float2 (&v)[NG]) {
  float va[NG], vb[NG];
  ld_native<NG, T>(row, t, s, m, va);
  ld_native<NG, T>(row, t + (m >> 1), s, m, vb);
#pragma unroll
  for (int o = 0; o < NG; ++o) v[o] = make_float2(va[o], vb[o]);
}
template <int NG, typename T>
__device__ __forceinline__ void st_native_pair(T* row, int t, int s, int m, const float2 (&v)[NG]) {
  float va[NG], vb[NG];
#pragma unroll
  for (int o = 0; o < NG; ++o) { va[o] = v[o].x; vb[o] = v[o].y; }
  st_native<NG, T>(row, t, s, m, va);
  st_native<NG, T>(row, t + (m >> 1), s, m, vb);
}

// ------------------------------------------------------------------------------------------ forward
template <int NG, int ACT, typename T, int MAXT, int MINB>
__global__ void __launch_bounds__(MAXT, MINB) pair_fwd_kernel(const RowsParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  using F = ActForm<ACT>;
  const int tid = threadIdx.x;
  const int N = p.N, m = p.m, R = p.R, L = p.L;
  const int mh = m >> 1;
  const int RN = R * N;
  T* in_x[2] = {reinterpret_cast<T*>(smem + p.off_in[0]), reinterpret_cast<T*>(smem + p.off_in[1])};
  const uint32_t work_addr = smem_u32(smem + p.off_work);  // (x, a) per 8-byte slot
  T* ox = reinterpret_cast<T*>(smem + p.off_out);
  T* oa = ox + RN;
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
    mbar_init(&bar[1], 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  fill_stage_table(recs, p, ckpt != nullptr, tid, blockDim.x);
  __syncthreads();

  auto issue_load = [&](long long tl, int b) {
    const long long row0 = tl * R;
    const int rows = (int)min((long long)R, p.B - row0);
    const uint32_t bytes = (uint32_t)(rows * N * sizeof(T));
    mbar_expect_tx(&bar[b], 2 * bytes);
    bulk_g2s(in_x[b], gx_in + row0 * N, bytes, &bar[b]);
    bulk_g2s(in_x[b] + RN, ga_in + row0 * N, bytes, &bar[b]);
  };

  long long tile = blockIdx.x;
  if (tid == 0 && tile < p.tiles) issue_load(tile, 0);
  uint32_t phase0 = 0, phase1 = 0;
  int buf = 0;
  const int r = tid / mh, t = tid - r * mh;  // this thread's row of the tile and pair index
  const int base = r * N;
  const uint32_t wrow = work_addr + ((uint32_t)base << 3);
  constexpr float sT = (float)F::sT;
  PairW w;
  w.alpha = f2(p.alpha * sT);

  for (; tile < p.tiles; tile += gridDim.x) {
    const long long next = tile + gridDim.x;
    if (p.nbuf == 2 && tid == 0 && next < p.tiles) issue_load(next, buf ^ 1);
    const uint32_t ph = buf ? phase1 : phase0;
    if (!mbar_wait_bounded(&bar[buf], ph)) *abort_flag = 1;
    if (buf) phase1 ^= 1; else phase0 ^= 1;
    if (L == 1 && tid == 0) bulk_wait_read0();
    __syncthreads();
    if (*abort_flag) break;

    const long long row0 = tile * R;
    const int rows = (int)min((long long)R, p.B - row0);
    const bool active = r < rows;
    const T* sx = in_x[buf] + base;
    const T* sa = sx + RN;
    float2* ck_tile = ckpt + row0 * N + base;

    StageRec rec_next = recs[0];
    for (int l = 0; l < L; ++l) {
      const StageRec rec = rec_next;
      if (l + 1 < L) rec_next = recs[l + 1];  // in flight during this stage's work
      const int s = rec.s;
      const bool first = (l == 0), last = (l == L - 1);
      if (active) {
        float2 X[NG], A[NG];
        uint32_t aa[NG], ab[NG];
        w.owi = f2(rec.owi * sT);
        w.owj = f2(rec.owj * sT);
        if (first) {
          ld_native_pair<NG, T>(sx, t, s, m, X);
          ld_native_pair<NG, T>(sa, t, s, m, A);
        } else {
          pair_addrs<NG, 3>(wrow, t, s, m, aa, ab);
#pragma unroll
          for (int o = 0; o < NG; ++o) {
            const float2 va = lds64(aa[o]);
            const float2 vb = lds64(ab[o]);
            X[o] = make_float2(va.x, vb.x);
            A[o] = make_float2(va.y, vb.y);
          }
        }
        pair_forward<NG, ACT>(X, A, w);
        if (rec.ck >= 0) {  // filed under this stage's groups: the backward of this stage reads o*m + g
          float2* ck = ck_tile + (long long)rec.ck * BN + t;
#pragma unroll
          for (int o = 0; o < NG; ++o) {
            ck[o * m] = make_float2(X[o].x, A[o].x);
            ck[o * m + mh] = make_float2(X[o].y, A[o].y);
          }
        }
        if (last) {
          if (residual) {
            float2 xin[NG];
            ld_native_pair<NG, T>(sx, t, s, m, xin);
#pragma unroll
            for (int o = 0; o < NG; ++o) X[o] = fadd2(X[o], xin[o]);
          }
          st_native_pair<NG, T>(ox + base, t, s, m, X);
          st_native_pair<NG, T>(oa + base, t, s, m, A);
        } else {
          if (first) pair_addrs<NG, 3>(wrow, t, s, m, aa, ab);
#pragma unroll
          for (int o = 0; o < NG; ++o) {
            sts64(aa[o], X[o].x, A[o].x);
            sts64(ab[o], X[o].y, A[o].y);
          }
        }
      }
      if (L > 1 && l == L - 2 && tid == 0) bulk_wait_read0();
      if (last) fence_proxy_async();
      __syncthreads();
      if (p.nbuf == 1 && tid == 0 && next < p.tiles && (residual ? last : first)) issue_load(next, 0);
    }
    if (tid == 0) {
      const uint32_t bytes = (uint32_t)(rows * N * sizeof(T));
      bulk_s2g(gy_out + row0 * N, ox, bytes);
      bulk_s2g(gya_out + row0 * N, oa, bytes);
      bulk_commit();
    }
    if (p.nbuf == 2) buf ^= 1;
  }
  if (tid == 0) {
    bulk_wait_all0();
    if (*abort_flag) atomicExch(p.status, DEV_WAIT_TIMEOUT);
  }
}

// ------------------------------------------------------------------------------------------
// Forward with ONE tile buffer and two pairs per thread: the TMA loads land in the buffer in native
// layout, the stage-local (x, a) slots overwrite it in place and the native results are staged in
// it for the TMA stores ("all threads read, barrier, all threads write" at the two changes of
// layout; a thread's two pairs fit in registers across the barrier).  A tile then costs 8 bytes
// per position, so four CTAs of half the threads fit one SM: four independent barrier domains
// whose stage boundaries and copies overlap each other's arithmetic.  With F_RESIDUAL a second
// native copy of x is kept for the final add.
template <int NG, int ACT, typename T, int MAXT, int MINB, int PPT = 2>
__global__ void __launch_bounds__(MAXT, MINB) pair_fwd_dual_kernel(const RowsParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  using F = ActForm<ACT>;
  const int tid = threadIdx.x, nthr = blockDim.x;
  const int N = p.N, m = p.m, R = p.R, L = p.L;
  const int mh = m >> 1;
  const int RN = R * N;
  T* win = reinterpret_cast<T*>(smem + p.off_work);  // native x at win, xa at win + RN
  const uint32_t work_addr = smem_u32(smem + p.off_work);
  T* sres = reinterpret_cast<T*>(smem + p.off_in[0]);  // F_RESIDUAL: native x of the tile
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
  fill_stage_table(recs, p, ckpt != nullptr, tid, nthr);
  __syncthreads();

  auto issue_load = [&](long long tl) {
    const long long row0 = tl * R;
    const int rows = (int)min((long long)R, p.B - row0);
    const uint32_t bytes = (uint32_t)(rows * N * sizeof(T));
    mbar_expect_tx(&bar[0], (residual ? 3 : 2) * bytes);
    bulk_g2s(win, gx_in + row0 * N, bytes, &bar[0]);
    bulk_g2s(win + RN, ga_in + row0 * N, bytes, &bar[0]);
    if (residual) bulk_g2s(sres, gx_in + row0 * N, bytes, &bar[0]);
  };

  uint32_t phase = 0;
  int rr[PPT], tt[PPT], base[PPT];
  uint32_t wrow[PPT];
#pragma unroll
  for (int pp = 0; pp < PPT; ++pp) {
    const int item = tid + pp * nthr;
    rr[pp] = item / mh;
    tt[pp] = item - rr[pp] * mh;
    base[pp] = rr[pp] * N;
    wrow[pp] = work_addr + ((uint32_t)base[pp] << 3);
  }
  constexpr float sT = (float)F::sT;
  PairW w;
  w.alpha = f2(p.alpha * sT);

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
    bool active[PPT];
#pragma unroll
    for (int pp = 0; pp < PPT; ++pp) active[pp] = rr[pp] < rows;

    float2 X[PPT][NG], A[PPT][NG];
    uint32_t aa[NG], ab[NG];

    StageRec rec_next = recs[0];
    for (int l = 0; l < L; ++l) {
      const StageRec rec = rec_next;
      if (l + 1 < L) rec_next = recs[l + 1];
      const int s = rec.s;
      const bool first = (l == 0), last = (l == L - 1);
      w.owi = f2(rec.owi * sT);
      w.owj = f2(rec.owj * sT);
      if (first) {
#pragma unroll
        for (int pp = 0; pp < PPT; ++pp)
          if (active[pp]) {
            ld_native_pair<NG, T>(win + base[pp], tt[pp], s, m, X[pp]);
            ld_native_pair<NG, T>(win + RN + base[pp], tt[pp], s, m, A[pp]);
          }
        __syncthreads();  // native inputs are in registers; the buffer may now take slots
      }
#pragma unroll
      for (int pp = 0; pp < PPT; ++pp) {
        if (active[pp]) {
          pair_addrs<NG, 3>(wrow[pp], tt[pp], s, m, aa, ab);
          if (!first) {
#pragma unroll
            for (int o = 0; o < NG; ++o) {
              const float2 va = lds64(aa[o]);
              const float2 vb = lds64(ab[o]);
              X[pp][o] = make_float2(va.x, vb.x);
              A[pp][o] = make_float2(va.y, vb.y);
            }
          }
          pair_forward<NG, ACT>(X[pp], A[pp], w);
          if (rec.ck >= 0) {  // filed under this stage's groups: the backward of this stage reads o*m + g
            float2* ck = ckpt + row0 * N + base[pp] + (long long)rec.ck * BN + tt[pp];
#pragma unroll
            for (int o = 0; o < NG; ++o) {
              ck[o * m] = make_float2(X[pp][o].x, A[pp][o].x);
              ck[o * m + mh] = make_float2(X[pp][o].y, A[pp][o].y);
            }
          }
          if (!last) {
#pragma unroll
            for (int o = 0; o < NG; ++o) {
              sts64(aa[o], X[pp][o].x, A[pp][o].x);
              sts64(ab[o], X[pp][o].y, A[pp][o].y);
            }
          }
        }
      }
      if (last) {
        __syncthreads();  // every slot has been read; the buffer may now take the native results
#pragma unroll
        for (int pp = 0; pp < PPT; ++pp)
          if (active[pp]) {
            if (residual) {
              float2 xin[NG];
              ld_native_pair<NG, T>(sres + base[pp], tt[pp], s, m, xin);
#pragma unroll
              for (int o = 0; o < NG; ++o) X[pp][o] = fadd2(X[pp][o], xin[o]);
            }
            st_native_pair<NG, T>(win + base[pp], tt[pp], s, m, X[pp]);
            st_native_pair<NG, T>(win + RN + base[pp], tt[pp], s, m, A[pp]);
          }
        fence_proxy_async();
      }
      __syncthreads();
    }
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
// Shared memory per tile is cut to the minimum so that two CTAs fit one SM (their barriers are
// independent, so one CTA computes while the other is in a stage boundary or waiting for copies):
//   W   R*N 16-byte slots.  The TMA loads land here in native layout (4 streams), the stage-local
//       slots (x, a, gx, ga) overwrite them in place, and the native results are staged here for
//       the TMA stores.  Every change of layout is "all threads read, barrier, all threads write";
//       a thread holds exactly one pair, so its whole share fits in registers across the barrier.
//   CK  the tile's checkpoints (8-byte slots); with F_RESIDUAL it keeps the native dy instead.
// Modes are those of rows_bwd_kernel (ncn_rows.cuh).
template <int NG, int ACT, typename T, int MAXT, int MINB>
__global__ void __launch_bounds__(MAXT, MINB) pair_bwd_kernel(const RowsParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  using F = ActForm<ACT>;
  const int tid = threadIdx.x, nthr = blockDim.x;
  const int lane = tid & 31, warp = tid >> 5, nwarp = (nthr + 31) >> 5;
  const int N = p.N, m = p.m, R = p.R, L = p.L;
  const int mh = m >> 1;
  const int RN = R * N;
  T* win = reinterpret_cast<T*>(smem + p.off_work);  // native streams q at win + q*RN
  const uint32_t work_addr = smem_u32(smem + p.off_work);
  float2* sck = reinterpret_cast<float2*>(smem + p.off_ckpt);
  T* sdy = reinterpret_cast<T*>(smem + p.off_ckpt);  // F_RESIDUAL: native dy of the tile
  float* red = reinterpret_cast<float*>(smem + p.off_red);  // [L][nwarp][2]
  StageRec* recs = reinterpret_cast<StageRec*>(smem + p.off_w);
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem + p.off_bar);
  int* abort_flag = reinterpret_cast<int*>(bar + 2);
  const T* g_in[4] = {static_cast<const T*>(p.in[0]), static_cast<const T*>(p.in[1]), static_cast<const T*>(p.in[2]),
                      static_cast<const T*>(p.in[3])};
  const float2* ckpt = reinterpret_cast<const float2*>(p.ckpt);
  const bool residual = (p.flags & F_RESIDUAL) != 0;
  const bool recompute = (p.flags & F_RECOMPUTE) != 0;
  const bool want_rec = p.out[2] != nullptr;
  const long long BN = p.B * (long long)N;
  const uint32_t n_ck = p.n_ckpt_slots;

  if (tid == 0) {
    mbar_init(&bar[0], 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  fill_stage_table(recs, p, ckpt != nullptr && !recompute, tid, nthr);
  for (int i = tid; i < 2 * L * nwarp; i += nthr) red[i] = 0.0f;
  __syncthreads();

  auto issue_load = [&](long long tl) {
    const long long row0 = tl * R;
    const int rows = (int)min((long long)R, p.B - row0);
    const uint32_t bytes = (uint32_t)(rows * N * sizeof(T));
    const uint32_t cbytes = (uint32_t)(rows * N * sizeof(float2));
    mbar_expect_tx(&bar[0], 4 * bytes + n_ck * cbytes + (residual ? bytes : 0));
#pragma unroll
    for (int q = 0; q < 4; ++q) bulk_g2s(win + q * RN, g_in[q] + row0 * N, bytes, &bar[0]);
    for (uint32_t k = 0; k < n_ck; ++k) bulk_g2s(sck + k * RN, ckpt + (long long)k * BN + row0 * N, cbytes, &bar[0]);
    if (residual) bulk_g2s(sdy, g_in[2] + row0 * N, bytes, &bar[0]);
  };

  uint32_t phase = 0;
  const int r = tid / mh, t = tid - r * mh;
  const int base = r * N;
  const uint32_t wrow = work_addr + ((uint32_t)base << 4);
  constexpr float sT = (float)F::sT;
  PairWB w;
  w.alpha = f2(p.alpha);
  w.oma = f2(p.oma);
  PairW wf;
  wf.alpha = f2(p.alpha * sT);

  for (long long tile = blockIdx.x; tile < p.tiles; tile += gridDim.x) {
    if (tid == 0) {
      bulk_wait_read0();  // the previous tile's stores have left W
      issue_load(tile);
    }
    if (!mbar_wait_bounded(&bar[0], phase)) *abort_flag = 1;
    phase ^= 1;
    __syncthreads();
    if (*abort_flag) break;

    const long long row0 = tile * R;
    const int rows = (int)min((long long)R, p.B - row0);
    const bool active = r < rows;
    const T* s0 = win + base;

    float2 X[NG], A[NG], H[NG], G[NG];
    uint32_t aa[NG], ab[NG];

    // ---- optional forward replay: net input (native) -> net output (slots .xy); dy, dya move to .zw
    if (recompute) {
      for (int l = 0; l < L; ++l) {
        const StageRec rec = recs[l];
        const int s = rec.s;
        wf.owi = f2(rec.owi * sT);
        wf.owj = f2(rec.owj * sT);
        if (active) pair_addrs<NG, 4>(wrow, t, s, m, aa, ab);
        if (l == 0) {
          if (active) {
            ld_native_pair<NG, T>(s0, t, s, m, X);
            ld_native_pair<NG, T>(s0 + RN, t, s, m, A);
            ld_native_pair<NG, T>(s0 + 2 * RN, t, s, m, H);
            ld_native_pair<NG, T>(s0 + 3 * RN, t, s, m, G);
          }
          __syncthreads();  // every native value is in registers; W may now take slots
        } else if (active) {
#pragma unroll
          for (int o = 0; o < NG; ++o) {
            const float2 va = lds64(aa[o]), vb = lds64(ab[o]);
            X[o] = make_float2(va.x, vb.x);
            A[o] = make_float2(va.y, vb.y);
          }
        }
        if (active) {
          pair_forward<NG, ACT>(X, A, wf);
          if (l == 0) {
#pragma unroll
            for (int o = 0; o < NG; ++o) {
              sts128(aa[o], X[o].x, A[o].x, H[o].x, G[o].x);
              sts128(ab[o], X[o].y, A[o].y, H[o].y, G[o].y);
            }
          } else {
#pragma unroll
            for (int o = 0; o < NG; ++o) {
              sts64(aa[o], X[o].x, A[o].x);
              sts64(ab[o], X[o].y, A[o].y);
            }
          }
        }
        __syncthreads();
      }
    }

    // ---- reverse sweep over the stages
    for (int l = L - 1; l >= 0; --l) {
      const StageRec rec = recs[l];
      const int s = rec.s;
      const bool first = (l == L - 1), last = (l == 0);
      w.owi = f2(rec.owi);
      w.owj = f2(rec.owj);
      w.owjs = f2(rec.owj * sT);
      float2 dwi = f2(0.0f), dwj = f2(0.0f);
      const bool from_native = first && !recompute;

      if (active) {
        pair_addrs<NG, 4>(wrow, t, s, m, aa, ab);
        if (from_native) {
          ld_native_pair<NG, T>(s0, t, s, m, X);
          ld_native_pair<NG, T>(s0 + RN, t, s, m, A);
          ld_native_pair<NG, T>(s0 + 2 * RN, t, s, m, H);
          ld_native_pair<NG, T>(s0 + 3 * RN, t, s, m, G);
        } else {
#pragma unroll
          for (int o = 0; o < NG; ++o) {
            const float4 va = lds128(aa[o]), vb = lds128(ab[o]);
            X[o] = make_float2(va.x, vb.x);
            A[o] = make_float2(va.y, vb.y);
            H[o] = make_float2(va.z, vb.z);
            G[o] = make_float2(va.w, vb.w);
          }
          if (rec.ck >= 0) {  // a state saved after stage l replaces the rebuilt one
            const float2* c = sck + rec.ck * RN + base + t;
#pragma unroll
            for (int o = 0; o < NG; ++o) {
              const float2 va = c[o * m], vb = c[o * m + mh];
              X[o] = make_float2(va.x, vb.x);
              A[o] = make_float2(va.y, vb.y);
            }
          }
        }
      }
      if (from_native) __syncthreads();  // native inputs are in registers; W may now take slots

      if (active) pair_backward<NG, ACT>(X, A, H, G, w, dwi, dwj);

      if (last) {
        __syncthreads();  // every slot has been read; W may now take the native results
        if (active) {
          if (residual) {
            float2 gin[NG];
            ld_native_pair<NG, T>(sdy + base, t, s, m, gin);
#pragma unroll
            for (int o = 0; o < NG; ++o) H[o] = fadd2(H[o], gin[o]);
          }
          T* wout = win + base;
          st_native_pair<NG, T>(wout, t, s, m, H);
          st_native_pair<NG, T>(wout + RN, t, s, m, G);
          if (want_rec) {
            st_native_pair<NG, T>(wout + 2 * RN, t, s, m, X);
            st_native_pair<NG, T>(wout + 3 * RN, t, s, m, A);
          }
        }
      } else if (active) {
#pragma unroll
        for (int o = 0; o < NG; ++o) {
          sts128(aa[o], X[o].x, A[o].x, H[o].x, G[o].x);
          sts128(ab[o], X[o].y, A[o].y, H[o].y, G[o].y);
        }
      }
      // ---- weight-gradient partial of this stage: fixed-order warp tree, one slot per warp
      {
        const float di = dwi.x + dwi.y, dj = dwj.x + dwj.y;
        const bool hi = (lane & 16) != 0;
        const float give = hi ? di : dj;
        float keep = hi ? dj : di;
        keep += __shfl_xor_sync(0xffffffffu, give, 16);
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) keep += __shfl_xor_sync(0xffffffffu, keep, o);
        if ((lane & 15) == 0) red[(l * nwarp + warp) * 2 + (hi ? 1 : 0)] += keep;
      }
      if (last) fence_proxy_async();
      __syncthreads();
    }
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

// ------------------------------------------------------------------------------------------
// Backward, aliased tile buffer with TWO pairs per thread: half the threads of pair_bwd_kernel for
// the same tile, so that two CTAs fit one SM with a full register budget (no spills) and one
// CTA's stage barriers overlap the other's arithmetic.  Backward from the net output or (F_TAPE) from
// the stored end state, checkpoints and F_RESIDUAL allowed; no forward replay.
template <int NG, int ACT, typename T, int MAXT>
__global__ void __launch_bounds__(MAXT, 2) pair_bwd_dual_kernel(const RowsParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  using F = ActForm<ACT>;
  constexpr int PPT = 2;
  const int tid = threadIdx.x, nthr = blockDim.x;
  const int lane = tid & 31, warp = tid >> 5, nwarp = (nthr + 31) >> 5;
  const int N = p.N, m = p.m, R = p.R, L = p.L;
  const int mh = m >> 1;
  const int RN = R * N;
  T* win = reinterpret_cast<T*>(smem + p.off_work);  // native streams q at win + q*RN
  const uint32_t work_addr = smem_u32(smem + p.off_work);
  float2* sck = reinterpret_cast<float2*>(smem + p.off_ckpt);
  float* red = reinterpret_cast<float*>(smem + p.off_red);  // [L][nwarp][2]
  StageRec* recs = reinterpret_cast<StageRec*>(smem + p.off_w);
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem + p.off_bar);
  int* abort_flag = reinterpret_cast<int*>(bar + 2);
  const T* g_in[4] = {static_cast<const T*>(p.in[0]), static_cast<const T*>(p.in[1]), static_cast<const T*>(p.in[2]),
                      static_cast<const T*>(p.in[3])};
  const float2* ckpt = reinterpret_cast<const float2*>(p.ckpt);
  T* sdy = reinterpret_cast<T*>(smem + p.off_in[0]);  // F_RESIDUAL: native dy of the tile
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
  fill_stage_table(recs, p, ckpt != nullptr, tid, nthr);
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
    for (uint32_t k = 0; k < n_ck; ++k) bulk_g2s(sck + k * RN, ckpt + (long long)k * BN + row0 * N, cbytes, &bar[0]);
    if (residual) bulk_g2s(sdy, g_in[2] + row0 * N, bytes, &bar[0]);
  };

  uint32_t phase = 0;
  int rr[PPT], tt[PPT], base[PPT];
  uint32_t wrow[PPT];
#pragma unroll
  for (int pp = 0; pp < PPT; ++pp) {
    const int item = tid + pp * nthr;
    rr[pp] = item / mh;
    tt[pp] = item - rr[pp] * mh;
    base[pp] = rr[pp] * N;
    wrow[pp] = work_addr + ((uint32_t)base[pp] << 4);
  }
  constexpr float sT = (float)F::sT;
  PairWB w;
  w.alpha = f2(p.alpha);
  w.oma = f2(p.oma);

  for (long long tile = blockIdx.x; tile < p.tiles; tile += gridDim.x) {
    if (tid == 0) {
      bulk_wait_read0();  // the previous tile's stores have left W
      issue_load(tile);
    }
    if (!mbar_wait_bounded(&bar[0], phase)) *abort_flag = 1;
    phase ^= 1;
    __syncthreads();
    if (*abort_flag) break;

    const long long row0 = tile * R;
    const int rows = (int)min((long long)R, p.B - row0);
    bool active[PPT];
#pragma unroll
    for (int pp = 0; pp < PPT; ++pp) active[pp] = rr[pp] < rows;

    float2 X[PPT][NG], A[PPT][NG], H[PPT][NG], G[PPT][NG];
    uint32_t aa[NG], ab[NG];

    StageRec rec_next = recs[L - 1];
    for (int l = L - 1; l >= 0; --l) {
      const StageRec rec = rec_next;
      if (l > 0) rec_next = recs[l - 1];
      const int s = rec.s;
      const bool first = (l == L - 1), last = (l == 0);
      w.owi = f2(rec.owi);
      w.owj = f2(rec.owj);
      w.owjs = f2(rec.owj * sT);
      float2 dwi = f2(0.0f), dwj = f2(0.0f);

      if (first) {
#pragma unroll
        for (int pp = 0; pp < PPT; ++pp)
          if (active[pp]) {
            const T* s0 = win + base[pp];
            if (!tape) {
              ld_native_pair<NG, T>(s0, tt[pp], s, m, X[pp]);
              ld_native_pair<NG, T>(s0 + RN, tt[pp], s, m, A[pp]);
            }
            ld_native_pair<NG, T>(s0 + 2 * RN, tt[pp], s, m, H[pp]);
            ld_native_pair<NG, T>(s0 + 3 * RN, tt[pp], s, m, G[pp]);
          }
        __syncthreads();  // native inputs are in registers; W may now take slots
      }
#pragma unroll
      for (int pp = 0; pp < PPT; ++pp) {
        if (active[pp]) {
          pair_addrs<NG, 4>(wrow[pp], tt[pp], s, m, aa, ab);
          if (!first) {
#pragma unroll
            for (int o = 0; o < NG; ++o) {
              const float4 va = lds128(aa[o]), vb = lds128(ab[o]);
              X[pp][o] = make_float2(va.x, vb.x);
              A[pp][o] = make_float2(va.y, vb.y);
              H[pp][o] = make_float2(va.z, vb.z);
              G[pp][o] = make_float2(va.w, vb.w);
            }
          }
          {
            if (rec.ck >= 0) {  // a state saved after stage l replaces the rebuilt one
              const float2* c = sck + rec.ck * RN + base[pp] + tt[pp];
#pragma unroll
              for (int o = 0; o < NG; ++o) {
                const float2 va = c[o * m], vb = c[o * m + mh];
                X[pp][o] = make_float2(va.x, vb.x);
                A[pp][o] = make_float2(va.y, vb.y);
              }
            }
          }
          pair_backward<NG, ACT>(X[pp], A[pp], H[pp], G[pp], w, dwi, dwj);
          if (!last) {
#pragma unroll
            for (int o = 0; o < NG; ++o) {
              sts128(aa[o], X[pp][o].x, A[pp][o].x, H[pp][o].x, G[pp][o].x);
              sts128(ab[o], X[pp][o].y, A[pp][o].y, H[pp][o].y, G[pp][o].y);
            }
          }
        }
      }
      if (last) {
        __syncthreads();  // every slot has been read; W may now take the native results
#pragma unroll
        for (int pp = 0; pp < PPT; ++pp)
          if (active[pp]) {
            if (residual) {
              float2 gin[NG];
              ld_native_pair<NG, T>(sdy + base[pp], tt[pp], s, m, gin);
#pragma unroll
              for (int o = 0; o < NG; ++o) H[pp][o] = fadd2(H[pp][o], gin[o]);
            }
            T* wout = win + base[pp];
            st_native_pair<NG, T>(wout, tt[pp], s, m, H[pp]);
            st_native_pair<NG, T>(wout + RN, tt[pp], s, m, G[pp]);
            if (want_rec) {
              st_native_pair<NG, T>(wout + 2 * RN, tt[pp], s, m, X[pp]);
              st_native_pair<NG, T>(wout + 3 * RN, tt[pp], s, m, A[pp]);
            }
          }
      }
      // ---- weight-gradient partial of this stage: fixed-order warp tree, one slot per warp
      {
        const float di = dwi.x + dwi.y, dj = dwj.x + dwj.y;
        const bool hi = (lane & 16) != 0;
        const float give = hi ? di : dj;
        float keep = hi ? dj : di;
        keep += __shfl_xor_sync(0xffffffffu, give, 16);
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) keep += __shfl_xor_sync(0xffffffffu, keep, o);
        if ((lane & 15) == 0) red[(l * nwarp + warp) * 2 + (hi ? 1 : 0)] += keep;
      }
      if (last) fence_proxy_async();
      __syncthreads();
    }
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

// ------------------------------------------------------------------------------------------
// Backward, wide variant: separate input, slot and output buffers (as rows_bwd_kernel), so the next
// tile's TMA loads run during this tile's stages and no layout change needs a read-barrier-write.
// One CTA of up to 512 threads per SM with a full register budget (no spills); the aliased kernel
// above trades registers for a second CTA per SM.
template <int NG, int ACT, typename T, int MAXT>
__global__ void __launch_bounds__(MAXT, 1) pair_bwd_wide_kernel(const RowsParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  using F = ActForm<ACT>;
  const int tid = threadIdx.x, nthr = blockDim.x;
  const int lane = tid & 31, warp = tid >> 5, nwarp = (nthr + 31) >> 5;
  const int N = p.N, m = p.m, R = p.R, L = p.L;
  const int mh = m >> 1;
  const int RN = R * N;
  T* in_s = reinterpret_cast<T*>(smem + p.off_in[0]);
  const uint32_t work_addr = smem_u32(smem + p.off_work);
  T* odx = reinterpret_cast<T*>(smem + p.off_out);
  float2* sck = p.n_ckpt_slots ? reinterpret_cast<float2*>(smem + p.off_ckpt) : nullptr;
  float* red = reinterpret_cast<float*>(smem + p.off_red);
  StageRec* recs = reinterpret_cast<StageRec*>(smem + p.off_w);
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem + p.off_bar);
  int* abort_flag = reinterpret_cast<int*>(bar + 2);
  const T* g_in[4] = {static_cast<const T*>(p.in[0]), static_cast<const T*>(p.in[1]), static_cast<const T*>(p.in[2]),
                      static_cast<const T*>(p.in[3])};
  const float2* ckpt = reinterpret_cast<const float2*>(p.ckpt);
  const bool residual = (p.flags & F_RESIDUAL) != 0;
  const bool recompute = (p.flags & F_RECOMPUTE) != 0;
  const bool want_rec = p.out[2] != nullptr;
  const long long BN = p.B * (long long)N;
  const bool ck_smem = p.n_ckpt_slots > 0;
  const bool tape = (p.flags & F_TAPE) != 0 && !recompute;
  // the staged checkpoints are free again after the stage that uses the earliest one
  const int ck_free_stage = (p.ckpt_every > 0 && (L - 1) / p.ckpt_every > 0) ? p.ckpt_every - 1 : L - 1;

  if (tid == 0) {
    mbar_init(&bar[0], 1);
    mbar_init(&bar[1], 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  fill_stage_table(recs, p, ckpt != nullptr && !recompute, tid, nthr);
  // weight-gradient partials: one (dwi, dwj) slot per stage and THREAD when they fit (a private
  // read-modify-write per stage, no shuffles), else one per stage and warp
  const bool red_thread = (p.flags & F_RED_THREAD) != 0;
  float2* red2 = reinterpret_cast<float2*>(red);
  for (int i = tid; i < (red_thread ? 2 * L * nthr : 2 * L * nwarp); i += nthr) red[i] = 0.0f;
  __syncthreads();

  auto issue_load = [&](long long tl) {
    const long long row0 = tl * R;
    const int rows = (int)min((long long)R, p.B - row0);
    const uint32_t bytes = (uint32_t)(rows * N * sizeof(T));
    mbar_expect_tx(&bar[0], (tape ? 2 : 4) * bytes);
#pragma unroll
    for (int q = 0; q < 4; ++q)
      if (q >= 2 || !tape) bulk_g2s(in_s + q * RN, g_in[q] + row0 * N, bytes, &bar[0]);  // tape: no y, ya
  };
  auto issue_ckpt = [&](long long tl) {
    const long long row0 = tl * R;
    const int rows = (int)min((long long)R, p.B - row0);
    const uint32_t cbytes = (uint32_t)(rows * N * sizeof(float2));
    mbar_expect_tx(&bar[1], p.n_ckpt_slots * cbytes);
    for (uint32_t k = 0; k < p.n_ckpt_slots; ++k)
      bulk_g2s(sck + k * RN, ckpt + (long long)k * BN + row0 * N, cbytes, &bar[1]);
  };

  long long tile = blockIdx.x;
  if (tid == 0 && tile < p.tiles) {
    issue_load(tile);
    if (ck_smem) issue_ckpt(tile);
  }
  uint32_t phase0 = 0, phase1 = 0;
  const int r = tid / mh, t = tid - r * mh;
  const int base = r * N;
  const uint32_t wrow = work_addr + ((uint32_t)base << 4);
  constexpr float sT = (float)F::sT;
  PairWB w;
  w.alpha = f2(p.alpha);
  w.oma = f2(p.oma);
  PairW wf;
  wf.alpha = f2(p.alpha * sT);

  for (; tile < p.tiles; tile += gridDim.x) {
    const long long next = tile + gridDim.x;
    if (!mbar_wait_bounded(&bar[0], phase0)) *abort_flag = 1;
    phase0 ^= 1;
    if (ck_smem) {
      if (!mbar_wait_bounded(&bar[1], phase1)) *abort_flag = 1;
      phase1 ^= 1;
    }
    if (L == 1 && tid == 0) bulk_wait_read0();
    __syncthreads();
    if (*abort_flag) break;

    const long long row0 = tile * R;
    const int rows = (int)min((long long)R, p.B - row0);
    const bool active = r < rows;
    const T* s0 = in_s + base;

    float2 X[NG], A[NG], H[NG], G[NG];
    uint32_t aa[NG], ab[NG];

    if (recompute) {
      for (int l = 0; l < L; ++l) {
        const StageRec rec = recs[l];
        const int s = rec.s;
        wf.owi = f2(rec.owi * sT);
        wf.owj = f2(rec.owj * sT);
        if (active) {
          pair_addrs<NG, 4>(wrow, t, s, m, aa, ab);
          if (l == 0) {
            ld_native_pair<NG, T>(s0, t, s, m, X);
            ld_native_pair<NG, T>(s0 + RN, t, s, m, A);
          } else {
#pragma unroll
            for (int o = 0; o < NG; ++o) {
              const float2 va = lds64(aa[o]), vb = lds64(ab[o]);
              X[o] = make_float2(va.x, vb.x);
              A[o] = make_float2(va.y, vb.y);
            }
          }
          pair_forward<NG, ACT>(X, A, wf);
#pragma unroll
          for (int o = 0; o < NG; ++o) {
            sts64(aa[o], X[o].x, A[o].x);
            sts64(ab[o], X[o].y, A[o].y);
          }
        }
        __syncthreads();
      }
    }

    StageRec rec_next = recs[L - 1];
    for (int l = L - 1; l >= 0; --l) {
      const StageRec rec = rec_next;
      if (l > 0) rec_next = recs[l - 1];  // in flight during this stage's work
      const int s = rec.s;
      const bool first = (l == L - 1), last = (l == 0);
      w.owi = f2(rec.owi);
      w.owj = f2(rec.owj);
      w.owjs = f2(rec.owj * sT);
      float2 dwi = f2(0.0f), dwj = f2(0.0f);

      if (active) {
        pair_addrs<NG, 4>(wrow, t, s, m, aa, ab);
        if (first) {
          ld_native_pair<NG, T>(s0 + 2 * RN, t, s, m, H);
          ld_native_pair<NG, T>(s0 + 3 * RN, t, s, m, G);
          if (tape) {
            // the state after the last stage comes from its checkpoint below
          } else if (!recompute) {
            ld_native_pair<NG, T>(s0, t, s, m, X);
            ld_native_pair<NG, T>(s0 + RN, t, s, m, A);
          } else {
#pragma unroll
            for (int o = 0; o < NG; ++o) {
              const float2 va = lds64(aa[o]), vb = lds64(ab[o]);
              X[o] = make_float2(va.x, vb.x);
              A[o] = make_float2(va.y, vb.y);
            }
          }
        } else {
#pragma unroll
          for (int o = 0; o < NG; ++o) {
            const float4 va = lds128(aa[o]), vb = lds128(ab[o]);
            X[o] = make_float2(va.x, vb.x);
            A[o] = make_float2(va.y, vb.y);
            H[o] = make_float2(va.z, vb.z);
            G[o] = make_float2(va.w, vb.w);
          }
        }
        {
          if (rec.ck >= 0) {
            if ((uint32_t)rec.ck < p.n_ckpt_slots) {
              const float2* c = sck + rec.ck * RN + base + t;
#pragma unroll
              for (int o = 0; o < NG; ++o) {
                const float2 va = c[o * m], vb = c[o * m + mh];
                X[o] = make_float2(va.x, vb.x);
                A[o] = make_float2(va.y, vb.y);
              }
            } else {
              const float2* c = ckpt + (long long)rec.ck * BN + row0 * N + base + t;
#pragma unroll
              for (int o = 0; o < NG; ++o) {
                const float2 va = __ldg(c + o * m), vb = __ldg(c + o * m + mh);
                X[o] = make_float2(va.x, vb.x);
                A[o] = make_float2(va.y, vb.y);
              }
            }
          }
        }
        pair_backward<NG, ACT>(X, A, H, G, w, dwi, dwj);
        if (last) {
          if (residual) {
            float2 gin[NG];
            ld_native_pair<NG, T>(s0 + 2 * RN, t, s, m, gin);
#pragma unroll
            for (int o = 0; o < NG; ++o) H[o] = fadd2(H[o], gin[o]);
          }
          T* wout = odx + base;
          st_native_pair<NG, T>(wout, t, s, m, H);
          st_native_pair<NG, T>(wout + RN, t, s, m, G);
          if (want_rec) {
            st_native_pair<NG, T>(wout + 2 * RN, t, s, m, X);
            st_native_pair<NG, T>(wout + 3 * RN, t, s, m, A);
          }
        } else {
#pragma unroll
          for (int o = 0; o < NG; ++o) {
            sts128(aa[o], X[o].x, A[o].x, H[o].x, G[o].x);
            sts128(ab[o], X[o].y, A[o].y, H[o].y, G[o].y);
          }
        }
      }
      if (red_thread) {
        float2 acc = red2[l * nthr + tid];
        acc.x += dwi.x + dwi.y;
        acc.y += dwj.x + dwj.y;
        red2[l * nthr + tid] = acc;
      } else {
        const float di = dwi.x + dwi.y, dj = dwj.x + dwj.y;
        const bool hi = (lane & 16) != 0;
        const float give = hi ? di : dj;
        float keep = hi ? dj : di;
        keep += __shfl_xor_sync(0xffffffffu, give, 16);
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) keep += __shfl_xor_sync(0xffffffffu, keep, o);
        if ((lane & 15) == 0) red[(l * nwarp + warp) * 2 + (hi ? 1 : 0)] += keep;
      }
      if (l == 1 && tid == 0) bulk_wait_read0();
      if (last) fence_proxy_async();
      __syncthreads();
      if (tid == 0 && next < p.tiles && (residual ? last : first)) issue_load(next);
      if (ck_smem && tid == 0 && next < p.tiles && l == ck_free_stage) issue_ckpt(next);
    }
    if (tid == 0) {
      const uint32_t bytes = (uint32_t)(rows * N * sizeof(T));
      bulk_s2g(static_cast<T*>(p.out[0]) + row0 * N, odx, bytes);
      bulk_s2g(static_cast<T*>(p.out[1]) + row0 * N, odx + RN, bytes);
      if (want_rec) {
        bulk_s2g(static_cast<T*>(p.out[2]) + row0 * N, odx + 2 * RN, bytes);
        bulk_s2g(static_cast<T*>(p.out[3]) + row0 * N, odx + 3 * RN, bytes);
      }
      bulk_commit();
    }
  }
  __syncthreads();
  for (int i = tid; i < 2 * L; i += nthr) {
    const int l = i >> 1, c = i & 1;
    float acc = 0.0f;
    if (red_thread) {
      for (int k = 0; k < nthr; ++k) acc += red[(l * nthr + k) * 2 + c];  // thread order: fixed
    } else {
      for (int w2 = 0; w2 < nwarp; ++w2) acc += red[(l * nwarp + w2) * 2 + c];
    }
    p.partials[(long long)blockIdx.x * 2 * L + i] = acc;
  }
  if (tid == 0) {
    bulk_wait_all0();
    if (*abort_flag) atomicExch(p.status, DEV_WAIT_TIMEOUT);
  }
}

}  // namespace ncn
