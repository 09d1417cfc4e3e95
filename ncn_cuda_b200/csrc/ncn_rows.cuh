// Fused all-stage NCN kernels for one feature per position (E = 1, n_head = 1).
//
// A persistent CTA owns tiles of R whole rows.  The rows of a tile arrive in shared memory
// by 1-D TMA bulk copies (cp.async.bulk + mbarrier), every stage of the stack runs on the
// shared-memory copy, and the results leave by TMA bulk stores; global memory is read once and
// written once per tensor.  Replaces, for this shape class, the per-stage launches of
// ncn_cuda/ncn_fwd_cuda_kernel.cu:28-161 and ncn_cuda/ncn_bwd_cuda_kernel.cu:27-288 and the
// Python stage loop of ncn_cuda/ncn_pytorch_wrapper_v2.py:132-144.
//
// Shared-memory layouts of one row of N = m*NG values:
//   native      pos = blk*NG + o           (what global memory holds; TMA in/out buffers)
//   stage-local adr = o*m + blk            (between stages: a thread that owns group g touches
//                                           blk = (g + o*s) mod m, so a warp reads consecutive words)
// One thread runs whole groups: its NG values of both streams live in registers for the NG steps.
#pragma once
#include "ncn_common.cuh"

namespace ncn {

template <int NG, int ACT, typename T, int MAXT>
__global__ void __launch_bounds__(MAXT, 1) rows_fwd_kernel(const RowsParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x, nthr = blockDim.x;
  const int N = p.N, m = p.m, R = p.R, L = p.L;
  const int RN = R * N;
  T* in_x[2] = {reinterpret_cast<T*>(smem + p.off_in[0]), reinterpret_cast<T*>(smem + p.off_in[1])};
  float* wx = reinterpret_cast<float*>(smem + p.off_work);
  float* wa = wx + RN;
  T* ox = reinterpret_cast<T*>(smem + p.off_out);
  T* oa = ox + RN;
  float* sw = reinterpret_cast<float*>(smem + p.off_w);
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem + p.off_bar);
  int* abort_flag = reinterpret_cast<int*>(bar + 2);
  const T* gx_in = static_cast<const T*>(p.in[0]);
  const T* ga_in = static_cast<const T*>(p.in[1]);
  T* gy_out = static_cast<T*>(p.out[0]);
  T* gya_out = static_cast<T*>(p.out[1]);
  const bool residual = (p.flags & F_RESIDUAL) != 0;
  const long long BN = p.B * (long long)N;

  if (tid == 0) {
    mbar_init(&bar[0], 1);
    mbar_init(&bar[1], 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  for (int i = tid; i < 2 * L; i += nthr) sw[i] = p.W[i] * p.oma;  // (1-alpha) folded into the weights
  __syncthreads();

  auto issue_load = [&](long long t, int b) {
    const long long row0 = t * R;
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
  const int r0 = tid / m, g0 = tid - r0 * m;
  const int dr = nthr / m, dg = nthr - dr * m;

  for (; tile < p.tiles; tile += gridDim.x) {
    const long long next = tile + gridDim.x;
    if (p.nbuf == 2 && tid == 0 && next < p.tiles) issue_load(next, buf ^ 1);
    const uint32_t ph = buf ? phase1 : phase0;
    if (!mbar_wait_bounded(&bar[buf], ph)) *abort_flag = 1;
    if (buf) phase1 ^= 1; else phase0 ^= 1;
    if (L == 1 && tid == 0) bulk_wait_read0();  // previous tile's store has left the out buffer
    __syncthreads();
    if (*abort_flag) break;

    const long long row0 = tile * R;
    const int rows = (int)min((long long)R, p.B - row0);
    const T* sx = in_x[buf];
    const T* sa = sx + RN;

    for (int l = 0; l < L; ++l) {
      const int s = stage_stride(p.l0 + l, m);
      const float wi_s = sw[2 * l], wj_s = sw[2 * l + 1];
      const bool first = (l == 0), last = (l == L - 1);
      const bool save = p.ckpt != nullptr && p.ckpt_every > 0 && !last && ((l + 1) % p.ckpt_every == 0);
      float* ck = save ? p.ckpt + (long long)((l + 1) / p.ckpt_every - 1) * 2 * BN + row0 * N : nullptr;

      int r = r0, g = g0;
      while (r < rows) {
        float x[NG], a[NG];
        const int base = r * N;
        // ---- load
        if (first) {
          if (s == 0) {
            ld_vec<NG>(sx + base + g * NG, x);
            ld_vec<NG>(sa + base + g * NG, a);
          } else {
            int blk = g;
#pragma unroll
            for (int o = 0; o < NG; ++o) {
              x[o] = Store<T>::ld(sx + base + blk * NG + o);
              a[o] = Store<T>::ld(sa + base + blk * NG + o);
              blk += s; if (blk >= m) blk -= m;
            }
          }
        } else {
          int blk = g;
#pragma unroll
          for (int o = 0; o < NG; ++o) {
            x[o] = wx[base + o * m + blk];
            a[o] = wa[base + o * m + blk];
            blk += s; if (blk >= m) blk -= m;
          }
        }
        // ---- all NG steps of this group
        group_forward<NG, ACT>(x, a, wi_s, wj_s, p.alpha);
        // ---- store
        if (last) {
          if (residual) {
            int blk = g;
#pragma unroll
            for (int o = 0; o < NG; ++o) {
              x[o] += Store<T>::ld(sx + base + blk * NG + o);
              blk += s; if (blk >= m) blk -= m;
            }
          }
          if (s == 0) {
            st_vec<NG>(ox + base + g * NG, x);
            st_vec<NG>(oa + base + g * NG, a);
          } else {
            int blk = g;
#pragma unroll
            for (int o = 0; o < NG; ++o) {
              Store<T>::st(ox + base + blk * NG + o, x[o]);
              Store<T>::st(oa + base + blk * NG + o, a[o]);
              blk += s; if (blk >= m) blk -= m;
            }
          }
        } else {
          int blk = g;
#pragma unroll
          for (int o = 0; o < NG; ++o) {
            wx[base + o * m + blk] = x[o];
            wa[base + o * m + blk] = a[o];
            if (save) {
              ck[base + o * m + blk] = x[o];
              ck[BN + base + o * m + blk] = a[o];
            }
            blk += s; if (blk >= m) blk -= m;
          }
        }
        r += dr; g += dg;
        if (g >= m) { g -= m; ++r; }
      }
      // the store of the previous tile must have finished reading the out buffer before the
      // last stage of this tile overwrites it
      if (L > 1 && l == L - 2 && tid == 0) bulk_wait_read0();
      if (last) fence_proxy_async();
      __syncthreads();
      if (p.nbuf == 1 && tid == 0 && next < p.tiles && (residual ? last : first))
        issue_load(next, 0);
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
// Backward.  Shared memory per tile: in buffer (4 native streams: state0, state1, dy, dya),
// work buffer (4 stage-local fp32 streams: x, a, gx, ga), out buffer (native dx, dxa and, when
// asked, the rebuilt x, xa), optional slots for checkpoints.
//   default       in[0..1] = net OUTPUT (y, ya); every stage input is rebuilt by the reversible
//                 inverse, restarting from a stored stage-boundary state wherever the forward
//                 saved one (p.ckpt), which bounds the rounding growth of long inverse chains.
//   F_RECOMPUTE   in[0..1] = net INPUT (x, xa); the forward is replayed in fp32 first.  Needed
//                 when the stored tensors are bf16 (an inverse started from rounded outputs is
//                 useless) and for residual layers.
// dW: each thread accumulates its groups, a warp shuffle tree and a per-warp slot in shared
// memory give per-CTA partials in a fixed order; p.partials[cta][L][2] is summed by
// dw_reduce_kernel in a fixed order, so dW is bitwise reproducible for a given launch shape.
template <int NG, int ACT, typename T, int MAXT>
__global__ void __launch_bounds__(MAXT, 1) rows_bwd_kernel(const RowsParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x, nthr = blockDim.x;
  const int lane = tid & 31, warp = tid >> 5, nwarp = (nthr + 31) >> 5;
  const int N = p.N, m = p.m, R = p.R, L = p.L;
  const int RN = R * N;
  T* in_s[2] = {reinterpret_cast<T*>(smem + p.off_in[0]), reinterpret_cast<T*>(smem + p.off_in[1])};
  float* wx = reinterpret_cast<float*>(smem + p.off_work);
  float* wa = wx + RN;
  float* wgx = wa + RN;
  float* wga = wgx + RN;
  T* odx = reinterpret_cast<T*>(smem + p.off_out);
  T* odxa = odx + RN;
  T* orx = odxa + RN;
  T* orxa = orx + RN;
  float* sck = p.n_ckpt_slots ? reinterpret_cast<float*>(smem + p.off_ckpt) : nullptr;
  float* red = reinterpret_cast<float*>(smem + p.off_red);  // [L][nwarp][2]
  float* sw = reinterpret_cast<float*>(smem + p.off_w);
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem + p.off_bar);
  int* abort_flag = reinterpret_cast<int*>(bar + 2);
  const T* g_in[4] = {static_cast<const T*>(p.in[0]), static_cast<const T*>(p.in[1]), static_cast<const T*>(p.in[2]),
                      static_cast<const T*>(p.in[3])};
  const bool residual = (p.flags & F_RESIDUAL) != 0;
  const bool recompute = (p.flags & F_RECOMPUTE) != 0;
  const bool want_rec = p.out[2] != nullptr;
  const long long BN = p.B * (long long)N;
  const int n_ck = (p.ckpt != nullptr && p.ckpt_every > 0) ? (L - 1) / p.ckpt_every : 0;

  if (tid == 0) {
    mbar_init(&bar[0], 1);
    mbar_init(&bar[1], 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  for (int i = tid; i < 2 * L; i += nthr) sw[i] = p.W[i];
  for (int i = tid; i < 2 * L * nwarp; i += nthr) red[i] = 0.0f;
  __syncthreads();

  auto issue_load = [&](long long t, int b) {
    const long long row0 = t * R;
    const int rows = (int)min((long long)R, p.B - row0);
    const uint32_t bytes = (uint32_t)(rows * N * sizeof(T));
    const uint32_t cbytes = (uint32_t)(rows * N * sizeof(float));
    mbar_expect_tx(&bar[b], 4 * bytes);
#pragma unroll
    for (int q = 0; q < 4; ++q) bulk_g2s(in_s[b] + q * RN, g_in[q] + row0 * N, bytes, &bar[b]);
  };
  // Checkpoints staged in shared memory (only with a single in buffer, so bar[1] is free for
  // them): all of a tile's checkpoints arrive together and stay until the stage that uses the
  // earliest one has run.
  const bool ck_smem = p.n_ckpt_slots > 0;
  auto issue_ckpt = [&](long long t) {
    const long long row0 = t * R;
    const int rows = (int)min((long long)R, p.B - row0);
    const uint32_t cbytes = (uint32_t)(rows * N * sizeof(float));
    mbar_expect_tx(&bar[1], 2 * p.n_ckpt_slots * cbytes);
    for (uint32_t k = 0; k < 2 * p.n_ckpt_slots; ++k)
      bulk_g2s(sck + k * RN, p.ckpt + (long long)k * BN + row0 * N, cbytes, &bar[1]);
  };

  long long tile = blockIdx.x;
  if (tid == 0 && tile < p.tiles) {
    issue_load(tile, 0);
    if (ck_smem) issue_ckpt(tile);
  }
  uint32_t phase0 = 0, phase1 = 0;
  int buf = 0;
  const int r0 = tid / m, g0 = tid - r0 * m;
  const int dr = nthr / m, dg = nthr - dr * m;

  for (; tile < p.tiles; tile += gridDim.x) {
    const long long next = tile + gridDim.x;
    if (p.nbuf == 2 && tid == 0 && next < p.tiles) issue_load(next, buf ^ 1);
    const uint32_t ph = buf ? phase1 : phase0;
    if (!mbar_wait_bounded(&bar[buf], ph)) *abort_flag = 1;
    if (buf) phase1 ^= 1; else phase0 ^= 1;
    if (ck_smem) {
      if (!mbar_wait_bounded(&bar[1], phase1)) *abort_flag = 1;
      phase1 ^= 1;
    }
    if (L == 1 && tid == 0) bulk_wait_read0();
    __syncthreads();
    if (*abort_flag) break;

    const long long row0 = tile * R;
    const int rows = (int)min((long long)R, p.B - row0);
    const T* s0 = in_s[buf];
    const T* s1 = s0 + RN;
    const T* sgy = s1 + RN;
    const T* sga = sgy + RN;

    // ---- optional forward replay: net input (native) -> net output (stage-local, fp32)
    if (recompute) {
      for (int l = 0; l < L; ++l) {
        const int s = stage_stride(p.l0 + l, m);
        const float wi_s = sw[2 * l] * p.oma, wj_s = sw[2 * l + 1] * p.oma;
        int r = r0, g = g0;
        while (r < rows) {
          float x[NG], a[NG];
          const int base = r * N;
          if (l == 0) {
            if (s == 0) {
              ld_vec<NG>(s0 + base + g * NG, x);
              ld_vec<NG>(s1 + base + g * NG, a);
            } else {
              int blk = g;
#pragma unroll
              for (int o = 0; o < NG; ++o) {
                x[o] = Store<T>::ld(s0 + base + blk * NG + o);
                a[o] = Store<T>::ld(s1 + base + blk * NG + o);
                blk += s; if (blk >= m) blk -= m;
              }
            }
          } else {
            int blk = g;
#pragma unroll
            for (int o = 0; o < NG; ++o) {
              x[o] = wx[base + o * m + blk];
              a[o] = wa[base + o * m + blk];
              blk += s; if (blk >= m) blk -= m;
            }
          }
          group_forward<NG, ACT>(x, a, wi_s, wj_s, p.alpha);
          int blk = g;
#pragma unroll
          for (int o = 0; o < NG; ++o) {
            wx[base + o * m + blk] = x[o];
            wa[base + o * m + blk] = a[o];
            blk += s; if (blk >= m) blk -= m;
          }
          r += dr; g += dg;
          if (g >= m) { g -= m; ++r; }
        }
        __syncthreads();
      }
    }

    // ---- reverse sweep over the stages
    for (int l = L - 1; l >= 0; --l) {
      const int s = stage_stride(p.l0 + l, m);
      const float wi = sw[2 * l], wj = sw[2 * l + 1];
      const bool first = (l == L - 1), last = (l == 0);
      // a state saved after stage l replaces the rebuilt one
      const bool use_ck = !recompute && !first && n_ck > 0 && ((l + 1) % p.ckpt_every == 0);
      const int ck_k = use_ck ? (l + 1) / p.ckpt_every - 1 : 0;
      float dwi = 0.0f, dwj = 0.0f;

      int r = r0, g = g0;
      while (r < rows) {
        float x[NG], a[NG], gx[NG], ga[NG];
        const int base = r * N;
        // ---- state
        if (first && !recompute) {
          if (s == 0) {
            ld_vec<NG>(s0 + base + g * NG, x);
            ld_vec<NG>(s1 + base + g * NG, a);
          } else {
            int blk = g;
#pragma unroll
            for (int o = 0; o < NG; ++o) {
              x[o] = Store<T>::ld(s0 + base + blk * NG + o);
              a[o] = Store<T>::ld(s1 + base + blk * NG + o);
              blk += s; if (blk >= m) blk -= m;
            }
          }
        } else if (use_ck) {
          int blk = g;
          if ((uint32_t)ck_k < p.n_ckpt_slots) {
            const float* cx = sck + (2 * ck_k) * RN;
            const float* ca = cx + RN;
#pragma unroll
            for (int o = 0; o < NG; ++o) {
              x[o] = cx[base + o * m + blk];
              a[o] = ca[base + o * m + blk];
              blk += s; if (blk >= m) blk -= m;
            }
          } else {
            const float* cx = p.ckpt + (long long)(2 * ck_k) * BN + row0 * N;
            const float* ca = cx + BN;
#pragma unroll
            for (int o = 0; o < NG; ++o) {
              x[o] = __ldg(cx + base + o * m + blk);
              a[o] = __ldg(ca + base + o * m + blk);
              blk += s; if (blk >= m) blk -= m;
            }
          }
        } else {
          int blk = g;
#pragma unroll
          for (int o = 0; o < NG; ++o) {
            x[o] = wx[base + o * m + blk];
            a[o] = wa[base + o * m + blk];
            blk += s; if (blk >= m) blk -= m;
          }
        }
        // ---- cotangents
        if (first) {
          if (s == 0) {
            ld_vec<NG>(sgy + base + g * NG, gx);
            ld_vec<NG>(sga + base + g * NG, ga);
          } else {
            int blk = g;
#pragma unroll
            for (int o = 0; o < NG; ++o) {
              gx[o] = Store<T>::ld(sgy + base + blk * NG + o);
              ga[o] = Store<T>::ld(sga + base + blk * NG + o);
              blk += s; if (blk >= m) blk -= m;
            }
          }
        } else {
          int blk = g;
#pragma unroll
          for (int o = 0; o < NG; ++o) {
            gx[o] = wgx[base + o * m + blk];
            ga[o] = wga[base + o * m + blk];
            blk += s; if (blk >= m) blk -= m;
          }
        }

        group_backward<NG, ACT>(x, a, gx, ga, wi, wj, p.alpha, p.oma, dwi, dwj);

        // ---- store
        if (last) {
          if (residual) {
            int blk = g;
#pragma unroll
            for (int o = 0; o < NG; ++o) {
              gx[o] += Store<T>::ld(sgy + base + blk * NG + o);
              blk += s; if (blk >= m) blk -= m;
            }
          }
          if (s == 0) {
            st_vec<NG>(odx + base + g * NG, gx);
            st_vec<NG>(odxa + base + g * NG, ga);
            if (want_rec) {
              st_vec<NG>(orx + base + g * NG, x);
              st_vec<NG>(orxa + base + g * NG, a);
            }
          } else {
            int blk = g;
#pragma unroll
            for (int o = 0; o < NG; ++o) {
              Store<T>::st(odx + base + blk * NG + o, gx[o]);
              Store<T>::st(odxa + base + blk * NG + o, ga[o]);
              if (want_rec) {
                Store<T>::st(orx + base + blk * NG + o, x[o]);
                Store<T>::st(orxa + base + blk * NG + o, a[o]);
              }
              blk += s; if (blk >= m) blk -= m;
            }
          }
        } else {
          int blk = g;
#pragma unroll
          for (int o = 0; o < NG; ++o) {
            wx[base + o * m + blk] = x[o];
            wa[base + o * m + blk] = a[o];
            wgx[base + o * m + blk] = gx[o];
            wga[base + o * m + blk] = ga[o];
            blk += s; if (blk >= m) blk -= m;
          }
        }
        r += dr; g += dg;
        if (g >= m) { g -= m; ++r; }
      }
      // ---- weight-gradient partial of this stage: fixed-order warp tree, one slot per warp
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        dwi += __shfl_xor_sync(0xffffffffu, dwi, o);
        dwj += __shfl_xor_sync(0xffffffffu, dwj, o);
      }
      if (lane == 0) {
        red[(l * nwarp + warp) * 2] += dwi;
        red[(l * nwarp + warp) * 2 + 1] += dwj;
      }
      if (l == 1 && tid == 0) bulk_wait_read0();
      if (last) fence_proxy_async();
      __syncthreads();
      if (p.nbuf == 1 && tid == 0 && next < p.tiles && (residual ? last : first))
        issue_load(next, 0);
      if (ck_smem && tid == 0 && next < p.tiles && l == p.ckpt_every - 1) issue_ckpt(next);
    }
    if (tid == 0) {
      const uint32_t bytes = (uint32_t)(rows * N * sizeof(T));
      bulk_s2g(static_cast<T*>(p.out[0]) + row0 * N, odx, bytes);
      bulk_s2g(static_cast<T*>(p.out[1]) + row0 * N, odxa, bytes);
      if (want_rec) {
        bulk_s2g(static_cast<T*>(p.out[2]) + row0 * N, orx, bytes);
        bulk_s2g(static_cast<T*>(p.out[3]) + row0 * N, orxa, bytes);
      }
      bulk_commit();
    }
    if (p.nbuf == 2) buf ^= 1;
  }
  // ---- per-CTA partial: sum the warp slots in warp order
  __syncthreads();
  for (int i = tid; i < 2 * L; i += nthr) {
    const int l = i >> 1, c = i & 1;
    float acc = 0.0f;
    for (int w = 0; w < nwarp; ++w) acc += red[(l * nwarp + w) * 2 + c];
    p.partials[(long long)blockIdx.x * 2 * L + i] = acc;
  }
  if (tid == 0) {
    bulk_wait_all0();
    if (*abort_flag) atomicExch(p.status, DEV_WAIT_TIMEOUT);
  }
}

}  // namespace ncn
