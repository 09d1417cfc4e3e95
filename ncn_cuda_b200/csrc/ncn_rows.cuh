// Fused all-stage NCN kernels for one feature per position (E = 1, n_head = 1).
//
// A persistent CTA owns tiles of R whole rows.  The rows of a tile arrive in shared memory
// by 1-D TMA bulk copies (cp.async.bulk + mbarrier), every stage of the stack runs on the
// shared-memory copy, and the results leave by TMA bulk stores; global memory is read once and
// written once per tensor.  Replaces, for this shape class, the per-stage launches of
// ncn_cuda/ncn_fwd_cuda_kernel.cu:28-161 and ncn_cuda/ncn_bwd_cuda_kernel.cu:27-288 and the
// Python stage loop of ncn_cuda/ncn_pytorch_wrapper_v2.py:132-144.
//
// One thread runs whole groups: the NG values of every stream of its group live in registers for
// the NG steps of a stage.  Shared-memory layouts of one row of N = m*NG positions:
//   native       pos = blk*NG + o, one array per stream (what global memory holds; TMA in/out)
//   stage-local  slot = o*m + blk, all streams of a position packed in one 8- or 16-byte slot.  The
//                thread that owns group g touches blk = (g + o*s) mod m, so a warp reads and writes
//                consecutive slots (no bank conflicts), and it writes exactly the slots it read, so
//                the stages can run in place with one barrier between them.
// Everything that depends only on the stage (scaled weights, stride, checkpoint slot) is put in
// a small table in shared memory once per CTA: a thread runs only NG*NG steps per stage, so
// per-stage scalar work (divisions, 64-bit moduli, pointer arithmetic) would otherwise rival them.
#pragma once
#include "ncn_common.cuh"

namespace ncn {

struct __align__(16) StageRec {
  float owi, owj;  // (1-alpha) wi, (1-alpha) wj
  int s;           // block stride of the stage
  int ck;          // index of the checkpoint written after (fwd) / read for (bwd) this stage, or -1
};

__device__ __forceinline__ int wrap_add(int v, int d, int m) {
  v += d;
  return v >= m ? v - m : v;
}

// 32-bit shared-memory addressing for the stage-local slots
__device__ __forceinline__ float2 lds64(uint32_t a) {
  float2 v;
  asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(a) : "memory");
  return v;
}
__device__ __forceinline__ void sts64(uint32_t a, float x, float y) {
  asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(a), "f"(x), "f"(y) : "memory");
}
__device__ __forceinline__ float4 lds128(uint32_t a) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(a) : "memory");
  return v;
}
__device__ __forceinline__ void sts128(uint32_t a, float x, float y, float z, float w) {
  asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(a), "f"(x), "f"(y), "f"(z), "f"(w) : "memory");
}

// gather / scatter of one group in the native layout (positions ((g + o*s) mod m)*NG + o)
template <int NG, typename T>
__device__ __forceinline__ void ld_native(const T* row, int g, int s, int m, float (&v)[NG]) {
  if (s == 0) {
    ld_vec<NG>(row + g * NG, v);
  } else {
    int blk = g;
#pragma unroll
    for (int o = 0; o < NG; ++o) {
      v[o] = Store<T>::ld(row + blk * NG + o);
      blk = wrap_add(blk, s, m);
    }
  }
}
template <int NG, typename T>
__device__ __forceinline__ void st_native(T* row, int g, int s, int m, const float (&v)[NG]) {
  if (s == 0) {
    st_vec<NG>(row + g * NG, v);
  } else {
    int blk = g;
#pragma unroll
    for (int o = 0; o < NG; ++o) {
      Store<T>::st(row + blk * NG + o, v[o]);
      blk = wrap_add(blk, s, m);
    }
  }
}

// byte addresses (shared window) of the NG slots of group g; slots are (1 << SHIFT) bytes
template <int NG, int SHIFT>
__device__ __forceinline__ void group_addrs(uint32_t row_addr, int g, int s, int m, uint32_t (&sa)[NG]) {
  int blk = g;
  uint32_t ro = row_addr;
  const uint32_t mstep = (uint32_t)m << SHIFT;
#pragma unroll
  for (int o = 0; o < NG; ++o) {
    sa[o] = ro + ((uint32_t)blk << SHIFT);
    ro += mstep;
    blk = wrap_add(blk, s, m);
  }
}

// Stage table: scaled weights, stride s = 0 for stage 0 else 2^(stage-1) mod m
// (torch_ref/ncn_pytorch.py:38), and the checkpoint index (a state is kept after every
// ckpt_every-th stage except the last; with F_TAPE the last stage's state takes the slot after those).
__device__ __forceinline__ void fill_stage_table(StageRec* rec, const float* W, float oma, int l0, int m, int L,
                                                 int ckpt_every, int flags, bool have_ckpt, int tid, int nthr) {
  for (int i = tid; i < L; i += nthr) {
    StageRec r;
    r.owi = W[2 * i] * oma;
    r.owj = W[2 * i + 1] * oma;
    r.s = stage_stride(l0 + i, m);
    r.ck = (have_ckpt && ckpt_every > 0 && i != L - 1 && ((i + 1) % ckpt_every == 0)) ? (i + 1) / ckpt_every - 1 : -1;
    if (have_ckpt && (flags & F_TAPE) && i == L - 1) r.ck = ckpt_every > 0 ? (L - 1) / ckpt_every : 0;
    rec[i] = r;
  }
}
__device__ __forceinline__ void fill_stage_table(StageRec* rec, const RowsParams& p, bool have_ckpt, int tid, int nthr) {
  fill_stage_table(rec, p.W, p.oma, p.l0, p.m, p.L, p.ckpt_every, p.flags, have_ckpt, tid, nthr);
}

template <int NG, int ACT, typename T, int MAXT>
__global__ void __launch_bounds__(MAXT, 1) rows_fwd_kernel(const RowsParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x, nthr = blockDim.x;
  const int N = p.N, m = p.m, R = p.R, L = p.L;
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
  fill_stage_table(recs, p, ckpt != nullptr, tid, nthr);
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
  StageW w;
  w.alpha = p.alpha; w.oma = p.oma;

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
    float2* ck_tile = ckpt + row0 * N;

    for (int l = 0; l < L; ++l) {
      const StageRec rec = recs[l];
      const int s = rec.s;
      const bool first = (l == 0), last = (l == L - 1);
      w.owi = rec.owi; w.owj = rec.owj;

      int r = r0, g = g0;
      while (r < rows) {
        float x[NG], a[NG];
        uint32_t adr[NG];
        const int base = r * N;
        if (first) {
          ld_native<NG, T>(sx + base, g, s, m, x);
          ld_native<NG, T>(sa + base, g, s, m, a);
        } else {
          group_addrs<NG, 3>(work_addr + ((uint32_t)base << 3), g, s, m, adr);
#pragma unroll
          for (int o = 0; o < NG; ++o) {
            const float2 v = lds64(adr[o]);
            x[o] = v.x; a[o] = v.y;
          }
        }
        group_forward<NG, ACT>(x, a, w);
        if (rec.ck >= 0) {  // filed under this stage's groups: the backward of this stage reads o*m + g
          float2* ck = ck_tile + (long long)rec.ck * BN + base + g;
#pragma unroll
          for (int o = 0; o < NG; ++o) ck[o * m] = make_float2(x[o], a[o]);
        }
        if (last) {
          if (residual) {
            float xin[NG];
            ld_native<NG, T>(sx + base, g, s, m, xin);
#pragma unroll
            for (int o = 0; o < NG; ++o) x[o] += xin[o];
          }
          st_native<NG, T>(ox + base, g, s, m, x);
          st_native<NG, T>(oa + base, g, s, m, a);
        } else {
          if (first) group_addrs<NG, 3>(work_addr + ((uint32_t)base << 3), g, s, m, adr);
#pragma unroll
          for (int o = 0; o < NG; ++o) sts64(adr[o], x[o], a[o]);
        }
        r += dr; g += dg;
        if (g >= m) { g -= m; ++r; }
      }
      // the store of the previous tile must have finished reading the out buffer before the
      // last stage of this tile overwrites it
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
// Backward.  Shared memory per tile: in buffer (4 native streams: state0, state1, dy, dya),
// work buffer (one 16-byte slot (x, a, gx, ga) per position), out buffer (native dx, dxa and,
// when asked, the rebuilt x, xa), optional slots for checkpoints.
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
  const uint32_t work_addr = smem_u32(smem + p.off_work);  // (x, a, gx, ga) per 16-byte slot
  T* odx = reinterpret_cast<T*>(smem + p.off_out);
  T* odxa = odx + RN;
  T* orx = odxa + RN;
  T* orxa = orx + RN;
  float2* sck = p.n_ckpt_slots ? reinterpret_cast<float2*>(smem + p.off_ckpt) : nullptr;
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
  const bool tape = (p.flags & F_TAPE) != 0 && !recompute;
  const long long BN = p.B * (long long)N;
  // the staged checkpoints are free again after the stage that uses the earliest one
  const int ck_free_stage = (p.ckpt_every > 0 && (L - 1) / p.ckpt_every > 0) ? p.ckpt_every - 1 : L - 1;

  if (tid == 0) {
    mbar_init(&bar[0], 1);
    mbar_init(&bar[1], 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  fill_stage_table(recs, p, ckpt != nullptr && !recompute, tid, nthr);
  for (int i = tid; i < 2 * L * nwarp; i += nthr) red[i] = 0.0f;
  __syncthreads();

  auto issue_load = [&](long long t, int b) {
    const long long row0 = t * R;
    const int rows = (int)min((long long)R, p.B - row0);
    const uint32_t bytes = (uint32_t)(rows * N * sizeof(T));
    mbar_expect_tx(&bar[b], (tape ? 2 : 4) * bytes);
#pragma unroll
    for (int q = 0; q < 4; ++q)
      if (q >= 2 || !tape) bulk_g2s(in_s[b] + q * RN, g_in[q] + row0 * N, bytes, &bar[b]);  // tape: no y, ya
  };
  // Checkpoints staged in shared memory (only with a single in buffer, so bar[1] is free for
  // them): all of a tile's checkpoints arrive together and stay until the stage that uses the
  // earliest one has run.
  const bool ck_smem = p.n_ckpt_slots > 0;
  auto issue_ckpt = [&](long long t) {
    const long long row0 = t * R;
    const int rows = (int)min((long long)R, p.B - row0);
    const uint32_t cbytes = (uint32_t)(rows * N * sizeof(float2));
    mbar_expect_tx(&bar[1], p.n_ckpt_slots * cbytes);
    for (uint32_t k = 0; k < p.n_ckpt_slots; ++k)
      bulk_g2s(sck + k * RN, ckpt + (long long)k * BN + row0 * N, cbytes, &bar[1]);
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
  StageW w;
  w.alpha = p.alpha; w.oma = p.oma;

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
        const StageRec rec = recs[l];
        const int s = rec.s;
        w.owi = rec.owi; w.owj = rec.owj;
        int r = r0, g = g0;
        while (r < rows) {
          float x[NG], a[NG];
          uint32_t adr[NG];
          const int base = r * N;
          group_addrs<NG, 4>(work_addr + ((uint32_t)base << 4), g, s, m, adr);
          if (l == 0) {
            ld_native<NG, T>(s0 + base, g, s, m, x);
            ld_native<NG, T>(s1 + base, g, s, m, a);
          } else {
#pragma unroll
            for (int o = 0; o < NG; ++o) {
              const float2 v = lds64(adr[o]);
              x[o] = v.x; a[o] = v.y;
            }
          }
          group_forward<NG, ACT>(x, a, w);
#pragma unroll
          for (int o = 0; o < NG; ++o) sts64(adr[o], x[o], a[o]);
          r += dr; g += dg;
          if (g >= m) { g -= m; ++r; }
        }
        __syncthreads();
      }
    }

    // ---- reverse sweep over the stages
    for (int l = L - 1; l >= 0; --l) {
      const StageRec rec = recs[l];
      const int s = rec.s;
      const bool first = (l == L - 1), last = (l == 0);
      w.owi = rec.owi; w.owj = rec.owj;
      const bool use_ck = rec.ck >= 0;  // a state saved after stage l replaces the rebuilt one
      float dwi = 0.0f, dwj = 0.0f;

      int r = r0, g = g0;
      while (r < rows) {
        float x[NG], a[NG], gx[NG], ga[NG];
        uint32_t adr[NG];
        const int base = r * N;
        group_addrs<NG, 4>(work_addr + ((uint32_t)base << 4), g, s, m, adr);
        if (first) {
          ld_native<NG, T>(sgy + base, g, s, m, gx);
          ld_native<NG, T>(sga + base, g, s, m, ga);
          if (use_ck) {
            // tape: filled below from the checkpoint
          } else if (!recompute) {
            ld_native<NG, T>(s0 + base, g, s, m, x);
            ld_native<NG, T>(s1 + base, g, s, m, a);
          } else {
#pragma unroll
            for (int o = 0; o < NG; ++o) {
              const float2 v = lds64(adr[o]);
              x[o] = v.x; a[o] = v.y;
            }
          }
        } else {
#pragma unroll
          for (int o = 0; o < NG; ++o) {
            const float4 v = lds128(adr[o]);
            x[o] = v.x; a[o] = v.y; gx[o] = v.z; ga[o] = v.w;
          }
        }
        {
          if (use_ck) {
            if ((uint32_t)rec.ck < p.n_ckpt_slots) {
              const float2* c = sck + rec.ck * RN + base + g;
#pragma unroll
              for (int o = 0; o < NG; ++o) {
                const float2 v = c[o * m];
                x[o] = v.x; a[o] = v.y;
              }
            } else {
              const float2* c = ckpt + (long long)rec.ck * BN + row0 * N + base + g;
#pragma unroll
              for (int o = 0; o < NG; ++o) {
                const float2 v = __ldg(c + o * m);
                x[o] = v.x; a[o] = v.y;
              }
            }
          }
        }

        group_backward<NG, ACT>(x, a, gx, ga, w, dwi, dwj);

        if (last) {
          if (residual) {
            float gin[NG];
            ld_native<NG, T>(sgy + base, g, s, m, gin);
#pragma unroll
            for (int o = 0; o < NG; ++o) gx[o] += gin[o];
          }
          st_native<NG, T>(odx + base, g, s, m, gx);
          st_native<NG, T>(odxa + base, g, s, m, ga);
          if (want_rec) {
            st_native<NG, T>(orx + base, g, s, m, x);
            st_native<NG, T>(orxa + base, g, s, m, a);
          }
        } else {
#pragma unroll
          for (int o = 0; o < NG; ++o) sts128(adr[o], x[o], a[o], gx[o], ga[o]);
        }
        r += dr; g += dg;
        if (g >= m) { g -= m; ++r; }
      }
      // ---- weight-gradient partial of this stage: fixed-order warp tree, one slot per warp.
      // The two sums share one tree: after the first exchange the low half-warp carries dwi and
      // the high half-warp dwj.
      {
        const bool hi = (lane & 16) != 0;
        const float give = hi ? dwi : dwj;
        float keep = hi ? dwj : dwi;
        keep += __shfl_xor_sync(0xffffffffu, give, 16);
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) keep += __shfl_xor_sync(0xffffffffu, keep, o);
        if ((lane & 15) == 0) red[(l * nwarp + warp) * 2 + (hi ? 1 : 0)] += keep;
      }
      if (l == 1 && tid == 0) bulk_wait_read0();
      if (last) fence_proxy_async();
      __syncthreads();
      if (p.nbuf == 1 && tid == 0 && next < p.tiles && (residual ? last : first)) issue_load(next, 0);
      if (ck_smem && tid == 0 && next < p.tiles && l == ck_free_stage) issue_ckpt(next);
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
    for (int w2 = 0; w2 < nwarp; ++w2) acc += red[(l * nwarp + w2) * 2 + c];
    p.partials[(long long)blockIdx.x * 2 * L + i] = acc;
  }
  if (tid == 0) {
    bulk_wait_all0();
    if (*abort_flag) atomicExch(p.status, DEV_WAIT_TIMEOUT);
  }
}

}  // namespace ncn
