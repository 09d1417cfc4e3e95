// Register-resident fused row kernels, software-pipelined (n = 4).
//
// Same idea as ncn_lanes.cuh (a thread keeps its groups in registers through all stages and the
// change of stride between two stages is a shift of each offset's array against the threads), with
// the exchange taken off the critical path.  Shuffles and shared-memory accesses share one pipe per
// SM, and in ncn_lanes.cuh every warp of a CTA is in its exchange at the same time, so that pipe's
// time adds to the arithmetic's.  Here a thread runs TWO half-rows half a stage apart:
//
//   set A: groups 2t, 2t+1 of the first half of the row      set B: the same in the second half
//
//   block A(l):  A publishes + shuffles out of stage l   ||   B computes stage l, then publishes
//   barrier
//   block B(l):  A fetches its halo, computes stage l'   ||   B shuffles out of stage l, fetches its halo
//   barrier                                                   (l' = next stage)
//
// Inside a block the exchange of one set and the arithmetic of the other are independent
// instructions of one basic block, so the compiler interleaves them and the shuffle / shared-memory
// pipe works while the FMA and special-function pipes do.  The two sets are the two halves of the
// ring of blocks; at the two seams a warp's neighbour belongs to the other set, which is why both
// sets publish before barrier 1 and fetch after it.
//
// A set's share of a thread is ONE register pair per stream and offset (groups 2t, 2t+1), so a
// shift by k blocks is: even k, both halves from lane +- k/2; odd k (only where the stride changes
// by one block), the halves swap and come from two lanes.  Lanes whose source lies in the
// neighbouring warp take it from the halo that warp published (its first / last k values per
// offset and stream).  The halo lives in the tile buffer, which is idle while the stages run.
#pragma once
#include <type_traits>

#include "ncn_lanes.cuh"

namespace ncn {

// byte addresses (shared window) of the halo areas one set of a thread works with, each already advanced to this
// lane's pair (8 bytes per lane)
struct PipeHalo {
  uint32_t mine8;  // this virtual warp's area
  uint32_t up8m;   // the area of the warp holding the next higher blocks, minus 256 (= 32 lanes): lane + q - 32
  uint32_t dn8;    // the area of the warp holding the next lower blocks
};

template <int I, int N, typename F>
__device__ __forceinline__ void static_for(F&& f) {
  if constexpr (I < N) {
    f(std::integral_constant<int, I>{});
    static_for<I + 1, N>(f);
  }
}
// predicated shared-memory accesses at [base + IMM]
template <int IMM>
__device__ __forceinline__ void sts64_io(bool on, uint32_t a, float x, float y) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.s32 p, %3, 0;\n\t@p st.shared.v2.f32 [%0+%4], {%1, %2};\n\t}" ::"r"(a), "f"(x), "f"(y),
               "r"((int)on), "n"(IMM)
               : "memory");
}
template <int IMM>
__device__ __forceinline__ void lds64_io(bool on, uint32_t a, float2& v) {  // v keeps its value where !on
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.s32 p, %3, 0;\n\t@p ld.shared.v2.f32 {%0, %1}, [%2+%4];\n\t}"
               : "+f"(v.x), "+f"(v.y)
               : "r"(a), "r"((int)on), "n"(IMM)
               : "memory");
}
template <int IMM>
__device__ __forceinline__ void lds32_io(bool on, uint32_t a, float& v) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.s32 p, %2, 0;\n\t@p ld.shared.f32 %0, [%1+%3];\n\t}" : "+f"(v) : "r"(a), "r"((int)on), "n"(IMM)
               : "memory");
}

// ---- publish: the values the neighbouring warp will want, before this set's registers are shuffled
// UP = false: consumers take from higher blocks, so a warp publishes its FIRST k values per offset;
// UP = true: its LAST k values.  k = o * ad (ad = |stride difference|).
template <int NG, int NS, bool UP>
__device__ __forceinline__ void pipe_publish(const float2 (&V)[NS][NG], int ad, const PipeHalo& h, int lane) {
  static_for<0, NS*(NG - 1)>([&](auto ic) {
    constexpr int idx = decltype(ic)::value;
    constexpr int s = idx / (NG - 1), o = idx % (NG - 1) + 1;
    constexpr int OFF = idx * (int)kPipeSo;
    const int k = o * ad;
    if (!UP) {
      sts64_io<OFF>(2 * lane < k, h.mine8, V[s][o].x, V[s][o].y);
    } else {
      const int kb = (64 - k) & ~1;  // first published index, rounded down to a pair
      sts64_io<OFF>(2 * lane >= kb, h.mine8 - 4u * (uint32_t)kb, V[s][o].x, V[s][o].y);
    }
  });
}

// ---- in-warp part of the shift (results for lanes whose source is in another warp are garbage
// until pipe_fetch has run)
template <int NG, int NS, bool UP, bool UNIT>
__device__ __forceinline__ void pipe_shuffle(float2 (&V)[NS][NG], int ad) {
#pragma unroll
  for (int s = 0; s < NS; ++s) {
#pragma unroll
    for (int o = 1; o < NG; ++o) {
      const float2 v = V[s][o];
      float2 n;
      if (UNIT && (o & 1)) {  // k = o odd: halves swap
        if (!UP) {
          n.x = (o >> 1) > 0 ? __shfl_down_sync(0xffffffffu, v.y, o >> 1) : v.y;
          n.y = __shfl_down_sync(0xffffffffu, v.x, (o + 1) >> 1);
        } else {
          n.x = __shfl_up_sync(0xffffffffu, v.y, (o + 1) >> 1);
          n.y = (o >> 1) > 0 ? __shfl_up_sync(0xffffffffu, v.x, o >> 1) : v.x;
        }
      } else {
        const int q = UNIT ? (o >> 1) : (o * ad) >> 1;
        if (!UP) {
          n.x = __shfl_down_sync(0xffffffffu, v.x, q);
          n.y = __shfl_down_sync(0xffffffffu, v.y, q);
        } else {
          n.x = __shfl_up_sync(0xffffffffu, v.x, q);
          n.y = __shfl_up_sync(0xffffffffu, v.y, q);
        }
      }
      V[s][o] = n;
    }
  }
}

// ---- halo part of the shift (after the barrier that follows the neighbours' pipe_publish)
template <int NG, int NS, bool UP, bool UNIT>
__device__ __forceinline__ void pipe_fetch(float2 (&V)[NS][NG], int ad, const PipeHalo& h, int lane) {
  static_for<0, NS*(NG - 1)>([&](auto ic) {
    constexpr int idx = decltype(ic)::value;
    constexpr int s = idx / (NG - 1), o = idx % (NG - 1) + 1;
    constexpr int OFF = idx * (int)kPipeSo;
    if constexpr (UNIT && (o & 1)) {
      // k = o odd.  down: x <- index 2L + k, y <- 2L + k + 1 of the chunk, minus 64 in the upper warp's halo.
      //            up:   x <- 2L - k, y <- 2L + 1 - k, plus 64; the lower warp's halo starts at kb = 63 - k.
      if (!UP) {
        constexpr int qx = o >> 1, qy = (o + 1) >> 1;
        lds32_io<OFF + 4 * o>(lane + qx >= 32, h.up8m, V[s][o].x);
        lds32_io<OFF + 4 * (o + 1)>(lane + qy >= 32, h.up8m, V[s][o].y);
      } else {
        constexpr int qx = (o + 1) >> 1, qy = o >> 1;
        lds32_io<OFF + 4>(lane < qx, h.dn8, V[s][o].x);
        lds32_io<OFF + 8>(lane < qy, h.dn8, V[s][o].y);
      }
    } else {
      const int q = UNIT ? (o >> 1) : (o * ad) >> 1;
      if (!UP) {
        lds64_io<OFF>(lane + q >= 32, h.up8m + 8u * (uint32_t)q, V[s][o]);
      } else {
        lds64_io<OFF>(lane < q, h.dn8, V[s][o]);
      }
    }
  });
}

// Whole shift of both sets with its own barriers (start and end of a tile, where nothing overlaps).
template <int NG, int NS>
__device__ __forceinline__ void pipe_exchange_both(float2 (&VA)[NS][NG], float2 (&VB)[NS][NG], int delta, const PipeHalo& ha,
                                                   const PipeHalo& hb, int lane) {
  if (delta == 0) return;
  const int ad = delta < 0 ? -delta : delta;
  if (delta > 0) {
    pipe_publish<NG, NS, false>(VA, ad, ha, lane);
    pipe_publish<NG, NS, false>(VB, ad, hb, lane);
    __syncthreads();
    if (ad == 1) {
      pipe_shuffle<NG, NS, false, true>(VA, ad); pipe_shuffle<NG, NS, false, true>(VB, ad);
      pipe_fetch<NG, NS, false, true>(VA, ad, ha, lane); pipe_fetch<NG, NS, false, true>(VB, ad, hb, lane);
    } else {
      pipe_shuffle<NG, NS, false, false>(VA, ad); pipe_shuffle<NG, NS, false, false>(VB, ad);
      pipe_fetch<NG, NS, false, false>(VA, ad, ha, lane); pipe_fetch<NG, NS, false, false>(VB, ad, hb, lane);
    }
  } else {
    pipe_publish<NG, NS, true>(VA, ad, ha, lane);
    pipe_publish<NG, NS, true>(VB, ad, hb, lane);
    __syncthreads();
    if (ad == 1) {
      pipe_shuffle<NG, NS, true, true>(VA, ad); pipe_shuffle<NG, NS, true, true>(VB, ad);
      pipe_fetch<NG, NS, true, true>(VA, ad, ha, lane); pipe_fetch<NG, NS, true, true>(VB, ad, hb, lane);
    } else {
      pipe_shuffle<NG, NS, true, false>(VA, ad); pipe_shuffle<NG, NS, true, false>(VB, ad);
      pipe_fetch<NG, NS, true, false>(VA, ad, ha, lane); pipe_fetch<NG, NS, true, false>(VB, ad, hb, lane);
    }
  }
  __syncthreads();  // the halo may be overwritten again
}

// a set's 2*NG contiguous positions of one stream <-> its register pairs (one 16-byte slot per group
// for fp32, one for both groups with bf16)
template <int NG, typename T>
__device__ __forceinline__ void pipe_ld_native(const T* chunk, float2 (&Sv)[NG], int t) {
  float2 tmp[1][NG];
  lane_ld_native<NG, 2, T>(chunk, tmp, t);
#pragma unroll
  for (int o = 0; o < NG; ++o) Sv[o] = tmp[0][o];
}
template <int NG, typename T>
__device__ __forceinline__ void pipe_st_native(T* chunk, const float2 (&Sv)[NG], int t) {
  float2 tmp[1][NG];
#pragma unroll
  for (int o = 0; o < NG; ++o) tmp[0][o] = Sv[o];
  lane_st_native<NG, 2, T>(chunk, tmp, t);
}

__device__ __forceinline__ void pipe_halo_init(PipeHalo& h, uint32_t base, uint32_t warp_bytes, int vw, int nvw, int row_first,
                                               int lane) {
  // vw: virtual warp within the row (0 .. nvw-1, set A first); row_first: first virtual warp of the row in the CTA
  const int up = vw + 1 == nvw ? 0 : vw + 1, dn = vw == 0 ? nvw - 1 : vw - 1;
  h.mine8 = base + (uint32_t)(row_first + vw) * warp_bytes + 8u * (uint32_t)lane;
  h.up8m = base + (uint32_t)(row_first + up) * warp_bytes + 8u * (uint32_t)lane - 256u;
  h.dn8 = base + (uint32_t)(row_first + dn) * warp_bytes + 8u * (uint32_t)lane;
}

// ------------------------------------------------------------------------------------------ forward
template <int NG, int ACT, typename T, int MAXT, int MINB>
__global__ void __launch_bounds__(MAXT, MINB) lanep_fwd_kernel(const LaneParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  using F = ActForm<ACT>;
  static_assert(NG == 4, "two sets of one register pair per offset");
  const int tid = threadIdx.x, nthr = blockDim.x;
  const int lane = tid & 31;
  const int N = p.N, R = p.R, L = p.L, TPR = p.tpr;
  const int RN = R * N, NH = N >> 1;
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
    mbar_expect_tx(&bar[0], (residual ? 3 : 2) * bytes);
    bulk_g2s(win, gx_in + row0 * N, bytes, &bar[0]);
    bulk_g2s(win + RN, ga_in + row0 * N, bytes, &bar[0]);
    if (residual) bulk_g2s(sres, gx_in + row0 * N, bytes, &bar[0]);
  };

  const int r = tid / TPR, t = tid - r * TPR;  // row of the tile, thread of the row
  const int wpr = TPR >> 5, wr = t >> 5;
  PipeHalo ha, hb;
  pipe_halo_init(ha, smem_u32(smem + p.off_work), p.halo_warp_bytes, wr, 2 * wpr, r * 2 * wpr, lane);
  pipe_halo_init(hb, smem_u32(smem + p.off_work), p.halo_warp_bytes, wpr + wr, 2 * wpr, r * 2 * wpr, lane);
  const int chunkA = r * N + t * (2 * NG);  // set A's positions of the tile; set B's are NH further
  constexpr float sT = (float)F::sT;
  PairW w;
  w.alpha = f2(p.alpha * sT);
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

    float2 VA[2][NG], VB[2][NG];  // x, xa of the two sets
    if (active) {
      pipe_ld_native<NG, T>(win + chunkA, VA[0], t);
      pipe_ld_native<NG, T>(win + RN + chunkA, VA[1], t);
      pipe_ld_native<NG, T>(win + chunkA + NH, VB[0], t);
      pipe_ld_native<NG, T>(win + RN + chunkA + NH, VB[1], t);
    } else {
#pragma unroll
      for (int s = 0; s < 2; ++s)
#pragma unroll
        for (int o = 0; o < NG; ++o) { VA[s][o] = f2(0.0f); VB[s][o] = f2(0.0f); }
    }
    __syncthreads();  // native inputs are in registers; the buffer now serves as halo
    if (tid == 0 && tile + gridDim.x < p.tiles) {  // next tile towards L2 while this one is worked on
      const long long nrow0 = (tile + gridDim.x) * R;
      const int nrows = (int)min((long long)R, p.B - nrow0);
      const uint32_t bytes = (uint32_t)(nrows * N * sizeof(T));
      l2_prefetch(gx_in + nrow0 * N, bytes);
      l2_prefetch(ga_in + nrow0 * N, bytes);
    }

    auto save_ckpt = [&](const float2 (&V)[2][NG], int ck, int set) {
      // order of a stored state: [stream][offset][pair of groups]; set A holds pair t, set B pair m/4 + t
      float2* c = ckpt + (long long)ck * BN + (row0 + r) * N + set * TPR + t;
#pragma unroll
      for (int s = 0; s < 2; ++s)
#pragma unroll
        for (int o = 0; o < NG; ++o) c[(s * NG + o) * (2 * TPR)] = V[s][o];
    };

    // ---- into the first stage's arrangement, then set A runs half a stage ahead of set B
    StageRec rec = recs[0];
    pipe_exchange_both<NG, 2>(VA, VB, rec.s, ha, hb, lane);
    w.owi = f2(rec.owi * sT);
    w.owj = f2(rec.owj * sT);
    lane_forward<NG, ACT>(VA[0], VA[1], w);
    if (rec.ck >= 0 && active) save_ckpt(VA, rec.ck, 0);
    for (int l = 0; l + 1 < L; ++l) {
      const StageRec nxt = recs[l + 1];
      const int ad = nxt.s - rec.s;  // strides grow: shifts towards higher blocks
      // One compile-time variant per kind of shift, each holding the exchange AND the arithmetic, so
      // that the two stay in one basic block.
      auto stage = [&](auto unit_tag) {
        constexpr bool UNIT = decltype(unit_tag)::value;
        // block A: A leaves stage l; B computes stage l
        pipe_publish<NG, 2, false>(VA, ad, ha, lane);
        pipe_shuffle<NG, 2, false, UNIT>(VA, ad);
        lane_forward<NG, ACT>(VB[0], VB[1], w);
        if (rec.ck >= 0 && active) save_ckpt(VB, rec.ck, 1);
        pipe_publish<NG, 2, false>(VB, ad, hb, lane);
        __syncthreads();
        // block B: A enters stage l + 1; B leaves stage l
        w.owi = f2(nxt.owi * sT);
        w.owj = f2(nxt.owj * sT);
        pipe_fetch<NG, 2, false, UNIT>(VA, ad, ha, lane);
        pipe_shuffle<NG, 2, false, UNIT>(VB, ad);
        lane_forward<NG, ACT>(VA[0], VA[1], w);
        pipe_fetch<NG, 2, false, UNIT>(VB, ad, hb, lane);
        if (nxt.ck >= 0 && active) save_ckpt(VA, nxt.ck, 0);
        __syncthreads();
      };
      if (ad == 1) stage(std::true_type{}); else stage(std::false_type{});
      rec = nxt;
    }
    lane_forward<NG, ACT>(VB[0], VB[1], w);
    if (rec.ck >= 0 && active) save_ckpt(VB, rec.ck, 1);
    pipe_exchange_both<NG, 2>(VA, VB, -rec.s, ha, hb, lane);  // back to stride 0 = native order
    if (active) {
      if (residual) {
        float2 xin[NG];
        pipe_ld_native<NG, T>(sres + chunkA, xin, t);
#pragma unroll
        for (int o = 0; o < NG; ++o) VA[0][o] = fadd2(VA[0][o], xin[o]);
        pipe_ld_native<NG, T>(sres + chunkA + NH, xin, t);
#pragma unroll
        for (int o = 0; o < NG; ++o) VB[0][o] = fadd2(VB[0][o], xin[o]);
      }
      pipe_st_native<NG, T>(win + chunkA, VA[0], t);
      pipe_st_native<NG, T>(win + RN + chunkA, VA[1], t);
      pipe_st_native<NG, T>(win + chunkA + NH, VB[0], t);
      pipe_st_native<NG, T>(win + RN + chunkA + NH, VB[1], t);
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
__global__ void __launch_bounds__(MAXT, MINB) lanep_bwd_kernel(const LaneParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  using F = ActForm<ACT>;
  static_assert(NG == 4, "two sets of one register pair per offset");
  const int tid = threadIdx.x, nthr = blockDim.x;
  const int lane = tid & 31, warp = tid >> 5, nwarp = (nthr + 31) >> 5;
  const int N = p.N, R = p.R, L = p.L, TPR = p.tpr;
  const int RN = R * N, NH = N >> 1;
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
  PipeHalo ha, hb;
  pipe_halo_init(ha, smem_u32(smem + p.off_work), p.halo_warp_bytes, wr, 2 * wpr, r * 2 * wpr, lane);
  pipe_halo_init(hb, smem_u32(smem + p.off_work), p.halo_warp_bytes, wpr + wr, 2 * wpr, r * 2 * wpr, lane);
  const int chunkA = r * N + t * (2 * NG);
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

    float2 VA[4][NG], VB[4][NG];  // x, xa, gx, ga of the two sets
#pragma unroll
    for (int s = 0; s < 4; ++s)
#pragma unroll
      for (int o = 0; o < NG; ++o) { VA[s][o] = f2(0.0f); VB[s][o] = f2(0.0f); }
    if (active) {
#pragma unroll
      for (int s = 0; s < 4; ++s)
        if (s >= 2 || !tape) {
          pipe_ld_native<NG, T>(win + s * RN + chunkA, VA[s], t);
          pipe_ld_native<NG, T>(win + s * RN + chunkA + NH, VB[s], t);
        }
    }
    __syncthreads();  // native inputs are in registers; the buffer now serves as halo
    if (tid == 0 && tile + gridDim.x < p.tiles) {  // next tile towards L2 while this one is worked on
      const long long nrow0 = (tile + gridDim.x) * R;
      const int nrows = (int)min((long long)R, p.B - nrow0);
      const uint32_t bytes = (uint32_t)(nrows * N * sizeof(T));
#pragma unroll
      for (int q = 0; q < 4; ++q)
        if (q >= 2 || !tape) l2_prefetch(g_in[q] + nrow0 * N, bytes);
      for (uint32_t k = 0; k < n_ck; ++k) l2_prefetch(ckpt + (long long)k * BN + nrow0 * N, (uint32_t)(nrows * N * sizeof(float2)));
    }

    auto load_ckpt = [&](float2 (&V)[4][NG], int ck, int set) {  // a state saved after a stage replaces the rebuilt one
      const float2* c = sck + ck * RN + r * N + set * TPR + t;
#pragma unroll
      for (int s = 0; s < 2; ++s)
#pragma unroll
        for (int o = 0; o < NG; ++o) V[s][o] = c[(s * NG + o) * (2 * TPR)];
    };
    auto set_w = [&](const StageRec& rc) {
      w.owi = f2(rc.owi);
      w.owj = f2(rc.owj);
      w.owjs = f2(rc.owj * sT);
    };
    auto reduce_dw = [&](float2 dwi, float2 dwj, int l) {  // fixed-order warp tree, one slot per warp and stage
      const float di = (dwi.x + dwi.y) * dsi, dj = (dwj.x + dwj.y) * dsj;
      const bool hi = (lane & 16) != 0;
      const float give = hi ? di : dj;
      float keep = hi ? dj : di;
      keep += __shfl_xor_sync(0xffffffffu, give, 16);
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) keep += __shfl_xor_sync(0xffffffffu, keep, o);
      if ((lane & 15) == 0 && active) red[(l * nwarp + warp) * 2 + (hi ? 1 : 0)] += keep;
    };

    // ---- into the last stage's arrangement, then set A runs half a stage ahead of set B
    StageRec rec = recs[L - 1];
    pipe_exchange_both<NG, 4>(VA, VB, rec.s, ha, hb, lane);
    set_w(rec);
    if (rec.ck >= 0) { load_ckpt(VA, rec.ck, 0); load_ckpt(VB, rec.ck, 1); }
    float2 dwi = f2(0.0f), dwj = f2(0.0f);
    lane_backward<NG, ACT>(VA[0], VA[1], VA[2], VA[3], w, dwi, dwj);
    for (int l = L - 1; l > 0; --l) {
      const StageRec nxt = recs[l - 1];
      const int ad = rec.s - nxt.s;  // strides shrink: shifts towards lower blocks
      // One compile-time variant per kind of shift, each holding the exchange AND the arithmetic, so
      // that the two stay in one basic block.
      auto stage = [&](auto unit_tag) {
        constexpr bool UNIT = decltype(unit_tag)::value;
        // block A: A leaves stage l; B computes stage l
        pipe_publish<NG, 4, true>(VA, ad, ha, lane);
        pipe_shuffle<NG, 4, true, UNIT>(VA, ad);
        lane_backward<NG, ACT>(VB[0], VB[1], VB[2], VB[3], w, dwi, dwj);
        reduce_dw(dwi, dwj, l);
        pipe_publish<NG, 4, true>(VB, ad, hb, lane);
        __syncthreads();
        // block B: A enters stage l - 1; B leaves stage l
        set_w(nxt);
        dwi = f2(0.0f); dwj = f2(0.0f);
        pipe_fetch<NG, 4, true, UNIT>(VA, ad, ha, lane);
        if (nxt.ck >= 0) load_ckpt(VA, nxt.ck, 0);
        pipe_shuffle<NG, 4, true, UNIT>(VB, ad);
        lane_backward<NG, ACT>(VA[0], VA[1], VA[2], VA[3], w, dwi, dwj);
        pipe_fetch<NG, 4, true, UNIT>(VB, ad, hb, lane);
        if (nxt.ck >= 0) load_ckpt(VB, nxt.ck, 1);
        __syncthreads();
      };
      if (ad == 1) stage(std::true_type{}); else stage(std::false_type{});
      rec = nxt;
    }
    lane_backward<NG, ACT>(VB[0], VB[1], VB[2], VB[3], w, dwi, dwj);
    reduce_dw(dwi, dwj, 0);
    pipe_exchange_both<NG, 4>(VA, VB, -rec.s, ha, hb, lane);  // back to stride 0 = native order
    if (active) {
      if (residual) {
        float2 gin[NG];
        pipe_ld_native<NG, T>(sdy + chunkA, gin, t);
#pragma unroll
        for (int o = 0; o < NG; ++o) VA[2][o] = fadd2(VA[2][o], gin[o]);
        pipe_ld_native<NG, T>(sdy + chunkA + NH, gin, t);
#pragma unroll
        for (int o = 0; o < NG; ++o) VB[2][o] = fadd2(VB[2][o], gin[o]);
      }
      pipe_st_native<NG, T>(win + chunkA, VA[2], t);
      pipe_st_native<NG, T>(win + RN + chunkA, VA[3], t);
      pipe_st_native<NG, T>(win + chunkA + NH, VB[2], t);
      pipe_st_native<NG, T>(win + RN + chunkA + NH, VB[3], t);
      if (want_rec) {
        pipe_st_native<NG, T>(win + 2 * RN + chunkA, VA[0], t);
        pipe_st_native<NG, T>(win + 3 * RN + chunkA, VA[1], t);
        pipe_st_native<NG, T>(win + 2 * RN + chunkA + NH, VB[0], t);
        pipe_st_native<NG, T>(win + 3 * RN + chunkA + NH, VB[1], t);
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
