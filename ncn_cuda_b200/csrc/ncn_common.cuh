// Shared device helpers for the NCN kernels (sm_100a only).
//
// The math follows the reference's torch implementation:
//   stage index map   torch_ref/ncn_pytorch.py:12-41
//   recurrence step   torch_ref/ncn_pytorch.py:74-94
//   activation codes  ncn_cuda/ncn_pytorch_wrapper_v2.py:111  (0 tanh, 1 relu, 2 sigmoid, else linear)
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ncn {

// The two-stream mixing constant is a literal 0.9 everywhere in the reference
// (torch_ref/ncn_pytorch.py:89); (1 - 0.9) is formed in double and rounded to fp32 there.
constexpr float kM = 0.9f;
constexpr float kC = 0.1f;  // fp32(1 - 0.9)
constexpr float kInvM = 1.0f / 0.9f;
constexpr float kCoverM = 0.1f / 0.9f;

enum Act : int { ACT_TANH = 0, ACT_RELU = 1, ACT_SIGMOID = 2, ACT_LINEAR = 3 };
enum DType : int { DT_F32 = 0, DT_BF16 = 1 };

// flags of the fused row kernels
enum : int {
  F_RESIDUAL = 1,   // forward: y = x + net(x); backward: dx = dx_net + dy
  F_RECOMPUTE = 2,  // backward: inputs are the net INPUT; replay the forward, then walk back
};

// error codes stored in the device status word by a kernel that gave up a wait
enum : int { DEV_OK = 0, DEV_WAIT_TIMEOUT = 1 };

// ------------------------------------------------------------------ PTX
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after ~2^22 polls (each poll may itself suspend for a
// hardware-defined time), so a copy that never lands cannot hang the GPU.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
  for (uint32_t it = 0; it < (1u << 22); ++it) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  return false;
}
// 1-D bulk copy global -> shared through the TMA unit; completion is counted on `bar`.
// Both addresses 16-byte aligned, size a multiple of 16 bytes.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst_smem)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
// 1-D bulk copy shared -> global (bulk async-group completion).
__device__ __forceinline__ void bulk_s2g(void* dst, const void* src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(smem_u32(src_smem)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// generic-proxy writes to shared memory -> visible to the async proxy (TMA store)
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float rcp_approx(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// ------------------------------------------------------------------ storage types
template <typename T>
struct Store;
template <>
struct Store<float> {
  static __device__ __forceinline__ float ld(const float* p) { return *p; }
  static __device__ __forceinline__ void st(float* p, float v) { *p = v; }
};
template <>
struct Store<__nv_bfloat16> {
  static __device__ __forceinline__ float ld(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  static __device__ __forceinline__ void st(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
};

// NG contiguous elements, vectorised as wide as the group allows.
template <int NG>
__device__ __forceinline__ void ld_vec(const float* p, float (&v)[NG]) {
  if constexpr (NG % 4 == 0) {
#pragma unroll
    for (int q = 0; q < NG / 4; ++q) {
      float4 t = reinterpret_cast<const float4*>(p)[q];
      v[4 * q] = t.x; v[4 * q + 1] = t.y; v[4 * q + 2] = t.z; v[4 * q + 3] = t.w;
    }
  } else if constexpr (NG == 2) {
    float2 t = *reinterpret_cast<const float2*>(p);
    v[0] = t.x; v[1] = t.y;
  } else {
#pragma unroll
    for (int q = 0; q < NG; ++q) v[q] = p[q];
  }
}
template <int NG>
__device__ __forceinline__ void st_vec(float* p, const float (&v)[NG]) {
  if constexpr (NG % 4 == 0) {
#pragma unroll
    for (int q = 0; q < NG / 4; ++q)
      reinterpret_cast<float4*>(p)[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
  } else if constexpr (NG == 2) {
    *reinterpret_cast<float2*>(p) = make_float2(v[0], v[1]);
  } else {
#pragma unroll
    for (int q = 0; q < NG; ++q) p[q] = v[q];
  }
}
template <int NG>
__device__ __forceinline__ void ld_vec(const __nv_bfloat16* p, float (&v)[NG]) {
  if constexpr (NG % 8 == 0) {
#pragma unroll
    for (int q = 0; q < NG / 8; ++q) {
      uint4 t = reinterpret_cast<const uint4*>(p)[q];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&t);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float2 f = __bfloat1622float2(h[e]);
        v[8 * q + 2 * e] = f.x; v[8 * q + 2 * e + 1] = f.y;
      }
    }
  } else if constexpr (NG == 4) {
    uint2 t = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&t);
    float2 f0 = __bfloat1622float2(h[0]), f1 = __bfloat1622float2(h[1]);
    v[0] = f0.x; v[1] = f0.y; v[2] = f1.x; v[3] = f1.y;
  } else if constexpr (NG == 2) {
    float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
    v[0] = f.x; v[1] = f.y;
  } else {
#pragma unroll
    for (int q = 0; q < NG; ++q) v[q] = __bfloat162float(p[q]);
  }
}
template <int NG>
__device__ __forceinline__ void st_vec(__nv_bfloat16* p, const float (&v)[NG]) {
  if constexpr (NG % 8 == 0) {
#pragma unroll
    for (int q = 0; q < NG / 8; ++q) {
      uint4 t;
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&t);
#pragma unroll
      for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(v[8 * q + 2 * e], v[8 * q + 2 * e + 1]);
      reinterpret_cast<uint4*>(p)[q] = t;
    }
  } else if constexpr (NG == 4) {
    uint2 t;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&t);
    h[0] = __floats2bfloat162_rn(v[0], v[1]);
    h[1] = __floats2bfloat162_rn(v[2], v[3]);
    *reinterpret_cast<uint2*>(p) = t;
  } else if constexpr (NG == 2) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(v[0], v[1]);
  } else {
#pragma unroll
    for (int q = 0; q < NG; ++q) p[q] = __float2bfloat16_rn(v[q]);
  }
}

// ------------------------------------------------------------------ activations
// act(T) and its derivative expressed through (T, F).
template <int ACT>
__device__ __forceinline__ float act_fwd(float t) {
  if constexpr (ACT == ACT_TANH) {
    // tanh(t) = 1 - 2 / (exp(2t) + 1); absolute error ~2e-7 (ex2 and rcp are ~1-2 ulp).
    float e = ex2_approx(t * 2.8853900817779268f);
    return fmaf(-2.0f, rcp_approx(e + 1.0f), 1.0f);
  } else if constexpr (ACT == ACT_RELU) {
    return fmaxf(t, 0.0f);
  } else if constexpr (ACT == ACT_SIGMOID) {
    float e = ex2_approx(t * -1.4426950408889634f);
    return rcp_approx(e + 1.0f);
  } else {
    return t;
  }
}
template <int ACT>
__device__ __forceinline__ float act_grad(float t, float f) {
  if constexpr (ACT == ACT_TANH) {
    return fmaf(-f, f, 1.0f);
  } else if constexpr (ACT == ACT_RELU) {
    return t > 0.0f ? 1.0f : 0.0f;
  } else if constexpr (ACT == ACT_SIGMOID) {
    return f * (1.0f - f);
  } else {
    return 1.0f;
  }
}

// ------------------------------------------------------------------ index map
// stride of a stage in blocks: 0 for stage 0, else 2^(stage-1) mod m  (torch_ref/ncn_pytorch.py:38)
__host__ __device__ __forceinline__ int stage_stride(int stage, int m) {
  if (stage <= 0) return 0;
  const int e = stage - 1;
  if (e < 62) return static_cast<int>((1ULL << e) % static_cast<unsigned long long>(m));
  // 2^e mod m by repeated doubling for very deep stacks
  unsigned long long r = (1ULL << 61) % static_cast<unsigned long long>(m);
  for (int k = 61; k < e; ++k) r = (r * 2ULL) % static_cast<unsigned long long>(m);
  return static_cast<int>(r);
}

// ------------------------------------------------------------------ step math (one feature per position)
// One group of NG positions, all NG steps.  T_i = alpha x_i + (1-alpha)(x_i wi + xj wj) xj is
// evaluated as x_i * p + q with p = alpha + (1-alpha) wi xj, q = (1-alpha) wj xj^2.
template <int NG, int ACT>
__device__ __forceinline__ void group_forward(float (&x)[NG], float (&a)[NG], float wi_s, float wj_s, float alpha) {
  // wi_s = (1-alpha) wi, wj_s = (1-alpha) wj
#pragma unroll
  for (int j = 0; j < NG; ++j) {
    const float xj = x[j];
    if constexpr (ACT == ACT_TANH) {
      constexpr float k2 = 2.8853900817779268f;  // 2 log2(e)
      const float p = fmaf(wi_s, xj, alpha) * k2;
      const float q = (wj_s * xj) * xj * k2;
#pragma unroll
      for (int i = 0; i < NG; ++i) {
        const float e = ex2_approx(fmaf(x[i], p, q));
        const float r = rcp_approx(e + 1.0f);
        // a' = m a + c (1 - 2r)
        a[i] = fmaf(r, -2.0f * kC, fmaf(a[i], kM, kC));
        x[i] = fmaf(a[i], kC, x[i] * kM);
      }
    } else {
      const float p = fmaf(wi_s, xj, alpha);
      const float q = (wj_s * xj) * xj;
#pragma unroll
      for (int i = 0; i < NG; ++i) {
        const float f = act_fwd<ACT>(fmaf(x[i], p, q));
        a[i] = fmaf(f, kC, a[i] * kM);
        x[i] = fmaf(a[i], kC, x[i] * kM);
      }
    }
  }
}

// Reverse sweep of one group: on entry (x, a) hold the group's OUTPUT and (gx, ga) the incoming
// cotangents; on exit they hold the group's input and the outgoing cotangents.  dwi/dwj are
// incremented by the group's weight-gradient contribution.
// Per step (torch_ref/ncn_pytorch_invertible.py:97-111 inverse, :164-172 gradient):
//   x = (y - c ya)/m ; F = act(T(x)) ; a = (ya - c F)/m
//   gA' = ga + c gy ; gT = c gA' act'(T) ; ga <- m gA'
//   gx_i = m gy_i + gT_i p ;  gx_j += (1-alpha) sum_i gT_i (x_i wi + 2 wj xj)
//   dWi += (1-alpha) xj sum_i gT_i x_i ;  dWj += (1-alpha) xj^2 sum_i gT_i
template <int NG, int ACT>
__device__ __forceinline__ void group_backward(float (&x)[NG], float (&a)[NG], float (&gx)[NG], float (&ga)[NG],
                                               float wi, float wj, float alpha, float oma, float& dwi, float& dwj) {
#pragma unroll
  for (int j = NG - 1; j >= 0; --j) {
#pragma unroll
    for (int i = 0; i < NG; ++i) x[i] = fmaf(a[i], -kCoverM, x[i] * kInvM);
    const float xj = x[j];
    const float p = fmaf(oma * wi, xj, alpha);
    const float q = (oma * wj * xj) * xj;
    float accI = 0.0f, accS = 0.0f;
#pragma unroll
    for (int i = 0; i < NG; ++i) {
      float dact;
      if constexpr (ACT == ACT_TANH) {
        constexpr float k2 = 2.8853900817779268f;
        const float e = ex2_approx(fmaf(x[i], p * k2, q * k2));
        const float r = rcp_approx(e + 1.0f);
        // a = (ya - c (1 - 2r)) / m ; act' = 1 - F^2 = 4 (r - r^2)
        a[i] = fmaf(r, 2.0f * kCoverM, fmaf(a[i], kInvM, -kCoverM));
        dact = 4.0f * fmaf(-r, r, r);
      } else {
        const float t = fmaf(x[i], p, q);
        const float f = act_fwd<ACT>(t);
        a[i] = fmaf(f, -kCoverM, a[i] * kInvM);
        dact = act_grad<ACT>(t, f);
      }
      const float gAp = fmaf(kC, gx[i], ga[i]);
      const float gT = (kC * gAp) * dact;
      ga[i] = kM * gAp;
      gx[i] = fmaf(gT, p, kM * gx[i]);
      accI = fmaf(gT, x[i], accI);
      accS += gT;
    }
    // sum_i gT_i (x_i wi + 2 wj xj) = wi accI + 2 wj xj accS
    const float oxj = oma * xj;
    gx[j] = fmaf(oma, fmaf(wi, accI, 2.0f * wj * xj * accS), gx[j]);
    dwi = fmaf(oxj, accI, dwi);
    dwj = fmaf(oxj * xj, accS, dwj);
  }
}

// ------------------------------------------------------------------ parameter block of the fused row kernels
struct RowsParams {
  const void* in[4];   // fwd: x, xa, -, - ; bwd: (y | x), (ya | xa), dy, dya
  void* out[4];        // fwd: y, ya, -, - ; bwd: dx, dxa, x_rec (or null), xa_rec (or null)
  float* ckpt;         // [K][2][B*N] fp32 stage-boundary states (stage-local layout), or null
  const float* W;      // [L][2]
  float* partials;     // bwd: [gridDim.x][L][2]
  int* status;         // device status word
  long long B;
  long long tiles;
  int N, m, R, L, l0, ckpt_every, flags, nbuf;
  float alpha, oma;
  uint32_t off_in[2];  // byte offsets into dynamic shared memory
  uint32_t off_work, off_out, off_ckpt, off_red, off_w, off_bar;
  uint32_t n_ckpt_slots;  // checkpoints staged in shared memory per tile (0 = read them from global)
};

constexpr uint32_t kNoOff = 0xFFFFFFFFu;

}  // namespace ncn
