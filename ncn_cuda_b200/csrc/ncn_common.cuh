// Shared device helpers for the NCN kernels (sm_100a only).
//
// The math follows the reference's torch implementation:
//   stage index map   torch_ref/ncn_pytorch.py:12-41
//   recurrence step   torch_ref/ncn_pytorch.py:74-94
//   activation codes  ncn_cuda/ncn_pytorch_wrapper_v2.py:111  (0 tanh, 1 relu, 2 sigmoid, else linear);
//                     3 = leaky-relu, slope 0.01 (torch_ref/ncn_pytorch_invertible.py:39-44, ncn_triton/ncn_triton.py:22-28)
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ncn {

// Host side: cudaFuncSetAttribute(MaxDynamicSharedMemorySize) only when this process has not yet granted the
// kernel at least `smem` bytes on the current device; repeated on every launch the call costs about a
// microsecond.  One SmemGrant per kernel (a function-local static of its launcher); races between threads
// are benign (at worst one more call).
struct SmemGrant {
  int bytes[16] = {};
};
template <typename K>
inline cudaError_t grant_smem(SmemGrant& g, K kernel, size_t smem) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) dev = -1;
  if (dev >= 0 && dev < 16 && g.bytes[dev] >= (int)smem) return cudaSuccess;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e == cudaSuccess && dev >= 0 && dev < 16) g.bytes[dev] = (int)smem;
  return e;
}


// The two-stream mixing constant is a literal 0.9 everywhere in the reference
// (torch_ref/ncn_pytorch.py:89); (1 - 0.9) is formed in double and rounded to fp32 there.
constexpr float kM = 0.9f;
constexpr float kC = 0.1f;  // fp32(1 - 0.9)
constexpr float kInvM = 1.0f / 0.9f;
constexpr float kCoverM = 0.1f / 0.9f;

// ACT_TANH_FAST is internal: tanh through the one-instruction tanh.approx.f32 (relative error 2^-11),
// used for bf16 storage, whose 2e-2 tolerance it does not threaten; it halves the special-function work.
// ACT_LEAKY runs on the shared-memory stage kernels only (ncn_generic.cuh).
enum Act : int { ACT_TANH = 0, ACT_RELU = 1, ACT_SIGMOID = 2, ACT_LINEAR = 3, ACT_TANH_FAST = 4, ACT_LEAKY = 5 };
enum DType : int { DT_F32 = 0, DT_BF16 = 1 };

// flags of the fused row kernels
enum : int {
  F_RESIDUAL = 1,   // forward: y = x + net(x); backward: dx = dx_net + dy
  F_RECOMPUTE = 2,  // backward: inputs are the net INPUT; replay the forward, then walk back
  F_RED_THREAD = 4, // backward (set by the launch plan): dW partial slots per thread instead of per warp
  F_TAPE = 8,       // the state after the LAST stage is checkpointed too (fp32); the backward starts from it
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
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, uint32_t tries = 1u << 22) {
  for (uint32_t it = 0; it < tries; ++it) {
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
__device__ __forceinline__ float tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
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
  } else if constexpr (ACT == ACT_LEAKY) {
    return t >= 0.0f ? t : 0.01f * t;
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
  } else if constexpr (ACT == ACT_LEAKY) {
    return t >= 0.0f ? 1.0f : 0.01f;
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
//
// One step of the reference (torch_ref/ncn_pytorch.py:74-94), per position i of a group:
//     T_i = alpha x_i + (1-alpha)(x_i wi + xj wj) xj ;  F = act(T)
//     a_i <- m a_i + c F ;  x_i <- m x_i + c a_i                     (m = 0.9, c = 0.1)
// Every position takes exactly one such step per j, so the factors of m can be carried as a
// scale that is uniform over the group: with k steps done, x = m^k (X + D_k), a = m^k (A + C_k),
// where X, A are the per-position registers and C_k, D_k compile-time constants (non-zero only
// when the activation has a constant part, F = f0 + f1 r).  In these variables a step is
//     X-part of T:  Ts = X P + Q   (P, Q formed once per step from xj)
//     A <- A + (c f1 / m^(k+1)) r ;  X <- X + c A
// i.e. four FMA-pipe instructions and the activation's special-function instructions per
// position and step.  After the NG steps of a stage the true values are restored.
constexpr double kMd = 0.89999997615814208984375;    // (double)0.9f
constexpr double kCd = 0.100000001490116119384765625;  // (double)0.1f

constexpr double cpow(double b, int e) {
  double r = 1.0;
  for (int i = 0; i < e; ++i) r *= b;
  return r;
}

// The per-position arithmetic is issued two positions at a time with the packed fp32
// instructions of sm_100 (fma.rn.f32x2 / add.f32x2 / mul.f32x2 through __ffma2_rn, __fadd2_rn,
// __fmul2_rn): the kernels are bound by instruction issue next to the special-function unit, and
// a packed instruction does the work of two in one issue slot.
__device__ __forceinline__ float2 f2(float v) { return make_float2(v, v); }

// Activation written as F = f0 + f1 * r(Ts), Ts = sT * T, and act'(T) = ds * u(Ts, r).
template <int ACT>
struct ActForm;
template <>
struct ActForm<ACT_TANH> {  // tanh T = 1 - 2 / (2^(2 log2e T) + 1) ; 1 - F^2 = 4 (r - r^2)
  static constexpr double sT = 2.8853900817779268, f0 = 1.0, f1 = -2.0, ds = 4.0;
  static __device__ __forceinline__ float2 r(float2 ts) {
    const float2 d = __fadd2_rn(make_float2(ex2_approx(ts.x), ex2_approx(ts.y)), f2(1.0f));
    return make_float2(rcp_approx(d.x), rcp_approx(d.y));
  }
  static __device__ __forceinline__ float2 gt(float2 g, float2, float2 r) {
    return __fmul2_rn(g, __ffma2_rn(make_float2(-r.x, -r.y), r, r));
  }
  // The same value with the reciprocal by Newton's iteration on the FMA pipe instead of the
  // special-function unit (start: exponent/mantissa trick, 12 % off; three steps square that to
  // below 1e-7).  For kernels that the special-function unit bounds while the FMA pipe idles.
  static __device__ __forceinline__ float2 r_fma(float2 ts) {
    const float2 d = __fadd2_rn(make_float2(ex2_approx(ts.x), ex2_approx(ts.y)), f2(1.0f));
    float2 y = make_float2(__int_as_float(0x7EF311C3 - __float_as_int(d.x)), __int_as_float(0x7EF311C3 - __float_as_int(d.y)));
    const float2 nd = make_float2(-d.x, -d.y);
#pragma unroll
    for (int it = 0; it < 3; ++it) y = __ffma2_rn(y, __ffma2_rn(nd, y, f2(1.0f)), y);  // y += y (1 - d y)
    return y;
  }
};
template <>
struct ActForm<ACT_SIGMOID> {  // 1 / (1 + 2^(-log2e T)) ; F' = F (1 - F)
  static constexpr double sT = -1.4426950408889634, f0 = 0.0, f1 = 1.0, ds = 1.0;
  static __device__ __forceinline__ float2 r(float2 ts) { return ActForm<ACT_TANH>::r(ts); }
  static __device__ __forceinline__ float2 gt(float2 g, float2 ts, float2 r) { return ActForm<ACT_TANH>::gt(g, ts, r); }
};
template <>
struct ActForm<ACT_TANH_FAST> {  // F = tanh.approx(T) ; F' = 1 - F^2
  static constexpr double sT = 1.0, f0 = 0.0, f1 = 1.0, ds = 1.0;
  static __device__ __forceinline__ float2 r(float2 ts) { return make_float2(tanh_approx(ts.x), tanh_approx(ts.y)); }
  static __device__ __forceinline__ float2 gt(float2 g, float2, float2 r) {
    return __fmul2_rn(g, __ffma2_rn(make_float2(-r.x, -r.y), r, f2(1.0f)));
  }
};
template <>
struct ActForm<ACT_RELU> {
  static constexpr double sT = 1.0, f0 = 0.0, f1 = 1.0, ds = 1.0;
  static __device__ __forceinline__ float2 r(float2 ts) { return make_float2(fmaxf(ts.x, 0.0f), fmaxf(ts.y, 0.0f)); }
  static __device__ __forceinline__ float2 gt(float2 g, float2 ts, float2) {
    return make_float2(ts.x > 0.0f ? g.x : 0.0f, ts.y > 0.0f ? g.y : 0.0f);
  }
};
template <>
struct ActForm<ACT_LINEAR> {
  static constexpr double sT = 1.0, f0 = 0.0, f1 = 1.0, ds = 1.0;
  static __device__ __forceinline__ float2 r(float2 ts) { return ts; }
  static __device__ __forceinline__ float2 gt(float2 g, float2, float2) { return g; }
};

// r = 1 / (1 + 2^ts) for all N values of an array at once (the positions of a group, or the features of a
// position).
// BATCH: reciprocals taken from one special-function reciprocal of the product of BATCH values
// (4: 1.25, 2: 1.5, 1: 2 special-function instructions per position and step; the smaller the batch
// the fewer multiplies on the FMA pipe).
template <int ACT, int NG, int BATCH>
__device__ __forceinline__ void act_r_all(const float2 (&ts)[NG], float2 (&r)[NG]) {
  if constexpr (ACT == ACT_TANH || ACT == ACT_SIGMOID) {
    // r_i = 1 / d_i, d_i = 1 + 2^ts_i.  The exponent is capped at 30: beyond it r < 1e-9 (tanh = 1 to the last
    // bit) and the product of four d stays a normal fp32 number, as does its reciprocal.
    float2 d[NG];
#pragma unroll
    for (int i = 0; i < NG; ++i)
      d[i] = __fadd2_rn(make_float2(ex2_approx(fminf(ts[i].x, 30.0f)), ex2_approx(fminf(ts[i].y, 30.0f))), f2(1.0f));
    if constexpr (BATCH == 1) {
#pragma unroll
      for (int i = 0; i < NG; ++i) r[i] = make_float2(rcp_approx(d[i].x), rcp_approx(d[i].y));
    } else if constexpr (NG == 2 || BATCH == 2) {
#pragma unroll
      for (int b = 0; b < NG; b += 2) {
        const float2 P = __fmul2_rn(d[b], d[b + 1]);
        const float2 R = make_float2(rcp_approx(P.x), rcp_approx(P.y));
        r[b] = __fmul2_rn(d[b + 1], R);
        r[b + 1] = __fmul2_rn(d[b], R);
      }
    } else {
#pragma unroll
      for (int b = 0; b < NG; b += 4) {
        const float2 P01 = __fmul2_rn(d[b], d[b + 1]);
        const float2 P23 = __fmul2_rn(d[b + 2], d[b + 3]);
        const float2 PP = __fmul2_rn(P01, P23);
        const float2 R = make_float2(rcp_approx(PP.x), rcp_approx(PP.y));
        const float2 i01 = __fmul2_rn(P23, R);
        const float2 i23 = __fmul2_rn(P01, R);
        r[b] = __fmul2_rn(d[b + 1], i01);
        r[b + 1] = __fmul2_rn(d[b], i01);
        r[b + 2] = __fmul2_rn(d[b + 3], i23);
        r[b + 3] = __fmul2_rn(d[b + 2], i23);
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < NG; ++i) r[i] = ActForm<ACT>::r(ts[i]);
  }
}

// forward offsets after k steps: C_k = sum_{i=1..k} c f0 / m^i ; D_k = sum_{i=1..k} c C_i
constexpr double fwd_C(int k, double f0) {
  double C = 0.0;
  for (int i = 1; i <= k; ++i) C += kCd * f0 / cpow(kMd, i);
  return C;
}
constexpr double fwd_D(int k, double f0) {
  double C = 0.0, D = 0.0;
  for (int i = 1; i <= k; ++i) {
    C += kCd * f0 / cpow(kMd, i);
    D += kCd * C;
  }
  return D;
}
// reverse offsets after k inverse steps: x = m^-k (X + DX_k), a = m^-k (A + CA_k)
//   CA_{k+1} = CA_k - c f0 m^k ;  DX_{k+1} = DX_k - c CA_k
constexpr double bwd_CA(int k, double f0) {
  double CA = 0.0;
  for (int i = 0; i < k; ++i) CA -= kCd * f0 * cpow(kMd, i);
  return CA;
}
constexpr double bwd_DX(int k, double f0) {
  double CA = 0.0, DX = 0.0;
  for (int i = 0; i < k; ++i) {
    DX -= kCd * CA;
    CA -= kCd * f0 * cpow(kMd, i);
  }
  return DX;
}

// weights of one stage as the step code wants them
struct StageW {
  float owi, owj;  // (1-alpha) wi, (1-alpha) wj
  float alpha, oma;
};

template <int NG, int ACT, int J>
struct FwdSteps {
  static __device__ __forceinline__ void run(float2 (&X)[NG / 2], float2 (&A)[NG / 2], float owi_s, float owj_s,
                                             float alpha_s) {
    using F = ActForm<ACT>;
    constexpr float mk = (float)cpow(kMd, J);
    constexpr float mkDk = (float)(cpow(kMd, J) * fwd_D(J, F::f0));
    constexpr float cA = (float)(kCd * F::f1 / cpow(kMd, J + 1));
    const float XJ = (J & 1) ? X[J / 2].y : X[J / 2].x;
    const float xj = fmaf(XJ, mk, mkDk);
    const float pp = fmaf(owi_s, xj, alpha_s);  // sT (alpha + (1-alpha) wi xj)
    const float2 P = f2(pp * mk);
    const float2 Q = f2(fmaf(pp, mkDk, (owj_s * xj) * xj));
#pragma unroll
    for (int i = 0; i < NG / 2; ++i) {
      const float2 r = F::r(__ffma2_rn(X[i], P, Q));
      A[i] = __ffma2_rn(r, f2(cA), A[i]);
      X[i] = __ffma2_rn(A[i], f2(kC), X[i]);
    }
    FwdSteps<NG, ACT, J + 1>::run(X, A, owi_s, owj_s, alpha_s);
  }
};
template <int NG, int ACT>
struct FwdSteps<NG, ACT, NG> {
  static __device__ __forceinline__ void run(float2 (&)[NG / 2], float2 (&)[NG / 2], float, float, float) {}
};

// All NG steps of one group; x, a hold true values on entry and on exit.
template <int NG, int ACT>
__device__ __forceinline__ void group_forward(float (&x)[NG], float (&a)[NG], const StageW& w) {
  static_assert(NG % 2 == 0, "positions are processed in pairs");
  using F = ActForm<ACT>;
  constexpr float sT = (float)F::sT;
  float2 X[NG / 2], A[NG / 2];
#pragma unroll
  for (int i = 0; i < NG / 2; ++i) {
    X[i] = make_float2(x[2 * i], x[2 * i + 1]);
    A[i] = make_float2(a[2 * i], a[2 * i + 1]);
  }
  FwdSteps<NG, ACT, 0>::run(X, A, w.owi * sT, w.owj * sT, w.alpha * sT);
  constexpr float mN = (float)cpow(kMd, NG);
  constexpr float mNC = (float)(cpow(kMd, NG) * fwd_C(NG, F::f0));
  constexpr float mND = (float)(cpow(kMd, NG) * fwd_D(NG, F::f0));
#pragma unroll
  for (int i = 0; i < NG / 2; ++i) {
    const float2 xo = __ffma2_rn(X[i], f2(mN), f2(mND));
    const float2 ao = __ffma2_rn(A[i], f2(mN), f2(mNC));
    x[2 * i] = xo.x; x[2 * i + 1] = xo.y;
    a[2 * i] = ao.x; a[2 * i + 1] = ao.y;
  }
}

// Reverse sweep (torch_ref/ncn_pytorch_invertible.py:97-111 inverse, :164-172 gradient).  With k
// inverse steps done: x = m^-k (X + DX_k), a = m^-k (A + CA_k), gy = m^k H, ga = m^k G.  Per step:
//   X <- X - c A                              (x_prev = (y - c ya)/m)
//   r from Ts = X Ps + Qs ;  A <- A - c f1 m^k r  (a_prev = (ya - c F)/m)
//   G <- G + c H            (gA' = ga + c gy ; ga_prev = m gA')
//   gt = G u                (gT = c ds m^k gt)
//   H <- H + gt (c ds p / m)                  (gx_i = m gy_i + gT_i p)
//   aI += gt X ; aS += gt                     (sums for gx_j, dWi, dWj)
template <int NG, int ACT, int J>
struct BwdSteps {
  static __device__ __forceinline__ void run(float2 (&X)[NG / 2], float2 (&A)[NG / 2], float2 (&H)[NG / 2],
                                             float2 (&G)[NG / 2], const StageW& w, float& dwi, float& dwj) {
    using F = ActForm<ACT>;
    constexpr int k = NG - 1 - J;
    constexpr double mkd = cpow(kMd, k);
    constexpr float imk1 = (float)(1.0 / cpow(kMd, k + 1));
    constexpr float DX1 = (float)bwd_DX(k + 1, F::f0);
    constexpr float imk1DX1 = (float)(bwd_DX(k + 1, F::f0) / cpow(kMd, k + 1));
    constexpr float cAr = (float)(-kCd * F::f1 * mkd);
    constexpr float sTimk1 = (float)(F::sT / cpow(kMd, k + 1));
    constexpr float sT = (float)F::sT;
    constexpr float cdsm = (float)(kCd * F::ds / kMd);
    constexpr float cdsmk = (float)(kCd * F::ds * mkd);
#pragma unroll
    for (int i = 0; i < NG / 2; ++i) X[i] = __ffma2_rn(f2(-kC), A[i], X[i]);
    const float XJ = (J & 1) ? X[J / 2].y : X[J / 2].x;
    const float xj = fmaf(XJ, imk1, imk1DX1);
    const float pp = fmaf(w.owi, xj, w.alpha);  // p = alpha + (1-alpha) wi xj
    const float ps = pp * sTimk1;
    const float2 Ps = f2(ps);
    const float2 Qs = f2(fmaf(ps, DX1, (w.owj * sT * xj) * xj));
    const float2 PH = f2(pp * cdsm);
    float2 aI = f2(0.0f), aS = f2(0.0f);
#pragma unroll
    for (int i = 0; i < NG / 2; ++i) {
      const float2 ts = __ffma2_rn(X[i], Ps, Qs);
      const float2 r = F::r(ts);
      A[i] = __ffma2_rn(r, f2(cAr), A[i]);
      G[i] = __ffma2_rn(f2(kC), H[i], G[i]);
      const float2 gt = F::gt(G[i], ts, r);
      H[i] = __ffma2_rn(gt, PH, H[i]);
      aI = __ffma2_rn(gt, X[i], aI);
      aS = __fadd2_rn(aS, gt);
    }
    const float sS = aS.x + aS.y;
    const float tI = fmaf(DX1, sS, aI.x + aI.y) * cdsm;  // sum_i gT_i x_i
    const float tS = sS * cdsmk;                          // sum_i gT_i
    // gx_j += (1-alpha) (wi sum gT x + 2 wj xj sum gT), in units of m^(k+1)
    const float add = fmaf(w.owi, tI, 2.0f * w.owj * xj * tS) * imk1;
    if (J & 1) H[J / 2].y += add; else H[J / 2].x += add;
    const float oxj = w.oma * xj;
    dwi = fmaf(oxj, tI, dwi);
    dwj = fmaf(oxj * xj, tS, dwj);
    BwdSteps<NG, ACT, J - 1>::run(X, A, H, G, w, dwi, dwj);
  }
};
template <int NG, int ACT>
struct BwdSteps<NG, ACT, -1> {
  static __device__ __forceinline__ void run(float2 (&)[NG / 2], float2 (&)[NG / 2], float2 (&)[NG / 2],
                                             float2 (&)[NG / 2], const StageW&, float&, float&) {}
};

// On entry (x, a) hold the group's OUTPUT and (gx, ga) the incoming cotangents; on exit the
// group's input and the outgoing cotangents.  dwi/dwj gain the group's weight gradient.
template <int NG, int ACT>
__device__ __forceinline__ void group_backward(float (&x)[NG], float (&a)[NG], float (&gx)[NG], float (&ga)[NG],
                                               const StageW& w, float& dwi, float& dwj) {
  static_assert(NG % 2 == 0, "positions are processed in pairs");
  using F = ActForm<ACT>;
  float2 X[NG / 2], A[NG / 2], H[NG / 2], G[NG / 2];
#pragma unroll
  for (int i = 0; i < NG / 2; ++i) {
    X[i] = make_float2(x[2 * i], x[2 * i + 1]);
    A[i] = make_float2(a[2 * i], a[2 * i + 1]);
    H[i] = make_float2(gx[2 * i], gx[2 * i + 1]);
    G[i] = make_float2(ga[2 * i], ga[2 * i + 1]);
  }
  BwdSteps<NG, ACT, NG - 1>::run(X, A, H, G, w, dwi, dwj);
  constexpr float imN = (float)(1.0 / cpow(kMd, NG));
  constexpr float imNDX = (float)(bwd_DX(NG, F::f0) / cpow(kMd, NG));
  constexpr float imNCA = (float)(bwd_CA(NG, F::f0) / cpow(kMd, NG));
  constexpr float mN = (float)cpow(kMd, NG);
#pragma unroll
  for (int i = 0; i < NG / 2; ++i) {
    const float2 xo = __ffma2_rn(X[i], f2(imN), f2(imNDX));
    const float2 ao = __ffma2_rn(A[i], f2(imN), f2(imNCA));
    const float2 ho = __fmul2_rn(H[i], f2(mN));
    const float2 go = __fmul2_rn(G[i], f2(mN));
    x[2 * i] = xo.x; x[2 * i + 1] = xo.y;
    a[2 * i] = ao.x; a[2 * i + 1] = ao.y;
    gx[2 * i] = ho.x; gx[2 * i + 1] = ho.y;
    ga[2 * i] = go.x; ga[2 * i + 1] = go.y;
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
  int variant;            // pair backward: 0 = aliased tile buffer (two CTAs per SM), 1 = separate buffers
};

constexpr uint32_t kNoOff = 0xFFFFFFFFu;

}  // namespace ncn
