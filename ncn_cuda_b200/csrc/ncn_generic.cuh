// Per-stage NCN kernels for any (E, n_head, n_cache): one warp per (batch row, head, group).
//
// Behaviour replaced: ncn_cuda/ncn_fwd_cuda_kernel.cu:28-112 (forward_kernel) and
// ncn_cuda/ncn_bwd_cuda_kernel.cu:27-229 (backward_kernel), with the step loop running over the
// n_cache positions of the group as torch_ref/ncn_pytorch.py:74 does, 64-bit element offsets,
// and the weight gradient reduced inside the library instead of a [B, N, 2E] buffer.
//
// The n x d tile of each stream sits in shared memory (row pitch d|1 so that a lane per position
// reads conflict-free); lanes are arranged as (32/LD positions) x (LD features), LD a power of two.
#pragma once
#include "ncn_common.cuh"

namespace ncn {

struct StageParams {
  const void* in[4];  // fwd: x, xa ; bwd: y, ya, dy, dya
  void* out[4];       // fwd: y, ya ; bwd: dx, dxa, x_rec|null, xa_rec|null
  const float* W;     // [2E]
  float* partials;    // bwd: [gridDim.x][2E]
  const int* ctxlen;  // [B] context length per batch row, or null: every group takes all n steps
  const void* xin[2]; // bwd: the saved stage input (x, xa) or null
  int replay_all;     // bwd with xin: also the last segment starts from replayed values (y, ya are not read)
  float* mid;         // fp32 states after every kSegment-th step (fwd: written if not null; bwd: read if not null):
                      // state k, stream s at mid + (2k + s) * bne, in the element order of the activations
  long long bne;      // elements per activation tensor
  int mid_end;        // the state after the last step is stored / read too (y, ya are not read by the backward)
  long long B;
  long long groups;   // B * C * m
  int N, E, C, d, n, m, stride, ld_shift;  // LD = 1 << ld_shift
  int pitch;                               // d | 1
  float alpha, oma;
  int warps;
  uint32_t warp_floats;  // shared floats per warp
};

// longest chain of steps the backward rebuilds by the inverse when it has the stage input or stored states
constexpr int kSegment = 16;

__device__ __forceinline__ float act_rt(int act, float t) {
  switch (act) {
    case ACT_TANH: return act_fwd<ACT_TANH>(t);
    case ACT_RELU: return act_fwd<ACT_RELU>(t);
    case ACT_SIGMOID: return act_fwd<ACT_SIGMOID>(t);
    case ACT_LEAKY: return act_fwd<ACT_LEAKY>(t);
    default: return t;
  }
}
__device__ __forceinline__ float act_grad_rt(int act, float t, float f) {
  switch (act) {
    case ACT_TANH: return act_grad<ACT_TANH>(t, f);
    case ACT_RELU: return act_grad<ACT_RELU>(t, f);
    case ACT_SIGMOID: return act_grad<ACT_SIGMOID>(t, f);
    case ACT_LEAKY: return act_grad<ACT_LEAKY>(t, f);
    default: return 1.0f;
  }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Steps group g of row b takes.  With per-row context lengths (the reference's earlier Triton kernels,
// ncn_triton/ncn_triton_old.py:91-96, 189-192) a group counts its members g*n .. g*n+n-1 against the
// row's length: groups that lie before it take all n steps, the group it cuts takes the steps of the
// members before it, groups beyond it take none (their positions pass through unchanged).
__device__ __forceinline__ int group_steps(const int* ctxlen, long long b, int g, int n) {
  if (ctxlen == nullptr) return n;
  const long long left = (long long)ctxlen[b] - (long long)g * n;
  return left <= 0 ? 0 : (left < n ? (int)left : n);
}

// element offset of (row b, position pos, feature f)
__device__ __forceinline__ long long elem_off(long long b, int pos, int f, int N, int E) {
  return (b * N + pos) * (long long)E + f;
}

// One forward step j of a group whose tile sits in shared memory (X, A: [n][pitch]); xj [d] and
// sim [n] are scratch of the warp.  Used by the forward kernel and by the backward's replay.
__device__ __forceinline__ void stage_forward_step(const StageParams& p, const int act, float* X, float* A, float* xj,
                                                   float* sim, const float* Wi, const float* Wj, const int j,
                                                   const int lane) {
  const int n = p.n, d = p.d, pitch = p.pitch;
  const int LD = 1 << p.ld_shift, LT = 32 >> p.ld_shift;
  const int li = lane >> p.ld_shift, lk = lane & (LD - 1);
  float cj = 0.0f;
  for (int k = lane; k < d; k += 32) {
    const float v = X[j * pitch + k];
    xj[k] = v;
    cj = fmaf(v, Wj[k], cj);
  }
  cj = warp_sum(cj);
  __syncwarp();
  for (int i = lane; i < n; i += 32) {
    float acc = 0.0f;
    for (int k = 0; k < d; ++k) acc = fmaf(X[i * pitch + k], Wi[k], acc);
    sim[i] = (acc + cj) * p.oma;
  }
  __syncwarp();
  for (int i = li; i < n; i += LT) {
    const float si = sim[i];
    for (int k = lk; k < d; k += LD) {
      const float x = X[i * pitch + k];
      const float t = fmaf(si, xj[k], p.alpha * x);
      const float f = act_rt(act, t);
      const float a = fmaf(f, kC, A[i * pitch + k] * kM);
      A[i * pitch + k] = a;
      X[i * pitch + k] = fmaf(a, kC, x * kM);
    }
  }
  __syncwarp();
}

template <typename T>
__global__ void __launch_bounds__(256) stage_fwd_kernel(const StageParams p, const int act) {
  extern __shared__ __align__(16) float sm[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* X = sm + (size_t)warp * p.warp_floats;
  float* A = X + p.n * p.pitch;
  float* xj = A + p.n * p.pitch;  // [d]
  float* sim = xj + p.d;          // [n]
  const int LD = 1 << p.ld_shift, LT = 32 >> p.ld_shift;
  const int li = lane >> p.ld_shift, lk = lane & (LD - 1);
  const int n = p.n, d = p.d, pitch = p.pitch;
  const T* gx = static_cast<const T*>(p.in[0]);
  const T* ga = static_cast<const T*>(p.in[1]);
  T* gy = static_cast<T*>(p.out[0]);
  T* gya = static_cast<T*>(p.out[1]);

  for (long long gid = (long long)blockIdx.x * p.warps + warp; gid < p.groups; gid += (long long)gridDim.x * p.warps) {
    const int g = (int)(gid % p.m);
    const long long bc = gid / p.m;
    const int c = (int)(bc % p.C);
    const long long b = bc / p.C;
    const float* Wi = p.W + c * d;
    const float* Wj = p.W + p.E + c * d;
    for (int i = li; i < n; i += LT) {
      const int pos = (int)(((long long)g + (long long)i * p.stride) % p.m) * n + i;
      const long long off = elem_off(b, pos, c * d, p.N, p.E);
      for (int k = lk; k < d; k += LD) {
        X[i * pitch + k] = Store<T>::ld(gx + off + k);
        A[i * pitch + k] = Store<T>::ld(ga + off + k);
      }
    }
    __syncwarp();
    const int steps = group_steps(p.ctxlen, b, g, n);
    for (int j = 0; j < steps; ++j) {
      stage_forward_step(p, act, X, A, xj, sim, Wi, Wj, j, lane);
      if (p.mid != nullptr && (j + 1) % kSegment == 0 && (j + 1 < steps || p.mid_end)) {
        float* mx = p.mid + (long long)(2 * ((j + 1) / kSegment - 1)) * p.bne;
        for (int i = li; i < n; i += LT) {
          const int pos = (int)(((long long)g + (long long)i * p.stride) % p.m) * n + i;
          const long long off = elem_off(b, pos, c * d, p.N, p.E);
          for (int k = lk; k < d; k += LD) {
            mx[off + k] = X[i * pitch + k];
            mx[p.bne + off + k] = A[i * pitch + k];
          }
        }
        __syncwarp();
      }
    }
    for (int i = li; i < n; i += LT) {
      const int pos = (int)(((long long)g + (long long)i * p.stride) % p.m) * n + i;
      const long long off = elem_off(b, pos, c * d, p.N, p.E);
      for (int k = lk; k < d; k += LD) {
        Store<T>::st(gy + off + k, X[i * pitch + k]);
        Store<T>::st(gya + off + k, A[i * pitch + k]);
      }
    }
    __syncwarp();
  }
}

// Backward of one stage from its OUTPUT (reversible reconstruction, as the reference's CUDA
// backward does); formulas as in group_backward (ncn_common.cuh) with dot products over d.
// With the stage INPUT saved as well (p.xin), the state at every kSegment-th step is rebuilt by
// running the forward from the input, so that no inverse chain is longer than kSegment steps
// (every inverse step grows earlier rounding by 1/m).

template <typename T>
__global__ void __launch_bounds__(256) stage_bwd_kernel(const StageParams p, const int act) {
  extern __shared__ __align__(16) float sm[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n = p.n, d = p.d, pitch = p.pitch, E = p.E;
  float* X = sm + (size_t)warp * p.warp_floats;
  float* A = X + n * pitch;
  float* GX = A + n * pitch;
  float* GA = GX + n * pitch;
  float* GT = GA + n * pitch;
  float* xj = GT + n * pitch;  // [d]
  float* sim = xj + d;         // [n]  (1-alpha) * sim_i
  float* gs = sim + n;         // [n]  (1-alpha) * (gT_i . xj)
  float* dW = gs + n;          // [2E] this warp's running weight gradient
  const int LD = 1 << p.ld_shift, LT = 32 >> p.ld_shift;
  const int li = lane >> p.ld_shift, lk = lane & (LD - 1);
  const T* gy = static_cast<const T*>(p.in[0]);
  const T* gya = static_cast<const T*>(p.in[1]);
  const T* gdy = static_cast<const T*>(p.in[2]);
  const T* gdya = static_cast<const T*>(p.in[3]);
  T* odx = static_cast<T*>(p.out[0]);
  T* odxa = static_cast<T*>(p.out[1]);
  T* orx = static_cast<T*>(p.out[2]);
  T* orxa = static_cast<T*>(p.out[3]);

  for (int k = lane; k < 2 * E; k += 32) dW[k] = 0.0f;
  __syncwarp();

  for (long long gid = (long long)blockIdx.x * p.warps + warp; gid < p.groups; gid += (long long)gridDim.x * p.warps) {
    const int g = (int)(gid % p.m);
    const long long bc = gid / p.m;
    const int c = (int)(bc % p.C);
    const long long b = bc / p.C;
    const float* Wi = p.W + c * d;
    const float* Wj = p.W + E + c * d;
    for (int i = li; i < n; i += LT) {
      const int pos = (int)(((long long)g + (long long)i * p.stride) % p.m) * n + i;
      const long long off = elem_off(b, pos, c * d, p.N, E);
      for (int k = lk; k < d; k += LD) {
        if (!p.replay_all && !(p.mid != nullptr && p.mid_end)) {
          X[i * pitch + k] = Store<T>::ld(gy + off + k);
          A[i * pitch + k] = Store<T>::ld(gya + off + k);
        }
        GX[i * pitch + k] = Store<T>::ld(gdy + off + k);
        GA[i * pitch + k] = Store<T>::ld(gdya + off + k);
      }
    }
    __syncwarp();
    const int steps = group_steps(p.ctxlen, b, g, n);
    for (int j = steps - 1; j >= 0; --j) {
      if (p.mid != nullptr) {
        if ((j + 1) % kSegment == 0 && (j + 1 < steps || p.mid_end)) {  // the state after step j as the forward stored it
          const float* mx = p.mid + (long long)(2 * ((j + 1) / kSegment - 1)) * p.bne;
          for (int i = li; i < n; i += LT) {
            const int pos = (int)(((long long)g + (long long)i * p.stride) % p.m) * n + i;
            const long long off = elem_off(b, pos, c * d, p.N, E);
            for (int k = lk; k < d; k += LD) {
              X[i * pitch + k] = mx[off + k];
              A[i * pitch + k] = mx[p.bne + off + k];
            }
          }
          __syncwarp();
        }
      } else if (p.xin[0] != nullptr && (((j + 1) % kSegment == 0 && j + 1 < steps) || (j == steps - 1 && p.replay_all))) {
        // the state after step j, exactly: the forward over steps 0..j from the saved input
        const T* gxi = static_cast<const T*>(p.xin[0]);
        const T* gxa = static_cast<const T*>(p.xin[1]);
        for (int i = li; i < n; i += LT) {
          const int pos = (int)(((long long)g + (long long)i * p.stride) % p.m) * n + i;
          const long long off = elem_off(b, pos, c * d, p.N, E);
          for (int k = lk; k < d; k += LD) {
            X[i * pitch + k] = Store<T>::ld(gxi + off + k);
            A[i * pitch + k] = Store<T>::ld(gxa + off + k);
          }
        }
        __syncwarp();
        for (int jf = 0; jf <= j; ++jf) stage_forward_step(p, act, X, A, xj, sim, Wi, Wj, jf, lane);
      }
      // x = (y - c ya) / m
      for (int i = li; i < n; i += LT)
        for (int k = lk; k < d; k += LD) X[i * pitch + k] = fmaf(A[i * pitch + k], -kCoverM, X[i * pitch + k] * kInvM);
      __syncwarp();
      float cj = 0.0f;
      for (int k = lane; k < d; k += 32) {
        const float v = X[j * pitch + k];
        xj[k] = v;
        cj = fmaf(v, Wj[k], cj);
      }
      cj = warp_sum(cj);
      __syncwarp();
      for (int i = lane; i < n; i += 32) {
        float acc = 0.0f;
        for (int k = 0; k < d; ++k) acc = fmaf(X[i * pitch + k], Wi[k], acc);
        sim[i] = (acc + cj) * p.oma;
      }
      __syncwarp();
      for (int i = li; i < n; i += LT) {
        const float si = sim[i];
        for (int k = lk; k < d; k += LD) {
          const float x = X[i * pitch + k];
          const float t = fmaf(si, xj[k], p.alpha * x);
          const float f = act_rt(act, t);
          A[i * pitch + k] = fmaf(f, -kCoverM, A[i * pitch + k] * kInvM);
          const float gAp = fmaf(kC, GX[i * pitch + k], GA[i * pitch + k]);
          GT[i * pitch + k] = (kC * gAp) * act_grad_rt(act, t, f);
          GA[i * pitch + k] = kM * gAp;
        }
      }
      __syncwarp();
      for (int i = lane; i < n; i += 32) {
        float acc = 0.0f;
        for (int k = 0; k < d; ++k) acc = fmaf(GT[i * pitch + k], xj[k], acc);
        gs[i] = acc * p.oma;
      }
      __syncwarp();
      for (int i = li; i < n; i += LT) {
        const float gsi = gs[i];
        for (int k = lk; k < d; k += LD)
          GX[i * pitch + k] = fmaf(gsi, Wi[k], fmaf(p.alpha, GT[i * pitch + k], kM * GX[i * pitch + k]));
      }
      __syncwarp();
      // column sums over the positions of the group: contribution to gx_j and to dW
      for (int k = lane; k < d; k += 32) {
        float cs = 0.0f, ci = 0.0f, sg = 0.0f;
        for (int i = 0; i < n; ++i) {
          cs = fmaf(sim[i], GT[i * pitch + k], cs);
          ci = fmaf(gs[i], X[i * pitch + k], ci);
          sg += gs[i];
        }
        GX[j * pitch + k] += fmaf(sg, Wj[k], cs);
        dW[c * d + k] += ci;
        dW[E + c * d + k] = fmaf(sg, xj[k], dW[E + c * d + k]);
      }
      __syncwarp();
    }
    for (int i = li; i < n; i += LT) {
      const int pos = (int)(((long long)g + (long long)i * p.stride) % p.m) * n + i;
      const long long off = elem_off(b, pos, c * d, p.N, E);
      for (int k = lk; k < d; k += LD) {
        Store<T>::st(odx + off + k, GX[i * pitch + k]);
        Store<T>::st(odxa + off + k, GA[i * pitch + k]);
        if (orx) {
          Store<T>::st(orx + off + k, X[i * pitch + k]);
          Store<T>::st(orxa + off + k, A[i * pitch + k]);
        }
      }
    }
    __syncwarp();
  }
  // per-CTA partial: warps summed in warp order
  __syncthreads();
  for (int k = threadIdx.x; k < 2 * E; k += blockDim.x) {
    float acc = 0.0f;
    for (int w = 0; w < p.warps; ++w) acc += sm[(size_t)w * p.warp_floats + 5 * n * pitch + d + 2 * n + k];
    p.partials[(long long)blockIdx.x * 2 * E + k] = acc;
  }
}

// Sum partials[rows][cols] over rows in a fixed order: one warp per column, each lane adds its
// rows in increasing order, then a shuffle tree.  out[c] = sum (+ out[c] when accumulate).
__global__ void dw_reduce_kernel(const float* __restrict__ partials, float* __restrict__ out, int rows, int cols,
                                 int accumulate) {
  const int lane = threadIdx.x & 31;
  const int col = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (col >= cols) return;
  float acc = 0.0f;
  for (int r = lane; r < rows; r += 32) acc += partials[(long long)r * cols + col];
  acc = warp_sum(acc);
  if (lane == 0) out[col] = accumulate ? out[col] + acc : acc;
}

}  // namespace ncn
