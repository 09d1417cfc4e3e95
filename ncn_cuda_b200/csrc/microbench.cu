// Pipe microbenchmarks behind the roofline reasoning of the one-feature kernels (not part of the
// library).  Build and run:  make -C ncn_cuda_b200/csrc microbench && ./ncn_cuda_b200/build/microbench
//
// Part 1: throughput of the instruction classes the kernels are made of, alone and mixed, in cycles
//         per warp instruction group and SM sub-partition (8 warps per sub-partition).
// Part 2: the step arithmetic of ncn_lanes.cuh (lane_forward / lane_backward) with nothing around
//         it, at the kernels' own CTA shapes, in cycles per warp.position.step and sub-partition
//         (one warp.position.step = 32 positions taking one recurrence step).
#include <cstdio>
#include <cstdlib>
#include <cuda_runtime.h>

#include "ncn_lanes.cuh"
using namespace ncn;

static double g_mhz = 1965.0;

// MODE: 0 shfl, 1 ffma2 x8, 2 ffma2 x8 + NS shfl, 3 (ex2 + fmul) x4, 4 the same + NS shfl, 5 lds64,
//       6 ffma2 x8 + NS lds64, 9 (ex2 + fmul) x4 + ffma2 x8, 10 the same + NS shfl
template <int MODE, int NS>
__global__ void __launch_bounds__(256, 4) pipe_kernel(float* out, int iters) {
  __shared__ float2 sm[1024];
  const int t = threadIdx.x;
  float v[8];
  for (int i = 0; i < 8; i++) v[i] = t * 0.001f + i;
  float2 a[8];
  for (int i = 0; i < 8; i++) a[i] = make_float2(0.5f + i * 0.01f, 0.25f);
  float m[4];
  for (int i = 0; i < 4; i++) m[i] = 0.1f * i + t * 1e-4f;
  for (int i = t; i < 1024; i += 256) sm[i] = make_float2(1.f, 2.f);
  __syncthreads();
  const float2 c1 = make_float2(0.999f, 1.001f), c2 = make_float2(1e-3f, -1e-3f);
  for (int it = 0; it < iters; ++it) {
    if (MODE == 0 || MODE == 2 || MODE == 4 || MODE == 10) {
#pragma unroll
      for (int i = 0; i < NS; i++) v[i & 7] = __shfl_down_sync(0xffffffffu, v[i & 7], 1 + (i & 3));
    }
    if (MODE == 1 || MODE == 2 || MODE == 6 || MODE == 9 || MODE == 10) {
#pragma unroll
      for (int i = 0; i < 8; i++) a[i] = __ffma2_rn(a[i], c1, c2);
    }
    if (MODE == 3 || MODE == 4 || MODE == 9 || MODE == 10) {
#pragma unroll
      for (int i = 0; i < 4; i++) m[i] = ex2_approx(m[i]) * 0.5f;
    }
    if (MODE == 5 || MODE == 6) {
#pragma unroll
      for (int i = 0; i < NS; i++) {
        const float2 r = sm[(t + 32 * i + it) & 1023];
        v[i & 7] += r.x;
      }
    }
  }
  float acc = 0;
  for (int i = 0; i < 8; i++) acc += v[i] + a[i].x + a[i].y;
  for (int i = 0; i < 4; i++) acc += m[i];
  out[blockIdx.x * blockDim.x + t] = acc;
}

template <int MODE, int NS>
static void run_pipe(const char* name) {
  float* out;
  cudaMalloc(&out, 148 * 4 * 256 * 4);
  const int iters = 2000;
  cudaEvent_t a, b;
  cudaEventCreate(&a);
  cudaEventCreate(&b);
  pipe_kernel<MODE, NS><<<148 * 4, 256>>>(out, 10);
  cudaEventRecord(a);
  pipe_kernel<MODE, NS><<<148 * 4, 256>>>(out, iters);
  cudaEventRecord(b);
  cudaEventSynchronize(b);
  float ms;
  cudaEventElapsedTime(&ms, a, b);
  printf("%-52s %7.2f cycles per group and sub-partition\n", name, ms * 1e-3 * g_mhz * 1e6 / ((double)iters * 8));
  cudaFree(out);
}

// VAR: 0 lane_backward, 1 pair_backward (ncn_pairs.cuh), 2 lane_forward, 3 pair_forward
template <int NG, int PAIRS, int VAR, int ACT, int THREADS, int MINB>
__global__ void __launch_bounds__(THREADS, MINB) step_kernel(float* out, int iters, int L, float wsc) {
  const int t = threadIdx.x;
  float2 X[PAIRS][NG], A[PAIRS][NG], H[PAIRS][NG], G[PAIRS][NG];
  for (int p = 0; p < PAIRS; p++)
    for (int i = 0; i < NG; i++) {
      X[p][i] = make_float2(0.3f + 0.1f * i + t * 1e-3f, 0.3f - 0.1f * i + p);
      A[p][i] = make_float2(0.01f * i, 0.02f * i);
      H[p][i] = make_float2(0.5f, -0.2f * i);
      G[p][i] = make_float2(0.1f * i, 0.3f);
    }
  PairWB w;
  w.owi = f2(0.003f * wsc); w.owj = f2(-0.002f * wsc); w.owjs = f2(-0.002f * 2.885f * wsc); w.alpha = f2(0.9f); w.oma = f2(0.1f);
  PairW wf;
  wf.owi = f2(0.003f * wsc); wf.owj = f2(-0.002f * wsc); wf.alpha = f2(0.9f * 2.885f);
  float2 dwi = f2(0.f), dwj = f2(0.f);
  for (int it = 0; it < iters; ++it)
    for (int l = L - 1; l >= 0; --l) {
#pragma unroll
      for (int p = 0; p < PAIRS; p++) {
        if (VAR == 0) lane_backward<NG, ACT>(X[p], A[p], H[p], G[p], w, dwi, dwj);
        if (VAR == 1) pair_backward<NG, ACT>(X[p], A[p], H[p], G[p], w, dwi, dwj);
        if (VAR == 2) lane_forward<NG, ACT>(X[p], A[p], wf);
        if (VAR == 3) pair_forward<NG, ACT>(X[p], A[p], wf);
      }
    }
  float acc = dwi.x + dwi.y + dwj.x + dwj.y;
  for (int p = 0; p < PAIRS; p++)
    for (int i = 0; i < NG; i++) acc += X[p][i].x + X[p][i].y + A[p][i].x + A[p][i].y + H[p][i].x + H[p][i].y + G[p][i].x + G[p][i].y;
  out[blockIdx.x * blockDim.x + threadIdx.x] = acc;
}

template <int NG, int PAIRS, int VAR, int ACT, int THREADS, int MINB>
static void run_step(const char* name) {
  float* out;
  cudaMalloc(&out, 148 * MINB * THREADS * sizeof(float));
  const int L = 6, iters = 200 * 4 / NG;
  cudaEvent_t a, b;
  cudaEventCreate(&a);
  cudaEventCreate(&b);
  step_kernel<NG, PAIRS, VAR, ACT, THREADS, MINB><<<148 * MINB, THREADS>>>(out, 2, L, 1.0f);
  cudaEventRecord(a);
  step_kernel<NG, PAIRS, VAR, ACT, THREADS, MINB><<<148 * MINB, THREADS>>>(out, iters, L, 1.0f);
  cudaEventRecord(b);
  cudaEventSynchronize(b);
  float ms;
  cudaEventElapsedTime(&ms, a, b);
  const double wps = (double)iters * L * NG * NG * 2 * PAIRS * THREADS * MINB / 32 / 4;
  printf("%-52s %7.2f cycles per warp.position.step and sub-partition\n", name, ms * 1e-3 * g_mhz * 1e6 / wps);
  cudaFree(out);
}

int main(int argc, char** argv) {
  if (argc > 1) g_mhz = atof(argv[1]);  // SM clock in MHz the cycle figures assume (default 1965)
  printf("-- instruction classes (8 warps per sub-partition, SM clock assumed %.0f MHz)\n", g_mhz);
  run_pipe<0, 8>("8 shfl");
  run_pipe<1, 8>("8 fma.rn.f32x2");
  run_pipe<2, 4>("8 fma.rn.f32x2 + 4 shfl");
  run_pipe<2, 8>("8 fma.rn.f32x2 + 8 shfl");
  run_pipe<3, 4>("4 (ex2 + fmul)");
  run_pipe<4, 8>("4 (ex2 + fmul) + 8 shfl");
  run_pipe<5, 8>("8 ld.shared.v2 (full warp)");
  run_pipe<6, 4>("8 fma.rn.f32x2 + 4 ld.shared.v2");
  run_pipe<9, 0>("4 (ex2 + fmul) + 8 fma.rn.f32x2");
  run_pipe<10, 8>("4 (ex2 + fmul) + 8 fma.rn.f32x2 + 8 shfl");
  printf("-- step arithmetic alone\n");
  run_step<4, 2, 0, ACT_TANH, 256, 2>("backward tanh g=4, 2 pairs/thread, 256 x 2 CTAs");
  run_step<4, 2, 1, ACT_TANH, 256, 2>("  (ncn_pairs.cuh arithmetic, same shape)");
  run_step<4, 2, 0, ACT_LINEAR, 256, 2>("backward linear g=4, 2 pairs/thread, 256 x 2 CTAs");
  run_step<4, 2, 2, ACT_TANH, 256, 4>("forward tanh g=4, 2 pairs/thread, 256 x 4 CTAs");
  run_step<4, 2, 3, ACT_TANH, 256, 4>("  (ncn_pairs.cuh arithmetic, same shape)");
  run_step<4, 2, 2, ACT_LINEAR, 256, 4>("forward linear g=4, 2 pairs/thread, 256 x 4 CTAs");
  run_step<8, 1, 0, ACT_TANH, 256, 2>("backward tanh g=8, 1 pair/thread, 256 x 2 CTAs");
  run_step<8, 1, 2, ACT_TANH, 256, 4>("forward tanh g=8, 1 pair/thread, 256 x 4 CTAs");
  run_step<8, 1, 0, ACT_TANH_FAST, 256, 2>("backward tanh.approx g=8 (bf16 storage)");
  run_step<8, 1, 2, ACT_TANH_FAST, 256, 4>("forward tanh.approx g=8 (bf16 storage)");
  return 0;
}
