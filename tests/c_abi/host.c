/* A plain C host of the library: no Python, no torch.  Reads a problem from a file, runs the
 * fused forward and backward through the C ABI of include/ncn_b200.h (the calls a binding in any
 * language makes in place of ncn_cuda_module.forward / backward, ncn_cuda/ncn_cuda.cpp:29-32)
 * and writes the results to another file.  Built and driven by tests/test_gpu_c_abi.py.
 *
 * file formats (little endian):
 *   in : int32 B, N, n_cache, L, ckpt_every, activation ; float32 x[B*N], xa[B*N], W[L*2], dy[B*N], dya[B*N]
 *   out: float32 y[B*N], ya[B*N], dx[B*N], dxa[B*N], dW[L*2]
 */
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#include "ncn_b200.h"

#define CK(call)                                                                     \
  do {                                                                               \
    cudaError_t e_ = (call);                                                         \
    if (e_ != cudaSuccess) {                                                         \
      fprintf(stderr, "%s: %s\n", #call, cudaGetErrorString(e_));                    \
      return 2;                                                                      \
    }                                                                                \
  } while (0)
#define NCN(call)                                                                    \
  do {                                                                               \
    int rc_ = (call);                                                                \
    if (rc_ != NCN_OK) {                                                             \
      fprintf(stderr, "%s: %s\n", #call, ncn_status_string(rc_));                    \
      return 3;                                                                      \
    }                                                                                \
  } while (0)

static float* dev_copy(const float* h, size_t n) {
  float* d = NULL;
  if (cudaMalloc((void**)&d, n * sizeof(float)) != cudaSuccess) return NULL;
  if (h && cudaMemcpy(d, h, n * sizeof(float), cudaMemcpyHostToDevice) != cudaSuccess) return NULL;
  return d;
}

int main(int argc, char** argv) {
  if (argc != 3) {
    fprintf(stderr, "usage: %s <in> <out>\n", argv[0]);
    return 1;
  }
  FILE* f = fopen(argv[1], "rb");
  if (!f) return 1;
  int32_t hdr[6];
  if (fread(hdr, sizeof(int32_t), 6, f) != 6) return 1;
  const int64_t B = hdr[0], N = hdr[1];
  const int n_cache = hdr[2], L = hdr[3], ckpt_every = hdr[4], activation = hdr[5];
  const size_t bn = (size_t)(B * N), nw = (size_t)L * 2;
  float* h = (float*)malloc((4 * bn + nw) * sizeof(float));
  if (!h || fread(h, sizeof(float), 4 * bn + nw, f) != 4 * bn + nw) return 1;
  fclose(f);
  const float *hx = h, *hxa = h + bn, *hW = h + 2 * bn, *hdy = h + 2 * bn + nw, *hdya = h + 3 * bn + nw;

  float *x = dev_copy(hx, bn), *xa = dev_copy(hxa, bn), *W = dev_copy(hW, nw), *dy = dev_copy(hdy, bn),
        *dya = dev_copy(hdya, bn);
  float *y = dev_copy(NULL, bn), *ya = dev_copy(NULL, bn), *dx = dev_copy(NULL, bn), *dxa = dev_copy(NULL, bn),
        *dW = dev_copy(NULL, nw);
  if (!x || !xa || !W || !dy || !dya || !y || !ya || !dx || !dxa || !dW) return 2;

  if (!ncn_net_supported(B, N, 1, n_cache, 1, L, NCN_F32, 0, ckpt_every)) {
    fprintf(stderr, "shape not covered by the fused calls\n");
    return 4;
  }
  float* ckpt = NULL;
  const size_t ck_bytes = ncn_ckpt_bytes(B, N, 1, L, ckpt_every, 0);
  if (ck_bytes) CK(cudaMalloc((void**)&ckpt, ck_bytes));
  void* ws = NULL;
  const size_t ws_bytes = ncn_bwd_workspace_bytes(B, N, 1, n_cache, 1, L, NCN_F32);
  CK(cudaMalloc(&ws, ws_bytes));
  cudaStream_t st;
  CK(cudaStreamCreate(&st));

  NCN(ncn_net_fwd(x, xa, W, y, ya, ckpt, ckpt_every, B, N, 1, n_cache, 1, 0, L, 0.9, activation, NCN_F32, 0, st));
  NCN(ncn_net_bwd(y, ya, dy, dya, W, dx, dxa, NULL, NULL, dW, ckpt, ckpt_every, ws, ws_bytes, B, N, 1, n_cache, 1, 0, L,
                  0.9, activation, NCN_F32, 0, 0, st));
  CK(cudaStreamSynchronize(st));
  NCN(ncn_device_status());

  float* out = (float*)malloc((4 * bn + nw) * sizeof(float));
  if (!out) return 1;
  CK(cudaMemcpy(out, y, bn * sizeof(float), cudaMemcpyDeviceToHost));
  CK(cudaMemcpy(out + bn, ya, bn * sizeof(float), cudaMemcpyDeviceToHost));
  CK(cudaMemcpy(out + 2 * bn, dx, bn * sizeof(float), cudaMemcpyDeviceToHost));
  CK(cudaMemcpy(out + 3 * bn, dxa, bn * sizeof(float), cudaMemcpyDeviceToHost));
  CK(cudaMemcpy(out + 4 * bn, dW, nw * sizeof(float), cudaMemcpyDeviceToHost));
  f = fopen(argv[2], "wb");
  if (!f || fwrite(out, sizeof(float), 4 * bn + nw, f) != 4 * bn + nw) return 1;
  fclose(f);
  printf("ncn_b200 version %d: forward + backward of %lld x %lld, n_cache %d, %d stages\n", ncn_version(), (long long)B,
         (long long)N, n_cache, L);
  return 0;
}
