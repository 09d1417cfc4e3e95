/* C ABI of the B200 NCN library (libncn_b200.so).
 *
 * Drop-in boundary for the reference's pybind11 extension `ncn_cuda_module`
 * (ncn_cuda/ncn_cuda.cpp:3-32), whose two functions are
 *   forward (X, Xa, W, alpha, activation, cache_dim, nhead, module_l) -> {Y, Ya}
 *   backward(Y, Ya, dY, dYa, W, alpha, activation, cache_dim, nhead, module_l) -> {X, Xa, dX, dXa, dW}
 * and for the Python stage loop above it (ncn_cuda/ncn_pytorch_wrapper_v2.py:107-144).
 *
 * Conventions
 *  - every tensor is a contiguous [B, N, E] array on the current CUDA device, element type
 *    `dtype` (NCN_F32 or NCN_BF16); weights and weight gradients are always fp32;
 *  - W of one stage is [2E] = [Wi | Wj] (torch_ref/ncn_pytorch.py:60-61); W of a net is [L][2E];
 *  - activation codes are the reference's (ncn_pytorch_wrapper_v2.py:111):
 *    0 tanh, 1 relu, 2 sigmoid, anything else (-1) linear; 3 is added for "leaky-relu" (slope 0.01,
 *    torch_ref/ncn_pytorch_invertible.py:39-44, ncn_triton/ncn_triton.py:22-28), which the per-stage
 *    calls run on their general kernels and the net calls answer with NCN_ERR_UNSUPPORTED;
 *  - the caller owns every buffer; nothing is allocated, freed or memset by the library
 *    (unless a function says otherwise); every output element is written exactly once;
 *  - work is enqueued on `stream` (a cudaStream_t passed as void*) and the call returns without
 *    synchronising; arguments are validated first and a non-zero status means nothing was
 *    enqueued;
 *  - the weight gradient is returned already summed over batch and positions (the reference
 *    returns a [B, N, 2E] buffer and lets the wrapper sum it, ncn_pytorch_wrapper_v2.py:48); the
 *    sum runs in a fixed order, so it is bitwise reproducible for equal arguments on one device.
 */
#ifndef NCN_B200_H_
#define NCN_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { NCN_F32 = 0, NCN_BF16 = 1 };

/* status codes */
enum {
  NCN_OK = 0,
  NCN_ERR_SHAPE = 1,       /* n_cache does not divide N, n_head does not divide E, sizes <= 0 */
  NCN_ERR_DTYPE = 2,       /* dtype is neither NCN_F32 nor NCN_BF16 */
  NCN_ERR_ALIGN = 3,       /* a tensor pointer is not 16-byte aligned (fused path only) */
  NCN_ERR_SMEM = 4,        /* the tile does not fit the shared memory of one SM */
  NCN_ERR_UNSUPPORTED = 5, /* the fused all-stage path does not cover these arguments; use the per-stage calls */
  NCN_ERR_WORKSPACE = 6,   /* workspace missing or smaller than ncn_bwd_workspace_bytes() */
  NCN_ERR_CUDA = 7,        /* a CUDA runtime call failed; see ncn_last_cuda_error() */
  NCN_ERR_NULL = 8,        /* a required pointer is null */
  NCN_ERR_DEVICE_WAIT = 9, /* (ncn_device_status) a kernel gave up a bounded wait on a copy */
  NCN_ERR_TOO_LARGE = 10   /* (ncn_net_bwd_noalloc) more scratch needed than the built-in array holds */
};

/* flags of the net calls */
enum {
  NCN_RESIDUAL = 1,  /* forward: y = x + net(x, xa).x ; backward: dx = dx_net + dy */
  NCN_RECOMPUTE = 2, /* backward: s0/s1 are the net INPUT (x, xa); the forward is replayed in fp32.
                        With bf16 storage or NCN_RESIDUAL use this or NCN_TAPE. */
  NCN_TAPE = 8       /* forward: also keep the fp32 state after the LAST stage (before the residual add) in
                        ckpt, one slot after the periodic ones.  backward (same flag, same ckpt, same
                        ckpt_every): starts from that state, s0/s1 are not read and may be null.  The
                        alternative to NCN_RECOMPUTE: no forward replay, 8 more bytes per element kept. */
};

/* One stage forward.  Replaces ncn_cuda_module.forward (ncn_cuda/ncn_cuda.cpp:30;
 * ncn_cuda/ncn_fwd_cuda_kernel.cu:115-161); the step loop runs over the n_cache positions of a
 * group as torch_ref/ncn_pytorch.py:74 does. */
int ncn_stage_fwd(const void* x, const void* xa, const float* W, void* y, void* ya, int64_t B, int64_t N, int64_t E,
                  int n_cache, int n_head, int module_l, double alpha, int activation, int dtype, void* stream);

/* One stage backward from the stage OUTPUT (reversible reconstruction).  Replaces
 * ncn_cuda_module.backward (ncn_cuda/ncn_cuda.cpp:31; ncn_cuda/ncn_bwd_cuda_kernel.cu:232-288)
 * plus the wrapper's torch.sum over the dW buffer (ncn_pytorch_wrapper_v2.py:48).
 * x_rec / xa_rec (the rebuilt stage input) may be null.  dW is [2E] fp32.
 * workspace: device memory of at least ncn_bwd_workspace_bytes(...) bytes, fully overwritten. */
int ncn_stage_bwd(const void* y, const void* ya, const void* dy, const void* dya, const float* W, void* dx, void* dxa,
                  void* x_rec, void* xa_rec, float* dW, void* workspace, size_t workspace_bytes, int64_t B, int64_t N,
                  int64_t E, int n_cache, int n_head, int module_l, double alpha, int activation, int dtype,
                  void* stream);

/* ncn_stage_bwd for callers that also kept the stage INPUT (x, xa).  No counterpart in the reference, whose
 * NCNFunction saves the stage output only (ncn_cuda/ncn_pytorch_wrapper_v2.py:21, 35) and rebuilds the input by
 * the inverse of torch_ref/ncn_pytorch_invertible.py:97-111: every rebuilt step divides by 0.9, so a stage of
 * n_cache = 32 steps leaves fp32 gradients at about 1e-5 of their size.  Here the state at every 16th step is
 * rebuilt exactly by running the forward from the saved input, so no inverse chain exceeds 16 steps and the
 * gradients keep the accuracy of plain autograd.  With bf16 storage the whole stage is replayed from the input
 * (y, ya are not read and may be null): an inverse started from rounded outputs would amplify their rounding.
 * With fp32 storage and n_cache <= 16 this is ncn_stage_bwd (x, xa are not read).  Results as ncn_stage_bwd. */
int ncn_stage_bwd_saved(const void* x, const void* xa, const void* y, const void* ya, const void* dy, const void* dya,
                        const float* W, void* dx, void* dxa, float* dW, void* workspace, size_t workspace_bytes, int64_t B,
                        int64_t N, int64_t E, int n_cache, int n_head, int module_l, double alpha, int activation,
                        int dtype, void* stream);

/* The same accuracy without the replay, for callers that can spend memory instead: the forward also stores the
 * fp32 state after every 16th step short of the last (n_cache = 32: one state, 8 bytes per element; with bf16
 * storage the state after the last step too, and the backward then reads neither y nor ya, which may be null),
 * and the backward restarts its inverse there.  No counterpart in the reference.  `mid` is opaque to the caller:
 * ncn_stage_mid_bytes(...) bytes of device memory, 16-byte aligned, written by ncn_stage_fwd_mid and handed
 * unchanged to ncn_stage_bwd_mid with the same shape arguments.  Where ncn_stage_mid_bytes is 0 (fp32 storage,
 * n_cache <= 16) the calls are ncn_stage_fwd / ncn_stage_bwd and mid may be null. */
size_t ncn_stage_mid_bytes(int64_t B, int64_t N, int64_t E, int n_cache, int dtype);
int ncn_stage_fwd_mid(const void* x, const void* xa, const float* W, void* y, void* ya, void* mid, size_t mid_bytes,
                      int64_t B, int64_t N, int64_t E, int n_cache, int n_head, int module_l, double alpha, int activation,
                      int dtype, void* stream);
int ncn_stage_bwd_mid(const void* y, const void* ya, const void* mid, size_t mid_bytes, const void* dy, const void* dya,
                      const float* W, void* dx, void* dxa, float* dW, void* workspace, size_t workspace_bytes, int64_t B,
                      int64_t N, int64_t E, int n_cache, int n_head, int module_l, double alpha, int activation,
                      int dtype, void* stream);

/* One stage with a context length per batch row, forward and backward.  Replace the step-count rule of the
 * reference's earlier Triton operator (ncn_triton/ncn_triton_old.py:70-96 forward, :186-197 backward:
 * `ctxlen = load(ctxlen_tensor + batch)`, `hi = GROUP if group*GROUP + GROUP < ctxlen else ctxlen - group*GROUP`,
 * steps 0 .. hi-1), applied to the stage index map of torch_ref/ncn_pytorch.py:12-41.
 * ctxlen: int32 [B] on the device.  Group g of row b counts its members g*n_cache .. g*n_cache+n_cache-1 against
 * ctxlen[b]: groups before it take all n_cache steps, the group it cuts takes the steps of the members before
 * it, groups at or beyond it take none.  Every position is still read and written: positions of groups that
 * take no step pass through unchanged (y = x, ya = xa; dx = dy, dxa = dya) - the reference leaves them
 * unwritten.  ctxlen[b] >= N gives ncn_stage_fwd / ncn_stage_bwd.  Other arguments as in those calls; these
 * entries always run the shared-memory kernels (any E, n_head, n_cache). */
int ncn_stage_fwd_ctx(const void* x, const void* xa, const float* W, const int* ctxlen, void* y, void* ya, int64_t B,
                      int64_t N, int64_t E, int n_cache, int n_head, int module_l, double alpha, int activation, int dtype,
                      void* stream);
int ncn_stage_bwd_ctx(const void* y, const void* ya, const void* dy, const void* dya, const float* W, const int* ctxlen,
                      void* dx, void* dxa, void* x_rec, void* xa_rec, float* dW, void* workspace, size_t workspace_bytes,
                      int64_t B, int64_t N, int64_t E, int n_cache, int n_head, int module_l, double alpha, int activation,
                      int dtype, void* stream);

/* All L stages (module_l = first_module .. first_module+L-1) in one kernel.  Replaces the stage
 * loops NCNNetCuda.forward / NCNNetTestCuda.forward (ncn_pytorch_wrapper_v2.py:114-117,132-144).
 * ckpt (may be null without NCN_TAPE): fp32 buffer of ncn_ckpt_bytes(...) bytes that receives the state
 * after every ckpt_every-th stage (ckpt_every <= 0: none) and, with NCN_TAPE, after the last one, for
 * ncn_net_bwd.  Returns NCN_ERR_UNSUPPORTED where only the per-stage calls
 * apply (E != 1, n_cache not in {2,4,8,16}, N not a multiple of 4 (fp32) / 8 (bf16)). */
int ncn_net_fwd(const void* x, const void* xa, const float* W, void* y, void* ya, float* ckpt, int ckpt_every,
                int64_t B, int64_t N, int64_t E, int n_cache, int n_head, int first_module, int L, double alpha,
                int activation, int dtype, int flags, void* stream);

/* Backward of ncn_net_fwd in one kernel.  s0/s1 are the net OUTPUT (y, ya) — every stage input is
 * rebuilt by the reversible inverse, restarting at each stored checkpoint — or, with NCN_RECOMPUTE,
 * the net INPUT, or unused with NCN_TAPE.  dW is [L][2E] fp32; with dw_accumulate != 0 the result is added to it.
 * x_rec / xa_rec may be null. */
int ncn_net_bwd(const void* s0, const void* s1, const void* dy, const void* dya, const float* W, void* dx, void* dxa,
                void* x_rec, void* xa_rec, float* dW, const float* ckpt, int ckpt_every, void* workspace,
                size_t workspace_bytes, int64_t B, int64_t N, int64_t E, int n_cache, int n_head, int first_module,
                int L, double alpha, int activation, int dtype, int flags, int dw_accumulate, void* stream);

/* ncn_net_bwd for callers that cannot allocate device memory.  It has no counterpart in the
 * reference.  Some hosts of this operator get no chance to reserve a workspace: a plugin whose
 * host hands it only the input and output tensors, a control loop that must never touch the
 * allocator because allocation may synchronise the device, code that runs after the application
 * has frozen its memory budget.  For them the scratch of the backward kernel (one row of 2L
 * partial weight-gradient sums per CTA) lives in a 64 KiB array inside the library image; every
 * GPU that loads the library carries that array until the process exits.
 *  - Arguments and results are those of ncn_net_bwd without workspace / workspace_bytes; results
 *    are bitwise those of ncn_net_bwd for equal arguments.
 *  - Limit: CTAs launched x 2L <= 16384 floats (on a 148-SM part with two CTAs per SM: L <= 27);
 *    beyond it the call returns NCN_ERR_TOO_LARGE and enqueues nothing.
 *  - It calls no cudaMalloc / cudaFree and no allocating library routine.
 *  - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with
 *    that device current).
 *  - All calls on a device share the one array and it keeps the last call's partial sums.  Nothing
 *    in it has to be cleared (the kernel writes every element the reduction reads), but two calls
 *    whose kernels overlap on the GPU (different streams, no ordering) race on it: order them. */
int ncn_net_bwd_noalloc(const void* s0, const void* s1, const void* dy, const void* dya, const float* W, void* dx,
                        void* dxa, void* x_rec, void* xa_rec, float* dW, const float* ckpt, int ckpt_every, int64_t B,
                        int64_t N, int64_t E, int n_cache, int n_head, int first_module, int L, double alpha,
                        int activation, int dtype, int flags, int dw_accumulate, void* stream);

/* 1 if ncn_net_fwd / ncn_net_bwd (without x_rec / xa_rec, whose staging needs more shared memory and
 * may still return NCN_ERR_SMEM for the longest rows) cover these arguments on the current device,
 * else 0.  flags and ckpt_every as they will be passed to the net calls. */
int ncn_net_supported(int64_t B, int64_t N, int64_t E, int n_cache, int n_head, int L, int dtype, int flags,
                      int ckpt_every);

/* Workspace (bytes) that ncn_stage_bwd (L = 1) or ncn_net_bwd needs for these arguments. */
size_t ncn_bwd_workspace_bytes(int64_t B, int64_t N, int64_t E, int n_cache, int n_head, int L, int dtype);

/* Size (bytes) of the checkpoint buffer: (L-1)/ckpt_every states (0 for ckpt_every <= 0), one more
 * with NCN_TAPE in flags, each 2 x [B, N, E] fp32. */
size_t ncn_ckpt_bytes(int64_t B, int64_t N, int64_t E, int L, int ckpt_every, int flags);

/* Reads and clears the device status word (synchronises the device): NCN_OK, or
 * NCN_ERR_DEVICE_WAIT if a kernel abandoned a bounded wait since the last call. */
int ncn_device_status(void);

/* Text for a status code; the last CUDA error string seen by this thread. */
const char* ncn_status_string(int status);
const char* ncn_last_cuda_error(void);

/* Library version (major*100 + minor). */
int ncn_version(void);

/* The NCN_* environment switches (kernel selection for A/B measurements: NCN_LANES, NCN_LANES_PIPE, NCN_FWD_DUAL, NCN_BWD_DUAL, NCN_NO_PAIR, NCN_NO_FEAT, NCN_EXACT_TANH, ...) are read once,
 * when the library is loaded, and launch plans are remembered per argument set.  This call reads the
 * switches again and forgets the remembered plans.  Not thread-safe against concurrent launches.
 * No counterpart in the reference (which has no such switches).
 * The library also remembers, per device, the addresses of its device-side status word and scratch array and the
 * shared-memory size it has granted each kernel.  cudaDeviceReset() invalidates all of that behind its back: a
 * process that resets a device must unload and reload the library before using it on that device again. */
void ncn_reload_env(void);

#ifdef __cplusplus
}
#endif
#endif /* NCN_B200_H_ */
