// C ABI of the NCN library: argument validation, launch planning, kernel launches.
// Declarations and the reference interfaces they replace are in include/ncn_b200.h.
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <utility>
#include <vector>

#include "../../include/ncn_b200.h"
#include "ncn_generic.cuh"
#include "ncn_rows_launch.h"
#include "ncn_lanes_launch.h"
#include "ncn_feat.cuh"
#include "ncn_feat_launch.h"

namespace ncn {

__device__ int g_status_word = 0;

static thread_local char tl_cuda_err[256] = "";

static int cuda_fail(cudaError_t e) {
  std::snprintf(tl_cuda_err, sizeof(tl_cuda_err), "%s: %s", cudaGetErrorName(e), cudaGetErrorString(e));
  return NCN_ERR_CUDA;
}

struct DevInfo {
  int dev = -1, sms = 0, smem_optin = 0;
  int* status = nullptr;
};

// Per-device facts, looked up once per device and cached (the table is tiny and written
// idempotently, so a race between two first calls is harmless).
static int get_dev(DevInfo& out) {
  static DevInfo table[64];
  static std::atomic<int> ready[64];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e);
  if (dev < 0 || dev >= 64) return NCN_ERR_CUDA;
  if (!ready[dev].load(std::memory_order_acquire)) {
    DevInfo d;
    d.dev = dev;
    if ((e = cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return cuda_fail(e);
    if ((e = cudaDeviceGetAttribute(&d.smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev)) != cudaSuccess)
      return cuda_fail(e);
    if ((e = cudaGetSymbolAddress(reinterpret_cast<void**>(&d.status), g_status_word)) != cudaSuccess)
      return cuda_fail(e);
    table[dev] = d;
    ready[dev].store(1, std::memory_order_release);
  }
  out = table[dev];
  return NCN_OK;
}

// Tuning switches of the environment, read once per process (they select among kernels for A/B
// measurements; the defaults are the fastest measured).
struct EnvSwitches {
  bool exact_tanh, no_pair, no_feat, bwd_wide_off, bwd_dual_off, fwd_dual_off, lanes_off, lanes_pipe_off;
  int fwd_threads, bwd_threads, nbuf, lane_rows;
  bool lanes_pipe_fwd;   // NCN_LANES_PIPE_FWD=1: the pipelined forward (measured slower; kept for A/B runs)
  bool test_short_wait;  // NCN_TEST_SHORT_WAIT=1: the lane forward gives up its first wait (tests of that path)
};
static EnvSwitches read_env_switches() {
  auto is = [](const char* name, char c) {
    const char* e = std::getenv(name);
    return e && e[0] == c;
  };
  auto num = [](const char* name) {
    const char* e = std::getenv(name);
    return e ? std::atoi(e) : 0;
  };
  EnvSwitches v;
  v.exact_tanh = is("NCN_EXACT_TANH", '1');
  v.no_pair = is("NCN_NO_PAIR", '1');
  v.no_feat = is("NCN_NO_FEAT", '1');
  v.bwd_wide_off = is("NCN_BWD_WIDE", '0');
  v.bwd_dual_off = is("NCN_BWD_DUAL", '0');
  v.fwd_dual_off = is("NCN_FWD_DUAL", '0');
  v.lanes_off = is("NCN_LANES", '0');
  v.lanes_pipe_off = is("NCN_LANES_PIPE", '0');
  v.fwd_threads = num("NCN_FWD_THREADS");
  v.bwd_threads = num("NCN_BWD_THREADS");
  v.nbuf = num("NCN_NBUF");
  v.lane_rows = num("NCN_LANE_ROWS");
  v.lanes_pipe_fwd = is("NCN_LANES_PIPE_FWD", '1');
  v.test_short_wait = is("NCN_TEST_SHORT_WAIT", '1');
  return v;
}
static EnvSwitches g_env = read_env_switches();
static std::atomic<int> g_plan_epoch{0};  // bumped by ncn_reload_env: cached launch plans of older epochs are stale
static const EnvSwitches& env_switches() { return g_env; }

// tanh with bf16 storage runs on tanh.approx inside the fused kernels (NCN_EXACT_TANH=1 turns that off)
static int fused_act(int act, int dtype) {
  if (act == ACT_TANH && dtype == DT_BF16 && !env_switches().exact_tanh) return ACT_TANH_FAST;
  return act;
}

static int map_act(int code) {
  switch (code) {
    case 0: return ACT_TANH;
    case 1: return ACT_RELU;
    case 2: return ACT_SIGMOID;
    case 3: return ACT_LEAKY;  // shared-memory stage kernels only
    default: return ACT_LINEAR;
  }
}

static inline uint32_t align_up(uint32_t v, uint32_t a) { return (v + a - 1) / a * a; }
static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static bool rows_shape_ok(int64_t N, int64_t E, int n, int C, int dtype) {
  if (E != 1 || C != 1) return false;
  if (!(n == 2 || n == 4 || n == 8 || n == 16)) return false;
  const int64_t quantum = dtype == DT_BF16 ? 8 : 4;  // 16-byte rows for the bulk copies
  if (N % quantum != 0) return false;
  if (N / n > (1 << 24)) return false;
  return true;
}

struct Plan {
  bool pair = false;  // two groups per thread (ncn_pairs.cuh)
  bool red_thread = false;  // dW partial slots per thread
  int variant = 0;    // pair backward: 0 aliased tile buffer, 1 separate buffers
  int threads = 0, R = 0, nbuf = 0, grid = 0;
  size_t smem = 0;
  uint32_t off_in[2] = {0, 0}, off_work = 0, off_out = 0, off_ckpt = kNoOff, off_red = 0, off_w = 0, off_bar = 0;
  uint32_t n_ckpt_slots = 0;
  long long tiles = 0;
};

typedef cudaError_t (*RowsLaunchFn)(int, int, const RowsParams&, int, int, size_t, cudaStream_t, int*);

static RowsLaunchFn pair_fn(int n, bool bwd) {
  if (bwd) {
    switch (n) {
      case 2: return launch_pair_bwd_n2;
      case 4: return launch_pair_bwd_n4;
      case 8: return launch_pair_bwd_n8;
      default: return nullptr;  // 16: the pair's four streams do not fit the register file
    }
  }
  switch (n) {
    case 2: return launch_pair_fwd_n2;
    case 4: return launch_pair_fwd_n4;
    case 8: return launch_pair_fwd_n8;
    case 16: return launch_pair_fwd_n16;
    default: return nullptr;
  }
}

static RowsLaunchFn rows_fn(int n, bool bwd) {
  switch (n) {
    case 2: return bwd ? launch_rows_bwd_n2 : launch_rows_fwd_n2;
    case 4: return bwd ? launch_rows_bwd_n4 : launch_rows_fwd_n4;
    case 8: return bwd ? launch_rows_bwd_n8 : launch_rows_fwd_n8;
    case 16: return bwd ? launch_rows_bwd_n16 : launch_rows_fwd_n16;
    default: return nullptr;
  }
}

// Lay the tile out in shared memory.  Preference: two input buffers (prefetch of the next tile
// starts a whole tile early) > checkpoints staged in shared memory > one input buffer.
static int plan_rows_impl(bool bwd, int64_t B, int N, int n, int L, int dtype, int flags, int n_ck, bool want_rec,
                          const DevInfo& dev, int act, bool want_wide, Plan& pl, bool want_dual = false) {
  const int w = dtype == DT_BF16 ? 2 : 4;
  const int m = N / n;
  // fast path: one pair of groups (g, g + m/2) per thread, if a row's pairs fit one CTA
  pl.pair = pair_fn(n, bwd) != nullptr && m % 2 == 0 && m / 2 <= pair_max_threads(n, bwd) && !env_switches().no_pair;
  const bool wide = bwd && pl.pair && want_wide && !want_dual;
  const bool dual = bwd && pl.pair && want_dual && n <= 8 && !(flags & F_RECOMPUTE);
  if (want_dual && (bwd ? !dual : !pl.pair)) return NCN_ERR_UNSUPPORTED;
  if (wide) pl.variant = 1;  // separate buffers: planned by the general layout below
  if (pl.pair && bwd && !wide && !dual && (flags & F_TAPE)) pl.pair = false;  // the aliased variant has no tape path
  if (pl.pair && bwd && !wide) {
    // pair backward: one 16-byte slot per position doubles as TMA landing zone and output staging
    const bool residual = (flags & F_RESIDUAL) != 0;
    const int slots = (flags & F_RECOMPUTE) ? 0 : n_ck;
    // dual: two pairs per thread, half the threads for the same tile
    const int ppt = dual ? 2 : 1;
    if (dual) pl.variant = 2;
    const int maxTp = pair_max_threads(n, true);
    int Rp = (m / 2) >= maxTp ? 1 : maxTp / (m / 2);
    if ((int64_t)Rp > B) Rp = (int)B;
    for (; Rp >= 1; Rp = (Rp > 1 ? Rp / 2 : 0)) {
      const int threads = (int)align_up((uint32_t)((Rp * (m / 2) + ppt - 1) / ppt), 32);
      const uint64_t RN = (uint64_t)Rp * N;
      uint64_t off = 0;
      auto take = [&](uint64_t bytes) { uint64_t o = off; off = (off + bytes + 127) / 128 * 128; return (uint32_t)o; };
      pl.off_in[0] = pl.off_in[1] = 0;
      pl.off_work = take(RN * 16);
      pl.off_out = pl.off_work;
      uint64_t ckb = (uint64_t)slots * RN * 8;
      if (!dual && residual && RN * w > ckb) ckb = RN * w;  // (aliased variant: dy shares the checkpoint area)
      pl.off_ckpt = take(ckb ? ckb : 16);
      if (dual && residual) pl.off_in[0] = pl.off_in[1] = take(RN * w);  // native dy for the final add
      pl.off_red = take((uint64_t)2 * L * (threads / 32) * 4);
      pl.off_w = take((uint64_t)16 * L);
      pl.off_bar = take(32);
      if (off <= (uint64_t)dev.smem_optin) {
        pl.threads = threads; pl.R = Rp; pl.nbuf = 1; pl.n_ckpt_slots = (uint32_t)slots; pl.smem = (size_t)off;
        pl.tiles = (B + Rp - 1) / Rp;
        int occ = 0;
        RowsParams dummy{};
        dummy.variant = pl.variant;
        cudaError_t e = pair_fn(n, true)(act, dtype, dummy, 0, pl.threads, pl.smem, nullptr, &occ);
        if (e != cudaSuccess) return cuda_fail(e);
        if (occ >= 1) {
          if (occ > 32) occ = 32;
          long long grid = (long long)dev.sms * occ;
          if (grid > pl.tiles) grid = pl.tiles;
          pl.grid = (int)grid;
          return NCN_OK;
        }
      }
    }
    pl.pair = false;  // does not fit: general kernel
  }
  if (pl.pair && !bwd && want_dual) {
    // pair forward, one buffer: 8 bytes per position (native in, slots, native out), two pairs per thread
    const bool residual = (flags & F_RESIDUAL) != 0;
    const int maxTp = pair_max_threads(n, false);
    const int fppt = 2;  // pairs per thread; four measured 18 % slower (the two layout changes spill)
    int Rp = (m / 2) >= maxTp ? 1 : maxTp / (m / 2);
    if ((int64_t)Rp > B) Rp = (int)B;
    for (; Rp >= 1; Rp = (Rp > 1 ? Rp / 2 : 0)) {
      const int threads = (int)align_up((uint32_t)((Rp * (m / 2) + fppt - 1) / fppt), 32);
      const uint64_t RN = (uint64_t)Rp * N;
      uint64_t off = 0;
      auto take = [&](uint64_t bytes) { uint64_t o = off; off = (off + bytes + 127) / 128 * 128; return (uint32_t)o; };
      pl.off_work = take(RN * 8);
      pl.off_out = pl.off_work;
      pl.off_in[0] = pl.off_in[1] = residual ? take(RN * w) : pl.off_work;
      pl.off_ckpt = kNoOff;
      pl.off_red = 0;
      pl.off_w = take((uint64_t)16 * L);
      pl.off_bar = take(32);
      if (off > (uint64_t)dev.smem_optin) continue;
      pl.variant = fppt;
      pl.threads = threads; pl.R = Rp; pl.nbuf = 1; pl.n_ckpt_slots = 0; pl.smem = (size_t)off;
      pl.tiles = (B + Rp - 1) / Rp;
      int occ = 0;
      RowsParams dummy{};
      dummy.variant = fppt;
      cudaError_t e = pair_fn(n, false)(act, dtype, dummy, 0, pl.threads, pl.smem, nullptr, &occ);
      if (e != cudaSuccess) return cuda_fail(e);
      if (occ < 1) continue;
      if (occ > 32) occ = 32;
      long long grid = (long long)dev.sms * occ;
      if (grid > pl.tiles) grid = pl.tiles;
      pl.grid = (int)grid;
      return NCN_OK;
    }
    return NCN_ERR_SMEM;
  }
  const int items = pl.pair ? m / 2 : m;  // work items per row
  int maxT = pl.pair ? pair_max_threads(n, bwd) : rows_max_threads(n, bwd);
  int force_nbuf = 0;
  {  // tuning experiments
    const int t = bwd ? env_switches().bwd_threads : env_switches().fwd_threads;
    if (t >= 32 && t <= maxT && t % 32 == 0) maxT = t;
  }
  force_nbuf = env_switches().nbuf;
  const bool recompute = (flags & F_RECOMPUTE) != 0;
  if (recompute) n_ck = 0;
  int R = items >= maxT ? 1 : maxT / items;
  if ((int64_t)R > B) R = (int)B;
  const uint32_t limit = (uint32_t)dev.smem_optin;

  auto layout = [&](int R_, int nbuf, int slots, Plan& p) -> bool {
    const int threads = (int)align_up((uint32_t)((int64_t)R_ * items < maxT ? R_ * items : maxT), 32);
    const int nwarp = threads / 32;
    const uint64_t RN = (uint64_t)R_ * N;
    const uint64_t in_b = (bwd ? 4 : 2) * RN * w;
    const bool need_work = bwd ? (L > 1 || recompute) : (L > 1);
    const uint64_t work_b = need_work ? (bwd ? 4 : 2) * RN * 4 : 0;
    const uint64_t out_b = (bwd ? (want_rec ? 4 : 2) : 2) * RN * w;
    const uint64_t ck_b = (uint64_t)slots * 2 * RN * 4;
    uint64_t off = 0;
    auto take = [&](uint64_t bytes) { uint64_t o = off; off = (off + bytes + 127) / 128 * 128; return (uint32_t)o; };
    p.off_in[0] = take(in_b);
    p.off_in[1] = nbuf == 2 ? take(in_b) : p.off_in[0];
    p.off_work = take(work_b);
    p.off_out = take(out_b);
    p.off_ckpt = slots ? take(ck_b) : kNoOff;
    const uint64_t red_warp = bwd ? (uint64_t)2 * L * nwarp * 4 : 0;
    const uint64_t red_thr = (uint64_t)2 * L * threads * 4;
    const uint64_t fixed_rest = 16ull * L + 32 + 512;
    const bool rt = bwd && pl.pair && pl.variant == 1 && off + red_thr + fixed_rest <= limit;
    p.red_thread = rt;
    p.off_red = take(rt ? red_thr : red_warp);
    p.off_w = take((uint64_t)16 * L);  // one StageRec per stage
    p.off_bar = take(32);
    if (off > limit) return false;
    p.threads = threads;
    p.R = R_;
    p.nbuf = nbuf;
    p.n_ckpt_slots = (uint32_t)slots;
    p.smem = (size_t)off;
    return true;
  };

  bool ok = false;
  for (; R >= 1 && !ok; R = (R > 1 ? R / 2 : 0)) {
    if (bwd && n_ck > 0) {
      ok = layout(R, 1, n_ck, pl) || layout(R, 1, 0, pl);
    } else {
      // pair forward: a single input buffer leaves room for a second CTA on the SM, whose stages
      // overlap this one's stage boundaries; that is worth more than the earlier prefetch
      const bool prefer_one = pl.pair && !bwd && force_nbuf != 2;
      ok = (force_nbuf != 1 && !prefer_one && layout(R, 2, 0, pl)) || layout(R, 1, 0, pl);
    }
    if (ok) break;
  }
  if (!ok) return NCN_ERR_SMEM;
  pl.tiles = (B + pl.R - 1) / pl.R;
  int occ = 0;
  RowsParams dummy{};
  dummy.variant = pl.variant;
  cudaError_t e = (pl.pair ? pair_fn(n, bwd) : rows_fn(n, bwd))(act, dtype, dummy, 0, pl.threads, pl.smem, nullptr, &occ);
  if (e != cudaSuccess) return cuda_fail(e);
  if (occ < 1) return NCN_ERR_SMEM;
  if (occ > 32) occ = 32;
  long long grid = (long long)dev.sms * occ;
  if (grid > pl.tiles) grid = pl.tiles;
  pl.grid = (int)grid;
  return NCN_OK;
}

// Pair backward: the variant with separate buffers (one CTA per SM, full register budget, next
// tile prefetched) measured slightly faster than the aliased one (two CTAs per SM) and is tried
// first; NCN_BWD_WIDE=0 forces the aliased variant.
static int plan_rows_uncached(bool bwd, int64_t B, int N, int n, int L, int dtype, int flags, int n_ck, bool want_rec,
                              const DevInfo& dev, int act, Plan& pl) {
  const bool allow_wide = !env_switches().bwd_wide_off;
  // Plain backward of small groups: two pairs per thread in the aliased tile buffer, two CTAs per
  // SM with a full register budget; measured 6-8 % faster than the wide variant.  NCN_BWD_DUAL=0
  // switches it off.
  if (bwd && !env_switches().bwd_dual_off) {
    Plan trial;
    const int rc = plan_rows_impl(true, B, N, n, L, dtype, flags, n_ck, want_rec, dev, act, false, trial, true);
    if (rc == NCN_OK && trial.pair && trial.variant == 2) {
      pl = trial;
      return rc;
    }
  }
  if (bwd && allow_wide) {
    Plan trial;
    const int rc = plan_rows_impl(true, B, N, n, L, dtype, flags, n_ck, want_rec, dev, act, true, trial);
    if (rc == NCN_OK) {
      pl = trial;
      return rc;
    }
  }
  // Forward of small groups: one tile buffer, two pairs per thread, four CTAs per SM.
  // NCN_FWD_DUAL=0 switches it off.
  if (!bwd && !env_switches().fwd_dual_off) {
    Plan trial;
    const int rc = plan_rows_impl(false, B, N, n, L, dtype, flags, n_ck, want_rec, dev, act, false, trial, true);
    if (rc == NCN_OK && trial.pair && trial.variant >= 2) {
      pl = trial;
      return rc;
    }
  }
  pl = Plan();
  return plan_rows_impl(bwd, B, N, n, L, dtype, flags, n_ck, want_rec, dev, act, false, pl);
}

// A plan costs up to three layouts, each with a cudaFuncSetAttribute and an occupancy query; it
// depends on nothing but these arguments and the device, so it is computed once per argument set.
struct RowsKey {
  int epoch, dev, bwd, N, n, L, dtype, flags, n_ck, want_rec, act;
  long long B;
  bool operator==(const RowsKey& o) const {
    return epoch == o.epoch && dev == o.dev && bwd == o.bwd && N == o.N && n == o.n && L == o.L && dtype == o.dtype && flags == o.flags &&
           n_ck == o.n_ck && want_rec == o.want_rec && act == o.act && B == o.B;
  }
};

static int plan_rows(bool bwd, int64_t B, int N, int n, int L, int dtype, int flags, int n_ck, bool want_rec,
                     const DevInfo& dev, int act, Plan& pl) {
  static std::mutex mu;
  static std::vector<std::pair<RowsKey, std::pair<int, Plan>>> cache;
  const RowsKey key{g_plan_epoch.load(), dev.dev, bwd ? 1 : 0, N, n, L, dtype, flags, n_ck, want_rec ? 1 : 0, act, (long long)B};
  {
    std::lock_guard<std::mutex> lk(mu);
    for (auto& kv : cache)
      if (kv.first == key) {
        pl = kv.second.second;
        return kv.second.first;
      }
  }
  const int rc = plan_rows_uncached(bwd, B, N, n, L, dtype, flags, n_ck, want_rec, dev, act, pl);
  if (rc != NCN_ERR_CUDA) {
    std::lock_guard<std::mutex> lk(mu);
    if (cache.size() >= 64) cache.erase(cache.begin());
    cache.emplace_back(key, std::make_pair(rc, pl));
  }
  return rc;
}

// ---- register-resident row kernels (ncn_lanes.cuh)
typedef cudaError_t (*LaneLaunchFn)(int, int, const LaneParams&, int, int, size_t, cudaStream_t, int*);

static LaneLaunchFn lane_fn(int n, bool bwd) {
  switch (n) {
    case 2: return bwd ? launch_lane_bwd_n2 : launch_lane_fwd_n2;
    case 4: return bwd ? launch_lane_bwd_n4 : launch_lane_fwd_n4;
    case 8: return bwd ? launch_lane_bwd_n8 : launch_lane_fwd_n8;
    default: return nullptr;
  }
}

// NCN_LANES=0 switches the family off (A/B measurements); read once.
// NCN_LANES=0 switches the register-resident family off, NCN_LANES_PIPE=0 its pipelined backward
// (A/B measurements).
static bool lanep_enabled() { return !env_switches().lanes_pipe_off; }
static bool lanes_enabled() { return !env_switches().lanes_off; }

struct LanePlan {
  int threads = 0, R = 0, grid = 0, tpr = 0, ea_max = 0, occ = 0;
  size_t smem = 0;
  uint32_t off_work = 0, off_res = 0, off_ckpt = 0, off_halo = 0, off_red = 0, off_w = 0, off_bar = 0;
  uint32_t halo_warp_bytes = 0, n_ckpt_slots = 0;
  int pipelined = 0;
  long long tiles = 0;
};

static int lane_ilog2(long long v) {
  int e = 0;
  while ((1LL << (e + 1)) <= v) ++e;
  return e;
}

// The family covers: one feature per position, n in {2,4,8}, m = N/n a power of two with a whole
// number of warps per row and at most one CTA of threads per row, and stage strides that do not
// wrap (2^(l-1) < m for every stage), so that every change of stride is a shift by a power of two.
static bool lane_shape_ok(int64_t N, int64_t E, int n, int C, int l0, int L, int dtype, int* e_needed_max) {
  if (E != 1 || C != 1 || lane_fn(n, false) == nullptr) return false;
  if (N % n != 0) return false;
  const int64_t m = N / n;
  if (m <= 0 || (m & (m - 1)) != 0) return false;
  const int G = lane_groups(n);
  if (m % (32 * G) != 0 || m / G > kLaneThreads) return false;
  const int64_t quantum = dtype == DT_BF16 ? 8 : 4;
  if (N % quantum != 0) return false;
  const int last = l0 + L - 1;
  if (last >= 1 && (last - 1) >= lane_ilog2(m)) return false;  // 2^(last-1) >= m: the stride wraps
  // largest shift: back from the last stride to 0 (2^(last-1)), or the first one up to stride(l0)
  int emax = -1;
  if (last >= 1) emax = last - 1;
  *e_needed_max = emax;
  return true;
}

// Lay one CTA out.  ea: shifts of up to 2^ea blocks go by shuffles + halo, longer ones through the
// tile buffer (which must then hold fp32 values).
static bool lane_layout(bool bwd, int N, int n, int L, int dtype, int flags, int n_ck, int R, int tpr, int ea, int e_need,
                        uint32_t limit, LanePlan& pl) {
  const int w = dtype == DT_BF16 ? 2 : 4;
  const int NS = bwd ? 4 : 2;
  const bool residual = (flags & F_RESIDUAL) != 0;
  const bool long_shifts = e_need > ea;
  const uint64_t RN = (uint64_t)R * N;
  const int threads = R * tpr;
  const int warps = threads / 32;
  uint64_t off = 0;
  auto take = [&](uint64_t bytes) { uint64_t o = off; off = (off + bytes + 127) / 128 * 128; return (uint32_t)o; };
  pl.off_work = take(NS * RN * (long_shifts ? 4 : w));
  pl.off_res = residual ? take(RN * w) : pl.off_work;
  pl.off_ckpt = take(n_ck ? (uint64_t)n_ck * RN * 8 : 16);
  pl.halo_warp_bytes = ea >= 0 ? (uint32_t)(NS * lane_halo_floats(n, ea) * 4) : 0;
  pl.halo_warp_bytes = (pl.halo_warp_bytes + 15u) / 16u * 16u;
  pl.off_halo = take((uint64_t)2 * warps * pl.halo_warp_bytes + 16);
  pl.off_red = take(bwd ? (uint64_t)2 * L * warps * 4 : 16);
  pl.off_w = take((uint64_t)16 * L);
  pl.off_bar = take(32);
  if (off > limit) return false;
  pl.threads = threads; pl.R = R; pl.tpr = tpr; pl.ea_max = ea; pl.smem = (size_t)off;
  pl.n_ckpt_slots = (uint32_t)n_ck;
  return true;
}

// Pipelined backward (n = 4, ncn_lanes_pipe.cuh): a thread runs the two halves of its row half a
// stage apart; every shift goes by shuffles + halo, and the halo lives in the tile buffer.  Needs
// every change of stride to stay within a warp's reach: 3 * 2^e / 2 <= 24 lanes, i.e. e <= 4.
static bool lanep_layout(bool bwd, int N, int L, int dtype, int flags, int n_ck, int R, int tpr, int e_need, uint32_t limit,
                         LanePlan& pl) {
  if (e_need > 4) return false;
  const int NS = bwd ? 4 : 2;  // streams a thread holds
  const int w = dtype == DT_BF16 ? 2 : 4;
  const bool residual = (flags & F_RESIDUAL) != 0;
  const uint64_t RN = (uint64_t)R * N;
  const int threads = R * tpr;
  const int warps = threads / 32;
  pl.halo_warp_bytes = NS * 3 * kPipeSo;  // a region of kPipeSo bytes per (stream, offset): enough for shifts of 3 * 2^4 blocks
  uint64_t work = NS * RN * w;
  const uint64_t halo = (uint64_t)2 * warps * pl.halo_warp_bytes;  // two half-row "warps" per warp
  if (halo > work) work = halo;
  uint64_t off = 0;
  auto take = [&](uint64_t bytes) { uint64_t o = off; off = (off + bytes + 127) / 128 * 128; return (uint32_t)o; };
  pl.off_work = take(work);
  pl.off_halo = pl.off_work;
  pl.off_res = residual ? take(RN * w) : pl.off_work;
  pl.off_ckpt = take(bwd && n_ck ? (uint64_t)n_ck * RN * 8 : 16);  // (the forward stores its states straight to global memory)
  pl.off_red = take((uint64_t)2 * L * warps * 4);
  pl.off_w = take((uint64_t)16 * L);
  pl.off_bar = take(32);
  if (off > limit) return false;
  pl.threads = threads; pl.R = R; pl.tpr = tpr; pl.ea_max = 4; pl.smem = (size_t)off;
  pl.n_ckpt_slots = (uint32_t)n_ck;
  pl.pipelined = 1;
  return true;
}

struct LaneKey {
  int epoch, dev, bwd, N, n, L, l0, dtype, flags, n_ck, act;
  long long B;
  bool operator==(const LaneKey& o) const {
    return epoch == o.epoch && dev == o.dev && bwd == o.bwd && N == o.N && n == o.n && L == o.L && l0 == o.l0 && dtype == o.dtype &&
           flags == o.flags && n_ck == o.n_ck && act == o.act && B == o.B;
  }
};

// NCN_OK with pl filled, NCN_ERR_UNSUPPORTED when the family does not cover the arguments.
// Plans are remembered per argument set: a plan costs a few occupancy queries.
static int plan_lanes(bool bwd, int64_t B, int64_t N, int64_t E, int n, int C, int l0, int L, int dtype, int flags,
                      int n_ck, const DevInfo& dev, int act, LanePlan& pl) {
  if (!lanes_enabled()) return NCN_ERR_UNSUPPORTED;
  if (flags & F_RECOMPUTE) return NCN_ERR_UNSUPPORTED;
  int e_need = -1;
  if (!lane_shape_ok(N, E, n, C, l0, L, dtype, &e_need)) return NCN_ERR_UNSUPPORTED;
  static std::mutex mu;
  static std::vector<std::pair<LaneKey, std::pair<int, LanePlan>>> cache;
  const LaneKey key{g_plan_epoch.load(), dev.dev, bwd ? 1 : 0, (int)N, n, L, l0, dtype, flags & (F_RESIDUAL | F_TAPE), n_ck, act, (long long)B};
  {
    std::lock_guard<std::mutex> lk(mu);
    for (auto& kv : cache)
      if (kv.first == key) {
        pl = kv.second.second;
        return kv.second.first;
      }
  }
  const int G = lane_groups(n);
  const int tpr = (int)(N / n) / G;
  int R = kLaneThreads / tpr;
  {
    // A CTA is one barrier domain.  With plenty of tiles per CTA, halves of kLaneThreads do better (more,
    // smaller domains per SM drift apart and fill each other's waits: the 12-layer bf16 stack 89.7 -> 84.3 ms);
    // with about one tile per CTA the per-CTA set-up counts and the larger tile wins (1024 x 1024: 0.23 against
    // 0.28 ms backward).
    const int r_small = kLaneThreads / 2 / tpr;
    if (r_small >= 1 && B / r_small >= 8LL * dev.sms * (bwd ? kLaneBwdBlocks : kLaneFwdBlocks) * 2) R = r_small;
  }
  if (env_switches().lane_rows > 0 && R > env_switches().lane_rows) R = env_switches().lane_rows;
  if ((int64_t)R > B) R = (int)B;
  if (R < 1) R = 1;
  // the register budget allows kLane*Blocks CTAs of kLaneThreads threads: smaller CTAs, more of them
  const int want_occ = (bwd ? kLaneBwdBlocks : kLaneFwdBlocks) * (kLaneThreads / (R * tpr));
  const int cap = lane_ea_cap(n);
  int ea_hi = e_need < cap ? e_need : cap;
  int ea_lo = lane_ilog2(G) - 1;  // longer shifts through the tile buffer must be multiples of G blocks
  if (ea_lo > ea_hi) ea_lo = ea_hi;
  int rc = NCN_ERR_UNSUPPORTED;
  LanePlan best;
  bool have_pipe = false;
  if (n == 4 && (bwd ? lanep_enabled() : env_switches().lanes_pipe_fwd)) {
    LanePlan trial;
    if (lanep_layout(bwd, (int)N, L, dtype, flags, n_ck, R, tpr, e_need, (uint32_t)dev.smem_optin, trial)) {
      int occ = 0;
      LaneParams dummy{};
      dummy.pipelined = 1;
      cudaError_t e = lane_fn(n, bwd)(act, dtype, dummy, 0, trial.threads, trial.smem, nullptr, &occ);
      if (e != cudaSuccess) return cuda_fail(e);
      if (occ >= 1) {
        trial.occ = occ > want_occ ? want_occ : occ;
        best = trial;
        rc = NCN_OK;
        have_pipe = true;
      }
    }
  }
  for (int ea = ea_hi; !have_pipe && ea >= ea_lo; --ea) {
    LanePlan trial;
    if (!lane_layout(bwd, (int)N, n, L, dtype, flags, n_ck, R, tpr, ea, e_need, (uint32_t)dev.smem_optin, trial)) continue;
    int occ = 0;
    LaneParams dummy{};
    cudaError_t e = lane_fn(n, bwd)(act, dtype, dummy, 0, trial.threads, trial.smem, nullptr, &occ);
    if (e != cudaSuccess) return cuda_fail(e);
    if (occ < 1) continue;
    if (occ > want_occ) occ = want_occ;
    trial.occ = occ;
    if (rc != NCN_OK || occ > best.occ) { best = trial; rc = NCN_OK; }
    if (occ >= want_occ) break;
  }
  if (rc == NCN_OK) {
    best.tiles = (B + best.R - 1) / best.R;
    long long grid = (long long)dev.sms * best.occ;
    if (grid > best.tiles) grid = best.tiles;
    best.grid = (int)grid;
    pl = best;
  }
  {
    std::lock_guard<std::mutex> lk(mu);
    if (cache.size() >= 64) cache.erase(cache.begin());
    cache.emplace_back(key, std::make_pair(rc, pl));
  }
  return rc;
}

static void fill_lane(LaneParams& p, const LanePlan& pl) {
  p.R = pl.R; p.tpr = pl.tpr; p.ea_max = pl.ea_max; p.tiles = pl.tiles;
  p.off_work = pl.off_work; p.off_res = pl.off_res; p.off_ckpt = pl.off_ckpt; p.off_halo = pl.off_halo;
  p.off_red = pl.off_red; p.off_w = pl.off_w; p.off_bar = pl.off_bar;
  p.halo_warp_bytes = pl.halo_warp_bytes; p.n_ckpt_slots = pl.n_ckpt_slots;
  p.pipelined = pl.pipelined;
}

static void fill_offsets(RowsParams& p, const Plan& pl) {
  p.off_in[0] = pl.off_in[0];
  p.off_in[1] = pl.off_in[1];
  p.off_work = pl.off_work;
  p.off_out = pl.off_out;
  p.off_ckpt = pl.off_ckpt;
  p.off_red = pl.off_red;
  p.off_w = pl.off_w;
  p.off_bar = pl.off_bar;
  p.n_ckpt_slots = pl.n_ckpt_slots;
  p.variant = pl.variant;
  p.R = pl.R;
  p.nbuf = pl.nbuf;
  p.tiles = pl.tiles;
}

static int check_common(int64_t B, int64_t N, int64_t E, int n, int C, int dtype) {
  if (B <= 0 || N <= 0 || E <= 0 || n <= 0 || C <= 0) return NCN_ERR_SHAPE;
  if (N % n != 0 || E % C != 0) return NCN_ERR_SHAPE;
  if (N > (1LL << 30) || E > (1LL << 24)) return NCN_ERR_SHAPE;
  if (dtype != DT_F32 && dtype != DT_BF16) return NCN_ERR_DTYPE;
  return NCN_OK;
}

static int reduce_dw(const float* partials, float* dW, int rows, int cols, int accumulate, cudaStream_t st) {
  const int warps = 4;
  dw_reduce_kernel<<<(cols + warps - 1) / warps, warps * 32, 0, st>>>(partials, dW, rows, cols, accumulate);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? NCN_OK : cuda_fail(e);
}

// ---- generic per-stage launches
struct GenericPlan {
  int warps = 0, grid = 0;
  size_t smem = 0;
  uint32_t warp_floats = 0;
};

template <typename K>
static int plan_generic(K kernel, bool bwd, int64_t groups, int n, int d, int E, const DevInfo& dev, GenericPlan& g) {
  const int pitch = d | 1;
  const uint64_t wf = bwd ? (uint64_t)5 * n * pitch + d + 2 * n + 2 * E : (uint64_t)2 * n * pitch + d + n;
  int warps = 8;
  while (warps > 1 && wf * 4 * warps > (uint64_t)dev.smem_optin) warps /= 2;
  if (wf * 4 * warps > (uint64_t)dev.smem_optin) return NCN_ERR_SMEM;
  g.warps = warps;
  g.warp_floats = (uint32_t)wf;
  g.smem = (size_t)(wf * 4 * warps);
  // The occupancy is remembered per (kernel, device, CTA shape); the shared-memory attribute is only ever raised
  // (a later, smaller request must not lower what an earlier, larger launch shape still needs).
  struct Seen { const void* k; int dev, warps; size_t smem; int occ; };
  struct Grant { const void* k; int dev; size_t bytes; };
  static std::mutex mu;
  static std::vector<Seen> seen;
  static std::vector<Grant> grants;
  int occ = -1;
  {
    std::lock_guard<std::mutex> lk(mu);
    for (const Seen& q : seen)
      if (q.k == (const void*)kernel && q.dev == dev.dev && q.warps == warps && q.smem == g.smem) { occ = q.occ; break; }
  }
  if (occ < 0) {
    std::lock_guard<std::mutex> lk(mu);
    Grant* gr = nullptr;
    for (Grant& q : grants)
      if (q.k == (const void*)kernel && q.dev == dev.dev) { gr = &q; break; }
    if (gr == nullptr || gr->bytes < g.smem) {
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g.smem);
      if (e != cudaSuccess) return cuda_fail(e);
      if (gr) gr->bytes = g.smem; else grants.push_back(Grant{(const void*)kernel, dev.dev, g.smem});
    }
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kernel, warps * 32, g.smem);
    if (e != cudaSuccess) return cuda_fail(e);
    if (seen.size() >= 64) seen.clear();
    seen.push_back(Seen{(const void*)kernel, dev.dev, warps, g.smem, occ});
  }
  if (occ < 1) return NCN_ERR_SMEM;
  if (occ > 8) occ = 8;
  long long grid = (groups + warps - 1) / warps;
  if (grid > (long long)dev.sms * occ) grid = (long long)dev.sms * occ;
  g.grid = (int)grid;
  return NCN_OK;
}

static void fill_stage(StageParams& p, int64_t B, int64_t N, int64_t E, int n, int C, int module_l, double alpha) {
  p.B = B;
  p.N = (int)N;
  p.E = (int)E;
  p.C = C;
  p.d = (int)(E / C);
  p.n = n;
  p.m = (int)(N / n);
  p.groups = B * C * (N / n);
  p.stride = stage_stride(module_l, p.m);
  p.pitch = p.d | 1;
  int sh = 0;
  while (sh < 5 && (2 << sh) <= p.d) ++sh;
  p.ld_shift = sh;
  p.alpha = (float)alpha;
  p.oma = (float)(1.0 - alpha);
}

// ---- register-tiled multi-feature stage kernels (ncn_feat.cuh)
typedef cudaError_t (*FeatLaunchFn)(int, int, int, const FeatParamsX&, int, int, cudaStream_t, int*);

static FeatLaunchFn feat_fn(int n, bool bwd) {
  switch (n) {
    case 2: return bwd ? launch_feat_bwd_n2 : launch_feat_fwd_n2;
    case 4: return bwd ? launch_feat_bwd_n4 : launch_feat_fwd_n4;
    case 8: return bwd ? launch_feat_bwd_n8 : launch_feat_fwd_n8;
    case 16: return bwd ? launch_feat_bwd_n16 : launch_feat_fwd_n16;
    case 32: return bwd ? launch_feat_bwd_n32 : launch_feat_fwd_n32;
    default: return nullptr;
  }
}

static FeatLaunchFn feat_mid_fn(int n) {
  switch (n) {
    case 16: return launch_feat_fwdm_n16;
    case 32: return launch_feat_fwdm_n32;
    default: return nullptr;
  }
}

static FeatLaunchFn feat_saved_fn(int n) {
  switch (n) {
    case 16: return launch_feat_bwds_n16;
    case 32: return launch_feat_bwds_n32;
    default: return nullptr;
  }
}

static long long gcd_ll(long long a, long long b) {
  while (b) { const long long t = a % b; a = b; b = t; }
  return a;
}

// NCN_OK: launched.  NCN_ERR_UNSUPPORTED: no such kernel for these arguments (the caller falls
// back to the shared-memory kernels); anything else is an error.
static int launch_feat(bool bwd, const void* const* in, void* const* out, const float* W, float* partials, int64_t B,
                       int64_t N, int64_t E, int n, int C, int module_l, double alpha, int activation, int dtype,
                       const DevInfo& dev, cudaStream_t st, int* grid_out, const void* x_saved = nullptr,
                       const void* xa_saved = nullptr, int saved = 0, float* mid = nullptr, int mid_end = 0) {
  const int d = (int)(E / C);
  const int gpw = feat_groups_per_warp(n, d);
  FeatLaunchFn fn = saved ? feat_saved_fn(n) : (mid && !bwd) ? feat_mid_fn(n) : feat_fn(n, bwd);
  if (saved && saved != 3 && (!aligned16(x_saved) || !aligned16(xa_saved))) return NCN_ERR_UNSUPPORTED;
  if (mid && !aligned16(mid)) return NCN_ERR_UNSUPPORTED;
  if (gpw == 0 || fn == nullptr || map_act(activation) == ACT_LEAKY) return NCN_ERR_UNSUPPORTED;
  if (env_switches().no_feat) return NCN_ERR_UNSUPPORTED;  // tuning experiments: force the shared-memory kernels
  const int act = fused_act(map_act(activation), dtype);
  for (int q = 0; q < (bwd ? 4 : 2); ++q)
    if (!aligned16(in[q])) return NCN_ERR_UNSUPPORTED;  // (null, where a mode does not read a tensor, counts as aligned)
  for (int q = 0; q < (bwd ? 4 : 2); ++q)
    if (out[q] && !aligned16(out[q])) return NCN_ERR_UNSUPPORTED;
  FeatParamsX p{};
  for (int q = 0; q < 4; ++q) { p.in[q] = in[q]; p.out[q] = out[q]; }
  p.xin[0] = x_saved; p.xin[1] = xa_saved;
  p.saved = saved;
  p.mid = mid; p.mid_end = mid_end; p.bne = B * N * E;
  p.W = W;
  p.partials = partials;
  p.B = B; p.N = (int)N; p.E = (int)E; p.C = C;
  p.m = (int)(N / n);
  p.mg = (p.m + gpw - 1) / gpw;
  p.units = B * p.mg;
  p.stride = stage_stride(module_l, p.m);
  p.alpha = (float)alpha;
  p.oma = (float)(1.0 - alpha);
  // few groups (the reference's own bench has 128): smaller CTAs, so that the warps spread over all SMs
  const long long want_warps = p.units * C;
  int wpc = kFeatWarps;
  while (wpc > 1 && want_warps < (long long)dev.sms * wpc) wpc /= 2;
  const int threads = wpc * 32;
  // resident CTAs per SM of this kernel: asked once per (kernel, device, CTA size)
  struct Seen { FeatLaunchFn fn; int d, act, dtype, threads, dev, occ; };
  static std::mutex mu;
  static std::vector<Seen> seen;
  int occ = -1;
  {
    std::lock_guard<std::mutex> lk(mu);
    for (const Seen& q : seen)
      if (q.fn == fn && q.d == d && q.act == act && q.dtype == dtype && q.threads == threads && q.dev == dev.dev) { occ = q.occ; break; }
  }
  cudaError_t e = cudaSuccess;
  if (occ < 0) {
    occ = 0;
    e = fn(d, act, dtype, p, 0, threads, nullptr, &occ);
    if (e == cudaErrorNotSupported) return NCN_ERR_UNSUPPORTED;
    if (e != cudaSuccess) return cuda_fail(e);
    std::lock_guard<std::mutex> lk(mu);
    if (seen.size() >= 128) seen.clear();
    seen.push_back(Seen{fn, d, act, dtype, threads, dev.dev, occ});
  }
  if (occ < 1) return NCN_ERR_UNSUPPORTED;
  if (occ > 32) occ = 32;
  // one warp per (head, unit) at most, a whole number of warps per head
  long long grid = (want_warps + wpc - 1) / wpc;
  if (grid > (long long)dev.sms * occ) grid = (long long)dev.sms * occ;
  const long long q = C / gcd_ll(C, wpc);
  grid = (grid + q - 1) / q * q;
  if (grid > (long long)dev.sms * 32) return NCN_ERR_UNSUPPORTED;  // more heads than the workspace covers
  e = fn(d, act, dtype, p, (int)grid, threads, st, nullptr);
  if (e != cudaSuccess) return cuda_fail(e);
  if (grid_out) *grid_out = (int)grid;
  return NCN_OK;
}

// ---- per-stage launches of the shared-memory kernels (any E, heads, n_cache; optional per-row context length)
static int stage_fwd_generic(const void* x, const void* xa, const float* W, const int* ctxlen, void* y, void* ya, int64_t B,
                             int64_t N, int64_t E, int n_cache, int n_head, int module_l, double alpha, int activation,
                             int dtype, const DevInfo& dev, void* stream, float* mid = nullptr, int mid_end = 0) {
  StageParams p{};
  fill_stage(p, B, N, E, n_cache, n_head, module_l, alpha);
  p.in[0] = x; p.in[1] = xa;
  p.out[0] = y; p.out[1] = ya;
  p.W = W;
  p.ctxlen = ctxlen;
  p.mid = mid; p.mid_end = mid_end; p.bne = B * N * E;
  GenericPlan g;
  int rc;
  const int act = map_act(activation);
  if (dtype == DT_BF16) {
    if ((rc = plan_generic(stage_fwd_kernel<__nv_bfloat16>, false, p.groups, p.n, p.d, p.E, dev, g)) != NCN_OK) return rc;
    p.warps = g.warps; p.warp_floats = g.warp_floats;
    stage_fwd_kernel<__nv_bfloat16><<<g.grid, g.warps * 32, g.smem, (cudaStream_t)stream>>>(p, act);
  } else {
    if ((rc = plan_generic(stage_fwd_kernel<float>, false, p.groups, p.n, p.d, p.E, dev, g)) != NCN_OK) return rc;
    p.warps = g.warps; p.warp_floats = g.warp_floats;
    stage_fwd_kernel<float><<<g.grid, g.warps * 32, g.smem, (cudaStream_t)stream>>>(p, act);
  }
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? NCN_OK : cuda_fail(e);
}

static int stage_bwd_generic(const void* y, const void* ya, const void* dy, const void* dya, const float* W,
                             const int* ctxlen, void* dx, void* dxa, void* x_rec, void* xa_rec, float* dW, float* partials,
                             int64_t B, int64_t N, int64_t E, int n_cache, int n_head, int module_l, double alpha,
                             int activation, int dtype, const DevInfo& dev, void* stream, const void* x_saved = nullptr,
                             const void* xa_saved = nullptr, int replay_all = 0, const float* mid = nullptr,
                             int mid_end = 0) {
  StageParams p{};
  fill_stage(p, B, N, E, n_cache, n_head, module_l, alpha);
  p.xin[0] = x_saved; p.xin[1] = xa_saved;
  p.replay_all = replay_all;
  p.mid = const_cast<float*>(mid); p.mid_end = mid_end; p.bne = B * N * E;
  p.in[0] = y; p.in[1] = ya; p.in[2] = dy; p.in[3] = dya;
  p.out[0] = dx; p.out[1] = dxa; p.out[2] = x_rec; p.out[3] = xa_rec;
  p.W = W;
  p.ctxlen = ctxlen;
  p.partials = partials;
  GenericPlan g;
  int rc;
  const int act = map_act(activation);
  if (dtype == DT_BF16) {
    if ((rc = plan_generic(stage_bwd_kernel<__nv_bfloat16>, true, p.groups, p.n, p.d, p.E, dev, g)) != NCN_OK) return rc;
    p.warps = g.warps; p.warp_floats = g.warp_floats;
    stage_bwd_kernel<__nv_bfloat16><<<g.grid, g.warps * 32, g.smem, (cudaStream_t)stream>>>(p, act);
  } else {
    if ((rc = plan_generic(stage_bwd_kernel<float>, true, p.groups, p.n, p.d, p.E, dev, g)) != NCN_OK) return rc;
    p.warps = g.warps; p.warp_floats = g.warp_floats;
    stage_bwd_kernel<float><<<g.grid, g.warps * 32, g.smem, (cudaStream_t)stream>>>(p, act);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e);
  return reduce_dw(p.partials, dW, g.grid, 2 * (int)E, 0, (cudaStream_t)stream);
}

static size_t workspace_floats(const DevInfo& dev, int64_t E, int L) {
  return (size_t)dev.sms * 32 * 2 * (size_t)E * (size_t)(L < 1 ? 1 : L);
}

}  // namespace ncn

using namespace ncn;

extern "C" {

int ncn_version(void) { return 103; }

void ncn_reload_env(void) {
  g_env = read_env_switches();
  g_plan_epoch.fetch_add(1);
}

const char* ncn_status_string(int s) {
  switch (s) {
    case NCN_OK: return "ok";
    case NCN_ERR_SHAPE: return "bad shape: n_cache must divide N, n_head must divide E, all sizes positive";
    case NCN_ERR_DTYPE: return "unsupported dtype (fp32 and bf16 only)";
    case NCN_ERR_ALIGN: return "tensor pointer not 16-byte aligned";
    case NCN_ERR_SMEM: return "tile does not fit in shared memory";
    case NCN_ERR_UNSUPPORTED: return "fused all-stage path does not cover these arguments";
    case NCN_ERR_WORKSPACE: return "workspace missing or too small";
    case NCN_ERR_CUDA: return "CUDA runtime error";
    case NCN_ERR_NULL: return "null pointer";
    case NCN_ERR_DEVICE_WAIT: return "a kernel abandoned a bounded wait on an asynchronous copy";
    case NCN_ERR_TOO_LARGE: return "problem needs more scratch than the fixed array of ncn_net_bwd_noalloc holds";
    default: return "unknown status";
  }
}

const char* ncn_last_cuda_error(void) { return tl_cuda_err; }

int ncn_device_status(void) {
  int v = 0, zero = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_status_word, sizeof(int));
  if (e != cudaSuccess) return cuda_fail(e);
  if (v != 0) {
    e = cudaMemcpyToSymbol(g_status_word, &zero, sizeof(int));
    if (e != cudaSuccess) return cuda_fail(e);
    return NCN_ERR_DEVICE_WAIT;
  }
  return NCN_OK;
}

size_t ncn_bwd_workspace_bytes(int64_t B, int64_t N, int64_t E, int n_cache, int n_head, int L, int dtype) {
  (void)B; (void)N; (void)n_cache; (void)n_head; (void)dtype;
  DevInfo dev;
  if (get_dev(dev) != NCN_OK) return 0;
  return workspace_floats(dev, E, L) * sizeof(float);
}

// stored states: one after every ckpt_every-th stage except the last, plus the last one with F_TAPE
static int ckpt_slots(int L, int ckpt_every, int flags) {
  if (L < 1) return 0;
  return (ckpt_every > 0 ? (L - 1) / ckpt_every : 0) + ((flags & F_TAPE) ? 1 : 0);
}

size_t ncn_ckpt_bytes(int64_t B, int64_t N, int64_t E, int L, int ckpt_every, int flags) {
  return (size_t)ckpt_slots(L, ckpt_every, flags) * 2 * (size_t)B * (size_t)N * (size_t)E * sizeof(float);
}

int ncn_net_supported(int64_t B, int64_t N, int64_t E, int n_cache, int n_head, int L, int dtype, int flags,
                      int ckpt_every) {
  if (check_common(B, N, E, n_cache, n_head, dtype) != NCN_OK || L < 1) return 0;
  if (!rows_shape_ok(N, E, n_cache, n_head, dtype)) return 0;
  DevInfo dev;
  if (get_dev(dev) != NCN_OK) return 0;
  Plan pl;
  if ((flags & F_TAPE) && (flags & F_RECOMPUTE)) return 0;
  const int n_ck = (flags & F_RECOMPUTE) ? 0 : ckpt_slots(L, ckpt_every, flags);
  {
    LanePlan lf, lb;
    const int act = fused_act(ACT_TANH, dtype);
    if (plan_lanes(false, B, N, E, n_cache, n_head, 0, L, dtype, flags, 0, dev, act, lf) == NCN_OK &&
        plan_lanes(true, B, N, E, n_cache, n_head, 0, L, dtype, flags, n_ck, dev, act, lb) == NCN_OK)
      return 1;
  }
  if (plan_rows(false, B, (int)N, n_cache, L, dtype, flags, 0, false, dev, ACT_TANH, pl) != NCN_OK) return 0;
  if (plan_rows(true, B, (int)N, n_cache, L, dtype, flags, n_ck, false, dev, ACT_TANH, pl) != NCN_OK) return 0;
  return 1;
}

int ncn_net_fwd(const void* x, const void* xa, const float* W, void* y, void* ya, float* ckpt, int ckpt_every,
                int64_t B, int64_t N, int64_t E, int n_cache, int n_head, int first_module, int L, double alpha,
                int activation, int dtype, int flags, void* stream) {
  int rc = check_common(B, N, E, n_cache, n_head, dtype);
  if (rc != NCN_OK) return rc;
  if (L < 1 || first_module < 0) return NCN_ERR_SHAPE;
  if (!x || !xa || !W || !y || !ya) return NCN_ERR_NULL;
  if ((flags & F_TAPE) && !ckpt) return NCN_ERR_NULL;
  if (!rows_shape_ok(N, E, n_cache, n_head, dtype) || map_act(activation) == ACT_LEAKY) return NCN_ERR_UNSUPPORTED;
  if (!aligned16(x) || !aligned16(xa) || !aligned16(y) || !aligned16(ya) || (ckpt && !aligned16(ckpt)))
    return NCN_ERR_ALIGN;
  DevInfo dev;
  if ((rc = get_dev(dev)) != NCN_OK) return rc;
  const int act = fused_act(map_act(activation), dtype);
  float* ck_used = (ckpt && ckpt_slots(L, ckpt_every, flags) > 0) ? ckpt : nullptr;
  {
    // register-resident family; its stored states have their own order, so with states it is used
    // only where the backward of the same arguments is of this family too
    LanePlan lp, lb;
    const int n_ck = ck_used ? ckpt_slots(L, ckpt_every, flags) : 0;
    bool lanes = plan_lanes(false, B, N, E, n_cache, n_head, first_module, L, dtype, flags, 0, dev, act, lp) == NCN_OK;
    if (lanes && n_ck > 0)
      lanes = plan_lanes(true, B, N, E, n_cache, n_head, first_module, L, dtype, flags, n_ck, dev, act, lb) == NCN_OK;
    if (lanes) {
      LaneParams q{};
      q.in[0] = x; q.in[1] = xa;
      q.out[0] = y; q.out[1] = ya;
      q.ckpt = ck_used;
      q.ckpt_every = ckpt_every;
      q.W = W;
      q.status = dev.status;
      q.B = B; q.N = (int)N; q.m = (int)(N / n_cache); q.L = L; q.l0 = first_module;
      q.flags = flags & (F_RESIDUAL | F_TAPE);
      q.alpha = (float)alpha;
      q.oma = (float)(1.0 - alpha);
      fill_lane(q, lp);
      q.test_short_wait = env_switches().test_short_wait ? 1 : 0;
      cudaError_t e = lane_fn(n_cache, false)(act, dtype, q, lp.grid, lp.threads, lp.smem, (cudaStream_t)stream, nullptr);
      return e == cudaSuccess ? NCN_OK : cuda_fail(e);
    }
  }
  Plan pl;
  if ((rc = plan_rows(false, B, (int)N, n_cache, L, dtype, flags, 0, false, dev, act, pl)) != NCN_OK) return rc;
  RowsParams p{};
  p.in[0] = x; p.in[1] = xa;
  p.out[0] = y; p.out[1] = ya;
  p.ckpt = ck_used;
  p.ckpt_every = ckpt_every;
  p.W = W;
  p.status = dev.status;
  p.B = B; p.N = (int)N; p.m = (int)(N / n_cache); p.L = L; p.l0 = first_module;
  p.flags = flags & (F_RESIDUAL | F_TAPE);
  p.alpha = (float)alpha;
  p.oma = (float)(1.0 - alpha);
  fill_offsets(p, pl);
  cudaError_t e = (pl.pair ? pair_fn(n_cache, false) : rows_fn(n_cache, false))(act, dtype, p, pl.grid, pl.threads, pl.smem,
                                                                               (cudaStream_t)stream, nullptr);
  return e == cudaSuccess ? NCN_OK : cuda_fail(e);
}

// Backward of a net, shared by ncn_net_bwd and ncn_net_bwd_noalloc: `partials` is the scratch for the
// per-CTA weight-gradient sums (capacity_floats of it); a launch that needs more returns short_err.
static int net_bwd_impl(const void* s0, const void* s1, const void* dy, const void* dya, const float* W, void* dx,
                        void* dxa, void* x_rec, void* xa_rec, float* dW, const float* ckpt, int ckpt_every,
                        float* partials, size_t capacity_floats, bool full_workspace, int short_err, int64_t B,
                        int64_t N, int64_t E,
                        int n_cache, int n_head, int first_module, int L, double alpha, int activation, int dtype,
                        int flags, int dw_accumulate, void* stream) {
  int rc = check_common(B, N, E, n_cache, n_head, dtype);
  if (rc != NCN_OK) return rc;
  if (L < 1 || first_module < 0) return NCN_ERR_SHAPE;
  const bool tape = (flags & F_TAPE) != 0;  // the state after the last stage comes from ckpt; s0, s1 unused
  if (tape && (flags & F_RECOMPUTE)) return NCN_ERR_UNSUPPORTED;
  if ((!tape && (!s0 || !s1)) || (tape && !ckpt) || !dy || !dya || !W || !dx || !dxa || !dW) return NCN_ERR_NULL;
  if ((x_rec == nullptr) != (xa_rec == nullptr)) return NCN_ERR_NULL;
  if (!rows_shape_ok(N, E, n_cache, n_head, dtype) || map_act(activation) == ACT_LEAKY) return NCN_ERR_UNSUPPORTED;
  if ((flags & F_RESIDUAL) && !(flags & (F_RECOMPUTE | F_TAPE))) return NCN_ERR_UNSUPPORTED;
  if (!aligned16(s0) || !aligned16(s1) || !aligned16(dy) || !aligned16(dya) || !aligned16(dx) || !aligned16(dxa) ||
      (x_rec && (!aligned16(x_rec) || !aligned16(xa_rec))) || (ckpt && !aligned16(ckpt)))
    return NCN_ERR_ALIGN;
  DevInfo dev;
  if ((rc = get_dev(dev)) != NCN_OK) return rc;
  if (!partials || (full_workspace && capacity_floats < workspace_floats(dev, E, L))) return short_err;
  const int act = fused_act(map_act(activation), dtype);
  const bool use_ck = ckpt && !(flags & F_RECOMPUTE) && ckpt_slots(L, ckpt_every, flags) > 0;
  const int n_ck = use_ck ? ckpt_slots(L, ckpt_every, flags) : 0;
  {
    // register-resident family (with stored states: only where the forward is of this family too)
    LanePlan lp, lf;
    bool lanes = plan_lanes(true, B, N, E, n_cache, n_head, first_module, L, dtype, flags, n_ck, dev, act, lp) == NCN_OK;
    if (lanes && n_ck > 0)
      lanes = plan_lanes(false, B, N, E, n_cache, n_head, first_module, L, dtype, flags, 0, dev, act, lf) == NCN_OK;
    if (lanes) {
      if ((size_t)lp.grid * 2 * (size_t)L > capacity_floats) return short_err;
      LaneParams q{};
      q.in[0] = s0; q.in[1] = s1; q.in[2] = dy; q.in[3] = dya;
      q.out[0] = dx; q.out[1] = dxa; q.out[2] = x_rec; q.out[3] = xa_rec;
      q.ckpt = use_ck ? const_cast<float*>(ckpt) : nullptr;
      q.ckpt_every = ckpt_every;
      q.W = W;
      q.partials = partials;
      q.status = dev.status;
      q.B = B; q.N = (int)N; q.m = (int)(N / n_cache); q.L = L; q.l0 = first_module;
      q.flags = flags & (F_RESIDUAL | F_TAPE);
      q.alpha = (float)alpha;
      q.oma = (float)(1.0 - alpha);
      fill_lane(q, lp);
      cudaError_t e = lane_fn(n_cache, true)(act, dtype, q, lp.grid, lp.threads, lp.smem, (cudaStream_t)stream, nullptr);
      if (e != cudaSuccess) return cuda_fail(e);
      return reduce_dw(partials, dW, lp.grid, 2 * L, dw_accumulate, (cudaStream_t)stream);
    }
  }
  Plan pl;
  if ((rc = plan_rows(true, B, (int)N, n_cache, L, dtype, flags, n_ck, x_rec != nullptr, dev, act, pl)) != NCN_OK)
    return rc;
  // one row of 2L partial sums per CTA
  if ((size_t)pl.grid * 2 * (size_t)L > capacity_floats) return short_err;
  RowsParams p{};
  p.in[0] = s0; p.in[1] = s1; p.in[2] = dy; p.in[3] = dya;
  p.out[0] = dx; p.out[1] = dxa; p.out[2] = x_rec; p.out[3] = xa_rec;
  p.ckpt = use_ck ? const_cast<float*>(ckpt) : nullptr;
  p.ckpt_every = ckpt_every;
  p.W = W;
  p.partials = partials;  // every element the reduction reads is written by the kernel first
  p.status = dev.status;
  p.B = B; p.N = (int)N; p.m = (int)(N / n_cache); p.L = L; p.l0 = first_module;
  p.flags = (flags & (F_RESIDUAL | F_RECOMPUTE | F_TAPE)) | (pl.red_thread ? F_RED_THREAD : 0);
  p.alpha = (float)alpha;
  p.oma = (float)(1.0 - alpha);
  fill_offsets(p, pl);
  cudaError_t e = (pl.pair ? pair_fn(n_cache, true) : rows_fn(n_cache, true))(act, dtype, p, pl.grid, pl.threads, pl.smem,
                                                                             (cudaStream_t)stream, nullptr);
  if (e != cudaSuccess) return cuda_fail(e);
  return reduce_dw(p.partials, dW, pl.grid, 2 * L, dw_accumulate, (cudaStream_t)stream);
}

int ncn_net_bwd(const void* s0, const void* s1, const void* dy, const void* dya, const float* W, void* dx, void* dxa,
                void* x_rec, void* xa_rec, float* dW, const float* ckpt, int ckpt_every, void* workspace,
                size_t workspace_bytes, int64_t B, int64_t N, int64_t E, int n_cache, int n_head, int first_module,
                int L, double alpha, int activation, int dtype, int flags, int dw_accumulate, void* stream) {
  return net_bwd_impl(s0, s1, dy, dya, W, dx, dxa, x_rec, xa_rec, dW, ckpt, ckpt_every, static_cast<float*>(workspace),
                      workspace_bytes / sizeof(float), true, NCN_ERR_WORKSPACE, B, N, E, n_cache, n_head, first_module, L,
                      alpha, activation, dtype, flags, dw_accumulate, stream);
}

int ncn_stage_fwd(const void* x, const void* xa, const float* W, void* y, void* ya, int64_t B, int64_t N, int64_t E,
                  int n_cache, int n_head, int module_l, double alpha, int activation, int dtype, void* stream) {
  int rc = check_common(B, N, E, n_cache, n_head, dtype);
  if (rc != NCN_OK) return rc;
  if (module_l < 0) return NCN_ERR_SHAPE;
  if (!x || !xa || !W || !y || !ya) return NCN_ERR_NULL;
  if (rows_shape_ok(N, E, n_cache, n_head, dtype) && aligned16(x) && aligned16(xa) && aligned16(y) && aligned16(ya)) {
    rc = ncn_net_fwd(x, xa, W, y, ya, nullptr, 0, B, N, E, n_cache, n_head, module_l, 1, alpha, activation, dtype, 0,
                     stream);
    if (rc != NCN_ERR_SMEM && rc != NCN_ERR_UNSUPPORTED) return rc;
  }
  DevInfo dev;
  if ((rc = get_dev(dev)) != NCN_OK) return rc;
  {
    const void* fin[4] = {x, xa, nullptr, nullptr};
    void* fout[4] = {y, ya, nullptr, nullptr};
    rc = launch_feat(false, fin, fout, W, nullptr, B, N, E, n_cache, n_head, module_l, alpha, activation, dtype, dev,
                     (cudaStream_t)stream, nullptr);
    if (rc != NCN_ERR_UNSUPPORTED) return rc;
  }
  return stage_fwd_generic(x, xa, W, nullptr, y, ya, B, N, E, n_cache, n_head, module_l, alpha, activation, dtype, dev,
                           stream);
}

int ncn_stage_bwd(const void* y, const void* ya, const void* dy, const void* dya, const float* W, void* dx, void* dxa,
                  void* x_rec, void* xa_rec, float* dW, void* workspace, size_t workspace_bytes, int64_t B, int64_t N,
                  int64_t E, int n_cache, int n_head, int module_l, double alpha, int activation, int dtype,
                  void* stream) {
  int rc = check_common(B, N, E, n_cache, n_head, dtype);
  if (rc != NCN_OK) return rc;
  if (module_l < 0) return NCN_ERR_SHAPE;
  if (!y || !ya || !dy || !dya || !W || !dx || !dxa || !dW) return NCN_ERR_NULL;
  if ((x_rec == nullptr) != (xa_rec == nullptr)) return NCN_ERR_NULL;
  DevInfo dev;
  if ((rc = get_dev(dev)) != NCN_OK) return rc;
  if (!workspace || workspace_bytes < workspace_floats(dev, E, 1) * sizeof(float)) return NCN_ERR_WORKSPACE;
  if (rows_shape_ok(N, E, n_cache, n_head, dtype) && aligned16(y) && aligned16(ya) && aligned16(dy) && aligned16(dya) &&
      aligned16(dx) && aligned16(dxa) && (!x_rec || (aligned16(x_rec) && aligned16(xa_rec)))) {
    rc = ncn_net_bwd(y, ya, dy, dya, W, dx, dxa, x_rec, xa_rec, dW, nullptr, 0, workspace, workspace_bytes, B, N, E,
                     n_cache, n_head, module_l, 1, alpha, activation, dtype, 0, 0, stream);
    if (rc != NCN_ERR_SMEM && rc != NCN_ERR_UNSUPPORTED) return rc;
  }
  {
    const void* fin[4] = {y, ya, dy, dya};
    void* fout[4] = {dx, dxa, x_rec, xa_rec};
    int fgrid = 0;
    rc = launch_feat(true, fin, fout, W, static_cast<float*>(workspace), B, N, E, n_cache, n_head, module_l, alpha,
                     activation, dtype, dev, (cudaStream_t)stream, &fgrid);
    if (rc == NCN_OK) return reduce_dw(static_cast<float*>(workspace), dW, fgrid, 2 * (int)E, 0, (cudaStream_t)stream);
    if (rc != NCN_ERR_UNSUPPORTED) return rc;
  }
  return stage_bwd_generic(y, ya, dy, dya, W, nullptr, dx, dxa, x_rec, xa_rec, dW, static_cast<float*>(workspace), B, N, E,
                           n_cache, n_head, module_l, alpha, activation, dtype, dev, stream);
}

int ncn_stage_bwd_saved(const void* x, const void* xa, const void* y, const void* ya, const void* dy, const void* dya,
                        const float* W, void* dx, void* dxa, float* dW, void* workspace, size_t workspace_bytes, int64_t B,
                        int64_t N, int64_t E, int n_cache, int n_head, int module_l, double alpha, int activation,
                        int dtype, void* stream) {
  int rc = check_common(B, N, E, n_cache, n_head, dtype);
  if (rc != NCN_OK) return rc;
  if (module_l < 0) return NCN_ERR_SHAPE;
  if (!x || !xa || !dy || !dya || !W || !dx || !dxa || !dW) return NCN_ERR_NULL;
  // fp32: the last segment is walked back from the output; bf16: everything is replayed from the input
  const int replay_all = dtype == DT_BF16 ? 1 : 0;
  if (!replay_all && (!y || !ya)) return NCN_ERR_NULL;
  if (!replay_all && n_cache <= kSegment)  // the chain from the output is short enough: the input is not needed
    return ncn_stage_bwd(y, ya, dy, dya, W, dx, dxa, nullptr, nullptr, dW, workspace, workspace_bytes, B, N, E, n_cache,
                         n_head, module_l, alpha, activation, dtype, stream);
  DevInfo dev;
  if ((rc = get_dev(dev)) != NCN_OK) return rc;
  if (!workspace || workspace_bytes < workspace_floats(dev, E, 1) * sizeof(float)) return NCN_ERR_WORKSPACE;
  {
    const void* fin[4] = {replay_all ? nullptr : y, replay_all ? nullptr : ya, dy, dya};
    void* fout[4] = {dx, dxa, nullptr, nullptr};
    int fgrid = 0;
    rc = launch_feat(true, fin, fout, W, static_cast<float*>(workspace), B, N, E, n_cache, n_head, module_l, alpha,
                     activation, dtype, dev, (cudaStream_t)stream, &fgrid, x, xa, replay_all ? 2 : 1);
    if (rc == NCN_OK) return reduce_dw(static_cast<float*>(workspace), dW, fgrid, 2 * (int)E, 0, (cudaStream_t)stream);
    if (rc != NCN_ERR_UNSUPPORTED) return rc;
  }
  return stage_bwd_generic(y, ya, dy, dya, W, nullptr, dx, dxa, nullptr, nullptr, dW, static_cast<float*>(workspace), B, N,
                           E, n_cache, n_head, module_l, alpha, activation, dtype, dev, stream, x, xa, replay_all);
}

// states the per-stage forward stores for ncn_stage_bwd_mid: one after every 16th step short of the last, and with
// bf16 storage the end state too
static int stage_mid_states(int n_cache, int dtype) { return (n_cache - 1) / kSegment + (dtype == DT_BF16 ? 1 : 0); }

size_t ncn_stage_mid_bytes(int64_t B, int64_t N, int64_t E, int n_cache, int dtype) {
  if (B <= 0 || N <= 0 || E <= 0 || n_cache <= 0) return 0;
  return (size_t)stage_mid_states(n_cache, dtype) * 2 * (size_t)B * (size_t)N * (size_t)E * sizeof(float);
}

int ncn_stage_fwd_mid(const void* x, const void* xa, const float* W, void* y, void* ya, void* mid, size_t mid_bytes,
                      int64_t B, int64_t N, int64_t E, int n_cache, int n_head, int module_l, double alpha, int activation,
                      int dtype, void* stream) {
  int rc = check_common(B, N, E, n_cache, n_head, dtype);
  if (rc != NCN_OK) return rc;
  if (module_l < 0) return NCN_ERR_SHAPE;
  if (!x || !xa || !W || !y || !ya) return NCN_ERR_NULL;
  const size_t need = ncn_stage_mid_bytes(B, N, E, n_cache, dtype);
  if (need == 0)  // nothing to store: chains of at most 16 steps from fp32 outputs
    return ncn_stage_fwd(x, xa, W, y, ya, B, N, E, n_cache, n_head, module_l, alpha, activation, dtype, stream);
  if (!mid) return NCN_ERR_NULL;
  if (mid_bytes < need) return NCN_ERR_WORKSPACE;
  const int mid_end = dtype == DT_BF16 ? 1 : 0;
  DevInfo dev;
  if ((rc = get_dev(dev)) != NCN_OK) return rc;
  {
    const void* fin[4] = {x, xa, nullptr, nullptr};
    void* fout[4] = {y, ya, nullptr, nullptr};
    rc = launch_feat(false, fin, fout, W, nullptr, B, N, E, n_cache, n_head, module_l, alpha, activation, dtype, dev,
                     (cudaStream_t)stream, nullptr, nullptr, nullptr, 0, static_cast<float*>(mid), mid_end);
    if (rc != NCN_ERR_UNSUPPORTED) return rc;
  }
  return stage_fwd_generic(x, xa, W, nullptr, y, ya, B, N, E, n_cache, n_head, module_l, alpha, activation, dtype, dev,
                           stream, static_cast<float*>(mid), mid_end);
}

int ncn_stage_bwd_mid(const void* y, const void* ya, const void* mid, size_t mid_bytes, const void* dy, const void* dya,
                      const float* W, void* dx, void* dxa, float* dW, void* workspace, size_t workspace_bytes, int64_t B,
                      int64_t N, int64_t E, int n_cache, int n_head, int module_l, double alpha, int activation,
                      int dtype, void* stream) {
  int rc = check_common(B, N, E, n_cache, n_head, dtype);
  if (rc != NCN_OK) return rc;
  if (module_l < 0) return NCN_ERR_SHAPE;
  if (!dy || !dya || !W || !dx || !dxa || !dW) return NCN_ERR_NULL;
  const size_t need = ncn_stage_mid_bytes(B, N, E, n_cache, dtype);
  if (need == 0)
    return ncn_stage_bwd(y, ya, dy, dya, W, dx, dxa, nullptr, nullptr, dW, workspace, workspace_bytes, B, N, E, n_cache,
                         n_head, module_l, alpha, activation, dtype, stream);
  if (!mid) return NCN_ERR_NULL;
  if (mid_bytes < need) return NCN_ERR_WORKSPACE;
  const int mid_end = dtype == DT_BF16 ? 1 : 0;
  if (!mid_end && (!y || !ya)) return NCN_ERR_NULL;
  DevInfo dev;
  if ((rc = get_dev(dev)) != NCN_OK) return rc;
  if (!workspace || workspace_bytes < workspace_floats(dev, E, 1) * sizeof(float)) return NCN_ERR_WORKSPACE;
  {
    const void* fin[4] = {mid_end ? nullptr : y, mid_end ? nullptr : ya, dy, dya};
    void* fout[4] = {dx, dxa, nullptr, nullptr};
    int fgrid = 0;
    rc = launch_feat(true, fin, fout, W, static_cast<float*>(workspace), B, N, E, n_cache, n_head, module_l, alpha,
                     activation, dtype, dev, (cudaStream_t)stream, &fgrid, nullptr, nullptr, 3,
                     const_cast<float*>(static_cast<const float*>(mid)), mid_end);
    if (rc == NCN_OK) return reduce_dw(static_cast<float*>(workspace), dW, fgrid, 2 * (int)E, 0, (cudaStream_t)stream);
    if (rc != NCN_ERR_UNSUPPORTED) return rc;
  }
  return stage_bwd_generic(y, ya, dy, dya, W, nullptr, dx, dxa, nullptr, nullptr, dW, static_cast<float*>(workspace), B, N,
                           E, n_cache, n_head, module_l, alpha, activation, dtype, dev, stream, nullptr, nullptr, 0,
                           static_cast<const float*>(mid), mid_end);
}

int ncn_stage_fwd_ctx(const void* x, const void* xa, const float* W, const int* ctxlen, void* y, void* ya, int64_t B,
                      int64_t N, int64_t E, int n_cache, int n_head, int module_l, double alpha, int activation, int dtype,
                      void* stream) {
  int rc = check_common(B, N, E, n_cache, n_head, dtype);
  if (rc != NCN_OK) return rc;
  if (module_l < 0) return NCN_ERR_SHAPE;
  if (!x || !xa || !W || !ctxlen || !y || !ya) return NCN_ERR_NULL;
  DevInfo dev;
  if ((rc = get_dev(dev)) != NCN_OK) return rc;
  return stage_fwd_generic(x, xa, W, ctxlen, y, ya, B, N, E, n_cache, n_head, module_l, alpha, activation, dtype, dev,
                           stream);
}

int ncn_stage_bwd_ctx(const void* y, const void* ya, const void* dy, const void* dya, const float* W, const int* ctxlen,
                      void* dx, void* dxa, void* x_rec, void* xa_rec, float* dW, void* workspace, size_t workspace_bytes,
                      int64_t B, int64_t N, int64_t E, int n_cache, int n_head, int module_l, double alpha, int activation,
                      int dtype, void* stream) {
  int rc = check_common(B, N, E, n_cache, n_head, dtype);
  if (rc != NCN_OK) return rc;
  if (module_l < 0) return NCN_ERR_SHAPE;
  if (!y || !ya || !dy || !dya || !W || !ctxlen || !dx || !dxa || !dW) return NCN_ERR_NULL;
  if ((x_rec == nullptr) != (xa_rec == nullptr)) return NCN_ERR_NULL;
  DevInfo dev;
  if ((rc = get_dev(dev)) != NCN_OK) return rc;
  if (!workspace || workspace_bytes < workspace_floats(dev, E, 1) * sizeof(float)) return NCN_ERR_WORKSPACE;
  return stage_bwd_generic(y, ya, dy, dya, W, ctxlen, dx, dxa, x_rec, xa_rec, dW, static_cast<float*>(workspace), B, N, E,
                           n_cache, n_head, module_l, alpha, activation, dtype, dev, stream);
}

}  // extern "C"

// ------------------------------------------------------------------------------------------
// Backward entry point that allocates nothing (declared in include/ncn_b200.h).
//
// The backward kernel needs scratch memory for its per-CTA weight-gradient partials.  The
// other entry points take that scratch from the caller; this one keeps it in the library
// image, for callers that have no way to obtain device memory where they call from.
namespace ncn {

constexpr size_t kNoAllocFloats = 16384;  // 64 KiB per device that loads the library

// File-scope device array.  In host code this NAME is only a handle for the runtime's symbol
// table, not a device address: the address is looked up with cudaGetSymbolAddress below.
static __device__ __align__(256) float g_noalloc_scratch[kNoAllocFloats];

// Device address of the array on the current device, looked up once per device.
static int noalloc_scratch(float** out) {
  static float* table[64];
  static std::atomic<int> ready[64];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e);
  if (dev < 0 || dev >= 64) return NCN_ERR_CUDA;
  if (!ready[dev].load(std::memory_order_acquire)) {
    float* ptr = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_scratch);
    if (e != cudaSuccess) return cuda_fail(e);
    if (ptr == nullptr) return NCN_ERR_CUDA;
    table[dev] = ptr;
    ready[dev].store(1, std::memory_order_release);
  }
  *out = table[dev];
  return NCN_OK;
}

}  // namespace ncn

extern "C" int ncn_net_bwd_noalloc(const void* s0, const void* s1, const void* dy, const void* dya, const float* W,
                                   void* dx, void* dxa, void* x_rec, void* xa_rec, float* dW, const float* ckpt,
                                   int ckpt_every, int64_t B, int64_t N, int64_t E, int n_cache, int n_head,
                                   int first_module, int L, double alpha, int activation, int dtype, int flags,
                                   int dw_accumulate, void* stream) {
  float* scratch = nullptr;
  const int rc = noalloc_scratch(&scratch);
  if (rc != NCN_OK) return rc;
  // one row of 2L partial sums per CTA must fit the fixed array
  return net_bwd_impl(s0, s1, dy, dya, W, dx, dxa, x_rec, xa_rec, dW, ckpt, ckpt_every, scratch, kNoAllocFloats,
                      false, NCN_ERR_TOO_LARGE, B, N, E, n_cache, n_head, first_module, L, alpha, activation, dtype, flags,
                      dw_accumulate, stream);
}
