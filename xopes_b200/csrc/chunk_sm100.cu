// Chunk-parallel scalar-decay pass on 5th-generation tensor cores (sm_100a).
//
// One CTA per (sequence, head) walks the sequence in 128-token chunks.  Per chunk it computes
//
//   P  = X Y^T                        tcgen05.mma, A and B from shared memory (K-major)
//   P~ = P (.) decay mask             registers, written back to tensor memory as 16-bit
//   W1 = P~ Z                         tcgen05.mma, A from tensor memory, B MN-major
//   W2 = X T_in                       tcgen05.mma, B = 16-bit copy of the running state
//   T  = e^g T_in + (Y (.) u)^T Z     tcgen05.mma accumulating into the resident fp32 state
//   W  = W1 + diag(s) W2              epilogue, stored with TMA
//
// The 128x128 fp32 state T never leaves tensor memory between chunks, so HBM sees each operand
// tile once per pass and the output once.  A producer warp keeps the next chunk's three tiles in
// flight with plain (non-multicast) TMA loads while the eight compute warps work on the current
// one.  X and Y of a stage go back to the producer as soon as the products that read them are
// done (mid-chunk); Z doubles as the staging buffer of the output tile, which a store warp writes
// out with TMA, and goes back after that.  Shared memory: 2 stages x 3 tiles x 32 KB + 32 KB
// state copy + 3 KB of barriers and per-row decay values = 227 KB; tensor memory:
// T | P | W1 | W2 = 4 x 128 columns.
//
// Every mbarrier wait is bounded (sm100_ptx.cuh: mbar_wait); a wait that runs out sets the device
// status word and the kernel finishes by itself.
#include <cuda.h>

#include <cstddef>
#include <cstdlib>
#include <mutex>

#include "chunk.cuh"
#include "sm100_ptx.cuh"
#include "tile_common.cuh"

namespace la {
namespace {

using namespace ptx;
using namespace tile;

constexpr int kChunk = 128;
constexpr int kTileBytes = 32768;  // [128][128] 16-bit = two TMA boxes of [128][64]
constexpr int kBoxBytes = 16384;
constexpr int kStages = 2;
constexpr int kStageBytes = 3 * kTileBytes;
constexpr int kOffTb = kStages * kStageBytes;
constexpr int kOffSmall = kOffTb + kTileBytes;
constexpr int kSmallBytes = 3072;
// All of the 227 KB a CTA may have.  There is no slack to round the base up: the kernel declares its
// dynamic shared memory 1024-byte aligned (the 128-byte swizzle needs that) and checks it.
constexpr int kSmemBytes = kOffSmall + kSmallBytes;
constexpr int kStAlign = 113;
constexpr int kComputeThreads = 256;                        // two warpgroups, each owns 64 columns
constexpr int kProducerWarp = 8;                            // TMA loads
constexpr int kMmaWarp = 9;                                 // tcgen05.mma issue
constexpr int kStoreWarp = 10;                              // TMA stores of finished output tiles
constexpr int kThreads = kComputeThreads + 3 * 32;
constexpr float kLog2e = 1.4426950408889634f;

// tensor-memory columns
constexpr uint32_t kColT = 0, kColP = 128, kColW1 = 256, kColW2 = 384;

// status codes written to the device status word
constexpr int kStFull = 101, kStEmpty = 102, kStP = 103, kStW = 104, kStD = 105, kStF = 106, kStH = 107,
              kStT = 108, kStY = 109, kStX = 110, kStL = 111, kStU = 113;

struct Small {
  // X and Y of a stage are released as soon as the products that read them are done (mid-chunk);
  // Z doubles as the staging buffer of the output tile and is released when that has been stored
  unsigned long long full[kStages];    // X and Y landed
  unsigned long long empty[kStages];   // X and Y free
  unsigned long long fullz[kStages];   // Z landed
  unsigned long long emptyz[kStages];  // Z free
  unsigned long long bar_p;   // P = X Y^T complete                       (MMA warp -> compute)
  unsigned long long bar_w;   // W1, W2 and the state update complete      (MMA warp -> compute)
  unsigned long long bar_t;   // state update complete (T final for the chunk) (MMA warp -> compute)
  unsigned long long bar_d;   // state copy written, T rescaled            (compute -> MMA warp)
  unsigned long long bar_y;   // rescaled Y written                        (compute -> MMA warp)
  unsigned long long bar_f;   // masked P~ written                         (compute -> MMA warp)
  unsigned long long bar_h;   // output tile staged, W1/W2 consumed        (compute -> store and MMA warps)
  unsigned long long bar_x;   // X T_in with the high half of the state copy complete (MMA warp -> compute)
  unsigned long long bar_l;   // low half of the state copy written, T rescaled (compute -> MMA warp)
  unsigned long long bar_u;   // X T_in with the low half complete: the copy tile is free (MMA warp -> compute)
  uint32_t tmem_base;
  int abort_flag;
  int issued;    // chunks whose X and Y loads were issued
  int issuedz;   // chunks whose Z load was issued
  int rg[4];                  // this CTA's range of the chunk space (Range), written once at start
  alignas(16) float wsum[2][4];     // per-quadrant decay sums, by chunk parity like cs/bs
  // double-buffered by chunk parity: the next chunk's values are computed while the tensor cores
  // still work on X Y^T of the current one
  alignas(16) float cs[2][kChunk];  // inclusive cumulative log2 decay of each row of the chunk
  alignas(16) float bs[2][kChunk];  // per-column factor of the factorised decay mask (read as float4)
  alignas(16) float rd[kChunk];   // row-dot partial of the second warpgroup
};
static_assert(sizeof(Small) <= kSmallBytes, "small area overflow");
static_assert(offsetof(Small, cs) % 16 == 0 && offsetof(Small, bs) % 16 == 0, "vector loads need 16 B");
static_assert(kOffSmall % 16 == 0, "small area must start 16-byte aligned");

struct ChunkArgs {
  const void *xrow;
  float *rowdot;
  void *out;
  const float *ld;
  long long ld_sb, ld_sn, ld_sh;
  const float *t0;
  float *tfinal;
  int state_transposed, reverse;
  const long long *cu;
  int B, N, H, M;
  int ld_act;  // 1: ld holds pre-activations x and the log decay is logsigmoid(x)
  int fx, fz;  // features of X and Y (the contraction of X Y^T) and of Z, the output and xrow; <= 128
  int *status;
};

// How the (sequence, head) pairs of a launch are spread over its CTAs.
//
// balanced = 0: CTA r owns pair r whole.
// balanced = 1: every pair is a run of chunks + kTaskUnits units in processing order (the extra
//   units stand for the cost of switching to the pair and are left out when all pairs have the
//   same length); the pairs' runs are laid end to end
//   (pair = sequence * H + head) and CTA r of R owns units [total r / R, total (r+1) / R), a
//   boundary inside a pair's switch units moving to the pair's start.  A pair cut by a boundary is worked on by two neighbouring
//   CTAs: the one that owns its first part publishes the running state to its hand-off slot, the
//   one that owns the rest picks it up there.  A CTA works on the part it publishes first and on
//   the part it has to wait for last, so with pairs shorter than a CTA's share nobody waits.
// npass = 2: two passes over the same tokens share the launch (even CTAs run pass 0, odd CTAs
//   pass 1, both on range blockIdx.x / 2), so that the operand tiles they have in common are
//   fetched from HBM once and found in L2 by the other.
struct Sched {
  int balanced, npass;
  long long total;           // sum of the units of all pairs (fixed-length launches; else H * wprefix[M])
  const long long *wprefix;  // cu_seqlens launches: exclusive prefix sum of units over sequences (M + 1)
  float *handoff;            // [gridDim.x][128 * 128] fp32, element (i, c) of T at c * 128 + i
  int *flags;                // [gridDim.x], zero before the launch; 1 = slot written
};

struct Launch {
  ChunkArgs a[2];
  Sched sc;
};
struct PassMaps {
  CUtensorMap x, y, z, o;
};
struct Maps {
  PassMaps p[2];
};

constexpr int kStHandoff = 112;

// first and last pair of a CTA's range, chunk offset inside the first, end offset inside the last
struct Range {
  int p_a, p_b, off_a, end_b;
};
struct Task {
  int seq, h, bidx;
  long long t_begin;
  int len, nc;   // tokens and chunks of the whole sequence
  int it0, cnt;  // this task covers processing steps [it0, it0 + cnt) of the sequence
  bool waits, publishes;
};

// A task switch (drain, new starting state, pipeline refill) costs about as much as two chunks, so
// a pair weighs its chunks plus kTaskUnits: a CTA that is handed many short pairs gets fewer chunks.
constexpr int kTaskUnits = 2;

// Position x of the weighted unit space -> (pair, processing step).  The first kTaskUnits units of a
// pair stand for its switch and map to step 0, so a boundary that falls there moves to the pair's
// start.  x = total maps to (number of pairs, 0).
__device__ __forceinline__ void locate(const ChunkArgs &a, const Sched &sc, long long x, long long total, int &p,
                                       int &step) {
  if (x >= total) {
    p = (a.cu != nullptr ? a.M : a.B) * a.H;
    step = 0;
    return;
  }
  if (a.cu == nullptr) {  // equal pairs: nothing to weigh, the split is even in chunks
    const int w = (a.N + kChunk - 1) / kChunk;
    p = (int)(x / w);
    step = (int)(x - (long long)p * w);
    return;
  }
  int lo = 0, hi = a.M - 1;  // largest seq with H * wprefix[seq] <= x
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if ((long long)a.H * sc.wprefix[mid] <= x) lo = mid; else hi = mid - 1;
  }
  const long long rem = x - (long long)a.H * sc.wprefix[lo];
  const long long w = sc.wprefix[lo + 1] - sc.wprefix[lo];
  const int h = (int)(rem / w);
  p = lo * a.H + h;
  step = max(0, (int)(rem - (long long)h * w) - kTaskUnits);
}

// CTA r owns the positions [start(r), start(r + 1)) in (pair, step) order, start(r) = the position
// of unit total r / R.
__device__ __forceinline__ Range cta_range(const ChunkArgs &a, const Sched &sc, int r, int R) {
  Range g;
  if (!sc.balanced) {
    g.p_a = g.p_b = r;
    g.off_a = 0;
    g.end_b = 0x7fffffff;
    return g;
  }
  const long long total = a.cu != nullptr ? (long long)a.H * sc.wprefix[a.M] : sc.total;
  int p_e, step_e;
  locate(a, sc, total * r / R, total, g.p_a, g.off_a);
  locate(a, sc, total * (r + 1) / R, total, p_e, step_e);
  if (step_e == 0) {  // ends with a whole pair
    g.p_b = p_e - 1;
    g.end_b = 0x7fffffff;
  } else {
    g.p_b = p_e;
    g.end_b = step_e;
  }
  return g;
}

__device__ __forceinline__ Task task_of(const ChunkArgs &a, const Range &g, int k, int ntasks) {
  Task t;
  const int p = (ntasks == 1) ? g.p_a : (k == 0 ? g.p_b : (k == ntasks - 1 ? g.p_a : g.p_a + k));
  t.seq = p / a.H;
  t.h = p - t.seq * a.H;
  if (a.cu != nullptr) {
    t.t_begin = a.cu[t.seq];
    t.len = (int)(a.cu[t.seq + 1] - t.t_begin);
    t.bidx = 0;
  } else {
    t.t_begin = 0;
    t.len = a.N;
    t.bidx = t.seq;
  }
  t.nc = (t.len + kChunk - 1) / kChunk;
  const int w = max(t.nc, 1);
  t.it0 = (p == g.p_a) ? g.off_a : 0;
  const int it1 = (p == g.p_b) ? min(g.end_b, w) : w;
  t.waits = t.it0 > 0;
  t.publishes = it1 < w;
  t.cnt = min(it1, t.nc) - t.it0;
  return t;
}

__device__ __forceinline__ int ld_acquire(const int *p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release(int *p, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// byte offset of the k-th 16-element slice of a K-major [128][128] tile (two boxes of 64 columns)
__device__ __forceinline__ uint32_t kslice(int ks) { return (uint32_t)(ks >> 2) * kBoxBytes + (uint32_t)(ks & 3) * 32u; }

// Thread layout of the compute warps: warpgroup wg = warp / 4 owns columns [64 wg, 64 wg + 64) of
// every 128-column row, quadrant q4 = warp % 4 owns rows (= tensor-memory lanes) [32 q4, 32 q4 + 32).
//
// Decay mask.  With c = in-chunk inclusive cumulative log2 decay, the weight of (row i, column j)
// is 2^(c_i - c_j) for j <= i (forward) or 2^(c_j - c_i) for j >= i (reverse).  For a 32-column
// batch that lies wholly on the allowed side of the diagonal the weight factorises as
// A_i(batch) * B_j with both exponents <= 0 (reference point: the batch edge nearest the diagonal),
// so only the diagonal batch pays one exponential per element.
//
// Every role walks the CTA's tasks in the same order and numbers the chunks it has handled with
// one running counter; pipeline stages and mbarrier parities follow that counter, so the
// pipeline never drains between tasks.
//
// F128 = true: every tensor has 128 features per head.  F128 = false: head dimensions below 128
// (multiples of 8).  The tiles stay 128 wide: the tensor maps then describe fewer features than a
// box holds, TMA fills the rest of the box with zeros on load and clips it on store, and the zero
// features add nothing to any product; only the accesses that bypass TMA (states, ragged last
// chunks, the row-dot operand) look at the real widths.
// ACT = true: ld holds pre-activations of a logsigmoid (an instantiation of its own: the extra
// arithmetic sits on the decay scan at the top of every chunk, which the plain path should not carry).
template <typename T, bool F128, bool ACT>
__global__ void __launch_bounds__(kThreads, 1)
chunk_pass_kernel(const __grid_constant__ Maps maps, const __grid_constant__ Launch lp) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  uint8_t *gbase = smem_raw;
  Small *sm = reinterpret_cast<Small *>(gbase + kOffSmall);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (base & 1023u) {  // uniform over the CTA; nothing has been set up yet
    if (tid == 0) atomicCAS(lp.a[0].status, 0, kStAlign);
    return;
  }
  // Arguments both passes of a merged launch share (sizes, strides, decay, direction) are read
  // from slot 0 as direct constant-bank operands; only the few that differ (`ap`: row-dot
  // operand, output, states) are indexed by the pass, and none of those is touched per chunk
  // unless a log-decay gradient was asked for.
  const Sched &sc = lp.sc;
  const int sh = sc.npass == 2 ? 1 : 0;
  const int pass = (int)(blockIdx.x & (unsigned)sh);
  const int r_cta = (int)(blockIdx.x >> sh), r_cnt = (int)(gridDim.x >> sh);
  const ChunkArgs &a = lp.a[0];
  const ChunkArgs &ap = lp.a[pass];
  const CUtensorMap *map_x = &maps.p[pass].x, *map_y = &maps.p[pass].y, *map_z = &maps.p[pass].z,
                    *map_o = &maps.p[pass].o;
  // The range lives in shared memory and every role re-reads it per task: it must not occupy
  // registers across the chunk loop of the compute warps.
  volatile int *rg_s = sm->rg;
  auto range = [&]() -> Range { return Range{rg_s[0], rg_s[1], rg_s[2], rg_s[3]}; };
  const bool rev = a.reverse != 0;

  const uint32_t bar_full = smem_u32(&sm->full[0]), bar_empty = smem_u32(&sm->empty[0]);
  const uint32_t bar_fullz = smem_u32(&sm->fullz[0]), bar_emptyz = smem_u32(&sm->emptyz[0]);
  const uint32_t bar_p = smem_u32(&sm->bar_p), bar_w = smem_u32(&sm->bar_w);
  const uint32_t bar_d = smem_u32(&sm->bar_d), bar_f = smem_u32(&sm->bar_f), bar_h = smem_u32(&sm->bar_h);
  const uint32_t bar_t = smem_u32(&sm->bar_t), bar_y = smem_u32(&sm->bar_y);
  const uint32_t bar_x = smem_u32(&sm->bar_x), bar_l = smem_u32(&sm->bar_l), bar_u = smem_u32(&sm->bar_u);
  // With a log-decay gradient requested the 16-bit state copy is split into a high and a low
  // half (two passes of X T_in over the same buffer): the gradient is a long cumulative sum of
  // nearly cancelling terms and the rounding of a single 16-bit copy dominates its error.  For the
  // same reason the rescaled operand Y (.) u of the state update is then fed to the tensor cores as
  // a high and a low 16-bit half (the low half borrows the copy tile once X T_in is done with it):
  // the states the dq pass and the dk pass build must agree to well below 16-bit rounding for the
  // inter-chunk terms of q.dq and k.dk to cancel.
  const bool split = ap.rowdot != nullptr;
  volatile int *abort_flag = &sm->abort_flag;

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
      mbar_init(bar_fullz + 8 * s, 1);
      mbar_init(bar_emptyz + 8 * s, 1);
    }
    mbar_init(bar_p, 1);
    mbar_init(bar_w, 1);
    mbar_init(bar_t, 1);
    mbar_init(bar_x, 1);
    mbar_init(bar_u, 1);
    mbar_init(bar_l, kComputeThreads);
    mbar_init(bar_d, kComputeThreads);
    mbar_init(bar_y, kComputeThreads);
    mbar_init(bar_f, kComputeThreads);
    mbar_init(bar_h, kComputeThreads);
    sm->abort_flag = 0;
    sm->issued = 0;
    sm->issuedz = 0;
    const Range g = cta_range(a, sc, r_cta, r_cnt);
    sm->rg[0] = g.p_a; sm->rg[1] = g.p_b; sm->rg[2] = g.off_a; sm->rg[3] = g.end_b;
    fence_barrier_init();
  }
  if (warp == kProducerWarp) {
    tmem_alloc(smem_u32(&sm->tmem_base), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm->tmem_base;
  const int ntasks = rg_s[1] - rg_s[0] + 1;

  if (warp == kProducerWarp) {
    // ------------------------------------------------------------------ TMA loads
    if (lane == 0) {
      prefetch_tmap(map_x);
      prefetch_tmap(map_y);
      prefetch_tmap(map_z);
      int g0 = 0, nxy = 0, nz = 0;
      for (int k = 0; k < ntasks && !*abort_flag; ++k) {
        const Task tk = task_of(a, range(), k, ntasks);
        int it = 0;
        for (; it < tk.cnt; ++it) {
          const int gi = g0 + it;
          const int n = rev ? (tk.nc - 1 - (tk.it0 + it)) : (tk.it0 + it);
          const int s = gi & 1;
          const uint32_t ph = (uint32_t)(gi >> 1) & 1u;
          const uint32_t dst = base + (uint32_t)s * kStageBytes;
          const int tok0 = (int)tk.t_begin + n * kChunk;
          mbar_wait(bar_empty + 8 * s, ph ^ 1u, abort_flag, a.status, kStEmpty);
          if (*abort_flag) break;
          const uint32_t fb = bar_full + 8 * s;
          mbar_arrive_expect_tx(fb, 2 * kTileBytes);
          tma_load_4d(dst, map_x, fb, 0, tk.h, tok0, tk.bidx);
          tma_load_4d(dst + kBoxBytes, map_x, fb, 64, tk.h, tok0, tk.bidx);
          tma_load_4d(dst + kTileBytes, map_y, fb, 0, tk.h, tok0, tk.bidx);
          tma_load_4d(dst + kTileBytes + kBoxBytes, map_y, fb, 64, tk.h, tok0, tk.bidx);
          nxy = gi + 1;
          mbar_wait(bar_emptyz + 8 * s, ph ^ 1u, abort_flag, a.status, kStEmpty);
          if (*abort_flag) break;
          const uint32_t fz = bar_fullz + 8 * s;
          mbar_arrive_expect_tx(fz, kTileBytes);
          tma_load_4d(dst + 2 * kTileBytes, map_z, fz, 0, tk.h, tok0, tk.bidx);
          tma_load_4d(dst + 2 * kTileBytes + kBoxBytes, map_z, fz, 64, tk.h, tok0, tk.bidx);
          nz = gi + 1;
        }
        g0 += it;
      }
      sm->issued = nxy;
      sm->issuedz = nz;
    }
    __syncwarp();
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------------ tensor-core issue
    if (lane == 0) {
      const uint32_t idesc_kk = instr_desc(Fmt<T>::kAB, 0, 0, 128, 128);
      const uint32_t idesc_kmn = instr_desc(Fmt<T>::kAB, 0, 1, 128, 128);
      const uint32_t idesc_mnmn = instr_desc(Fmt<T>::kAB, 1, 1, 128, 128);
      const uint64_t d_tb = desc_mnmajor(base + kOffTb, kBoxBytes);
      int g0 = 0;
      for (int k = 0; k < ntasks; ++k) {
        const Task tk = task_of(a, range(), k, ntasks);
        for (int it = 0; it < tk.cnt; ++it) {
          const int gi = g0 + it;
          const int s = gi & 1;
          const uint32_t ph = (uint32_t)(gi >> 1) & 1u, par = (uint32_t)gi & 1u;
          const uint32_t xs = base + (uint32_t)s * kStageBytes, ys = xs + kTileBytes, zs = ys + kTileBytes;
          const uint64_t d_xk = desc_kmajor(xs), d_yk = desc_kmajor(ys);
          const uint64_t d_ymn = desc_mnmajor(ys, kBoxBytes), d_zmn = desc_mnmajor(zs, kBoxBytes);
          // descriptor advance per 16-element K slice, in 16-byte units: K-major tiles step 32 B
          // inside a 128 B row and jump to the second box after 4 slices; MN-major tiles step 16 rows
          mbar_wait(bar_full + 8 * s, ph, abort_flag, a.status, kStFull);
          tc_fence_after();
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            const uint64_t ko = (uint64_t)((ks >> 2) * (kBoxBytes >> 4) + (ks & 3) * 2);
            mma_ss(tmem + kColP, d_xk + ko, d_yk + ko, idesc_kk, ks > 0);
          }
          mma_commit(bar_p);
          // W2 = X T_in: needs the state copy of this chunk and the previous epilogue's reads of W2
          mbar_wait(bar_d, par, abort_flag, a.status, kStD);
          if (gi > 0) mbar_wait(bar_h, par ^ 1u, abort_flag, a.status, kStH);
          tc_fence_after();
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            const uint64_t ko = (uint64_t)((ks >> 2) * (kBoxBytes >> 4) + (ks & 3) * 2);
            mma_ss(tmem + kColW2, d_xk + ko, d_tb + (uint64_t)(ks * 128), idesc_kmn, ks > 0);
          }
          if (split) {
            mma_commit(bar_x);  // the compute warps may now overwrite the copy with its low half
            mbar_wait(bar_l, par, abort_flag, a.status, kStL);
            tc_fence_after();
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
              const uint64_t ko = (uint64_t)((ks >> 2) * (kBoxBytes >> 4) + (ks & 3) * 2);
              mma_ss(tmem + kColW2, d_xk + ko, d_tb + (uint64_t)(ks * 128), idesc_kmn, 1);
            }
            mma_commit(bar_u);  // the copy tile may now take the low half of Y (.) u
          }
          // T += (Y (.) u)^T Z as soon as the rescaled Y is there; its completion frees T for the
          // next chunk's state copy while P~ Z still runs
          mbar_wait(bar_y, par, abort_flag, a.status, kStY);
          mbar_wait(bar_fullz + 8 * s, ph, abort_flag, a.status, kStFull);
          tc_fence_after();
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)
            mma_ss(tmem + kColT, d_ymn + (uint64_t)(ks * 128), d_zmn + (uint64_t)(ks * 128), idesc_mnmn, 1);
          if (split) {  // low half of Y (.) u, in the copy tile (same layout as Y)
#pragma unroll
            for (int ks = 0; ks < 8; ++ks)
              mma_ss(tmem + kColT, d_tb + (uint64_t)(ks * 128), d_zmn + (uint64_t)(ks * 128), idesc_mnmn, 1);
          }
          mma_commit(bar_t);
          // every product that reads this stage's X or Y has been issued: the producer may refill
          // them (for the chunk after the next one) as soon as those products are done
          mma_commit(bar_empty + 8 * s);
          mbar_wait(bar_f, par, abort_flag, a.status, kStF);
          tc_fence_after();
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)
            mma_ts(tmem + kColW1, tmem + kColP + (ks >> 1) * 32 + (ks & 1) * 8, d_zmn + (uint64_t)(ks * 128),
                   idesc_kmn, ks > 0);
          mma_commit(bar_w);
          // the next chunk's X Y^T overwrites P, which the product above reads as P~
          mbar_wait(bar_w, par, abort_flag, a.status, kStW);
        }
        g0 += tk.cnt;
      }
    }
    __syncwarp();
  } else if (warp == kStoreWarp) {
    // ------------------------------------------------------------------ TMA stores
    if (lane == 0) {
      int g0 = 0;
      for (int k = 0; k < ntasks; ++k) {
        const Task tk = task_of(a, range(), k, ntasks);
        for (int it = 0; it < tk.cnt; ++it) {
          const int gi = g0 + it;
          const int n = rev ? (tk.nc - 1 - (tk.it0 + it)) : (tk.it0 + it);
          const int s = gi & 1;
          const uint32_t par = (uint32_t)gi & 1u;
          const int L = min(kChunk, tk.len - n * kChunk);
          mbar_wait(bar_h, par, abort_flag, a.status, kStH);
          if (L == kChunk) {
            const uint32_t zs = base + (uint32_t)s * kStageBytes + 2 * kTileBytes;
            const int tok0 = (int)tk.t_begin + n * kChunk;
            tma_store_4d(map_o, zs, 0, tk.h, tok0, tk.bidx);
            if (F128 || ap.fz > 64) tma_store_4d(map_o, zs + kBoxBytes, 64, tk.h, tok0, tk.bidx);
            tma_store_commit();
            tma_store_wait_read();
          }
          mbar_arrive(bar_emptyz + 8 * s);
        }
        g0 += tk.cnt;
      }
      tma_store_wait_all();
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ compute warps
    const int wg = warp >> 2, q4 = warp & 3;
    const int i = q4 * 32 + lane;  // row of every 128-row tile this thread works on
    const uint32_t tl = tmem + ((uint32_t)(32 * q4) << 16);
    // per-task quantities (kept few: they stay live across the chunk loop)
    int n_first = 0, t_len = 0, t_cnt = 0;  // first chunk index, tokens of the sequence, chunks of the task
    const float *ld_row = a.ld;             // &ld[b, t_begin + i, h]
    long long row_base = 0;                 // element offset of row (b, t_begin + i, h, 0)

    auto chunk_of = [&](int it) -> int { return rev ? n_first - it : n_first + it; };
    auto load_ld = [&](int it) -> float {
      if (it >= t_cnt) return 0.f;
      const int n = chunk_of(it);
      if (i >= t_len - n * kChunk) return 0.f;
      const float raw = ld_row[(long long)n * kChunk * a.ld_sn];
      return ACT ? log2_sigmoid(raw) : raw * kLog2e;
    };

    // Per-chunk decay quantities of this thread's row.
    struct Decay {
      float c;         // inclusive in-chunk cumulative log2 decay of row i
      float a0, a1;    // row factors of the factorised mask for this thread's two column batches
      float eg, s, u;  // e^g, output-row scale, Y-row scale
      bool wide;       // this row batch decays by more than 2^-64 end to end (warp-uniform)
    };
    // A: cumulative decays of step `it` of the task, cs/bs into buffer `buf`.  Contains a named
    // barrier.  A buffer is rewritten two chunks after it was filled; by then every thread has
    // arrived on bar_f of the chunk that read it (the tensor cores, and so the epilogue every
    // thread has since passed, wait for that).
    auto decay_of = [&](int it, float ldv, int buf) -> Decay {
      Decay d;
      const int L = t_len - chunk_of(it) * kChunk;  // rows >= L are padding
      float c = ldv;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const float nb = __shfl_up_sync(0xffffffffu, c, off);
        if (lane >= off) c += nb;
      }
      if (wg == 0 && lane == 31) sm->wsum[buf][q4] = c;
      named_bar_sync(1, kComputeThreads);
      // cumulative decay at the start (w_lo) / end (w_hi) of this thread's 32-row batch, over the
      // chunk (g), and at the reference edge of its two column batches wg and wg + 2
      const int e0 = rev ? wg : wg + 1, e1 = e0 + 2;
      float w_lo = 0.f, w_hi = 0.f, g = 0.f, r0 = 0.f, r1 = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float ws = sm->wsum[buf][w];
        g += ws;
        if (w < q4) w_lo += ws;
        if (w <= q4) w_hi += ws;
        if (w < e0) r0 += ws;
        if (w < e1) r1 += ws;
      }
      c += w_lo;
      d.c = c;
      d.wide = (w_lo - w_hi) > 64.f;
      d.a0 = rev ? ex2(r0 - c) : ex2(c - r0);
      d.a1 = rev ? ex2(r1 - c) : ex2(c - r1);
      d.eg = ex2(g);
      d.s = rev ? ex2(g - c) : ex2(c);
      d.u = (i < L) ? (rev ? ex2(c) : ex2(g - c)) : 0.f;
      if (wg == 0) {
        sm->cs[buf][i] = c;
        sm->bs[buf][i] = rev ? ((i < L) ? ex2(c - w_lo) : 0.f) : ex2(w_hi - c);
      }
      return d;
    };
    // D: state in -> 16-bit copy in shared memory (B operand of X T_in); T <- e^g T
    // low half of the split copy: T - round16(T), written over the high half once X T_hi is done;
    // the rescaling of T that state_copy skipped in split mode happens here
    auto state_copy_low = [&](float eg, uint32_t par) {
      mbar_wait(bar_x, par, abort_flag, a.status, kStX);
      tc_fence_after();
      uint8_t *box = gbase + kOffTb + wg * kBoxBytes;
      const float2 eg2 = make_float2(eg, eg);
#pragma unroll 1
      for (int hf = 0; hf < 2; ++hf) {  // 32 columns at a time keeps the register peak low
        uint32_t r[32];
        tmem_ld32(tl + kColT + (2 * wg + hf) * 32, r);
        tmem_wait_ld();
#pragma unroll
        for (int pc = 0; pc < 4; ++pc) {
          uint32_t w[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float x0 = __uint_as_float(r[pc * 8 + 2 * j]), x1 = __uint_as_float(r[pc * 8 + 2 * j + 1]);
            const float2 hi = Fmt<T>::unpack(Fmt<T>::pack(x0, x1));
            w[j] = Fmt<T>::pack(x0 - hi.x, x1 - hi.y);
          }
          *reinterpret_cast<uint4 *>(box + sw128_offset(i, hf * 4 + pc)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
#pragma unroll
        for (int k = 0; k < 32; k += 2) {
          const float2 a0 = mul2(f2(r[k], r[k + 1]), eg2);
          r[k] = __float_as_uint(a0.x); r[k + 1] = __float_as_uint(a0.y);
        }
        tmem_st32(tl + kColT + (2 * wg + hf) * 32, r);
      }
      tmem_wait_st();
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(bar_l);
    };
    auto state_copy = [&](float eg) {
      uint8_t *box = gbase + kOffTb + wg * kBoxBytes;
      const float2 eg2 = make_float2(eg, eg);
#pragma unroll 1
      for (int hf = 0; hf < 2; ++hf) {
        uint32_t r[32];
        tmem_ld32(tl + kColT + (2 * wg + hf) * 32, r);
        tmem_wait_ld();
#pragma unroll
        for (int pc = 0; pc < 4; ++pc) {
          uint4 v;
          v.x = Fmt<T>::pack(__uint_as_float(r[pc * 8 + 0]), __uint_as_float(r[pc * 8 + 1]));
          v.y = Fmt<T>::pack(__uint_as_float(r[pc * 8 + 2]), __uint_as_float(r[pc * 8 + 3]));
          v.z = Fmt<T>::pack(__uint_as_float(r[pc * 8 + 4]), __uint_as_float(r[pc * 8 + 5]));
          v.w = Fmt<T>::pack(__uint_as_float(r[pc * 8 + 6]), __uint_as_float(r[pc * 8 + 7]));
          *reinterpret_cast<uint4 *>(box + sw128_offset(i, hf * 4 + pc)) = v;
        }
        if (!split) {
#pragma unroll
          for (int k = 0; k < 32; k += 2) {
            const float2 a0 = mul2(f2(r[k], r[k + 1]), eg2);
            r[k] = __float_as_uint(a0.x); r[k + 1] = __float_as_uint(a0.y);
          }
          tmem_st32(tl + kColT + (2 * wg + hf) * 32, r);
        }
      }
      if (!split) tmem_wait_st();
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(bar_d);
    };

    int g0 = 0;
    for (int k = 0; k < ntasks; ++k) {
      {
        const Task tk = task_of(a, range(), k, ntasks);
        n_first = rev ? (tk.nc - 1 - tk.it0) : tk.it0;
        t_len = tk.len;
        t_cnt = tk.cnt;
        ld_row = a.ld + tk.bidx * a.ld_sb + tk.h * a.ld_sh + (tk.t_begin + i) * a.ld_sn;
        row_base = ((tk.bidx * (long long)a.N + tk.t_begin + i) * a.H + tk.h) * (long long)(F128 ? kChunk : ap.fz);

        // starting state -> tensor memory (this warpgroup's 64 columns): the caller's state, or
        // what the neighbouring CTA left in its hand-off slot
        const float *src = nullptr;
        bool src_tr = true;
        if (tk.waits) {
          if (tid == 0) {
            const int *flag = sc.flags + (blockIdx.x - sc.npass);
            const uint64_t t0 = globaltimer_ns();
            while (ld_acquire(flag) == 0 && *abort_flag == 0) {
              __nanosleep(200);
              if (globaltimer_ns() - t0 > 2000000000ull) {  // 2 s
                *abort_flag = 1;
                atomicCAS(a.status, 0, kStHandoff);
              }
            }
          }
          named_bar_sync(3, kComputeThreads);
          src = sc.handoff + (size_t)(blockIdx.x - sc.npass) * (kChunk * kChunk);
        } else if (ap.t0 != nullptr) {
          src = ap.t0 + ((long long)tk.seq * a.H + tk.h) * (long long)(F128 ? kChunk * kChunk : ap.fx * ap.fz);
          src_tr = ap.state_transposed != 0;
        }
        const bool narrow = !F128 && !tk.waits;  // the caller's state has the real widths
        for (int b2 = 0; b2 < 2; ++b2) {
          const int bt = 2 * wg + b2;
          uint32_t r[32];
          if (src == nullptr) {
#pragma unroll
            for (int kk = 0; kk < 32; ++kk) r[kk] = 0u;
          } else if (narrow) {  // (fx, fz) state: T[i][c] at c * fx + i (transposed) or i * fz + c
            const int fx = ap.fx, fz = ap.fz;
#pragma unroll
            for (int kk = 0; kk < 32; ++kk) {
              const int c = bt * 32 + kk;
              float val = 0.f;
              if (i < fx && c < fz) val = __ldcg(src + (src_tr ? c * fx + i : i * fz + c));
              r[kk] = __float_as_uint(val);
            }
          } else if (src_tr) {  // element (i, c) at c * 128 + i: a warp reads 128 contiguous bytes
#pragma unroll
            for (int kk = 0; kk < 32; ++kk) r[kk] = __float_as_uint(__ldcg(src + (bt * 32 + kk) * kChunk + i));
          } else {              // row i contiguous: 16-byte loads
            const float4 *row = reinterpret_cast<const float4 *>(src + i * kChunk + bt * 32);
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
              // the eight loads of a thread fall into one 128-byte line: through L1 (the caller's
              // state is read-only for the launch; hand-off slots never take this branch)
              const float4 v = __ldg(row + kk);
              r[4 * kk + 0] = __float_as_uint(v.x); r[4 * kk + 1] = __float_as_uint(v.y);
              r[4 * kk + 2] = __float_as_uint(v.z); r[4 * kk + 3] = __float_as_uint(v.w);
            }
          }
          tmem_st32(tl + kColT + bt * 32, r);
        }
        tmem_wait_st();
        // the next task's starting state: pull it into L2 now, it is needed when this task ends
        if (ap.t0 != nullptr && k + 1 < ntasks) {
          const Task nx = task_of(a, range(), k + 1, ntasks);
          if (!nx.waits) {
            if (F128) {
              const char *pn = reinterpret_cast<const char *>(ap.t0 + ((long long)nx.seq * a.H + nx.h) * (long long)(kChunk * kChunk));
              asm volatile("prefetch.global.L2 [%0];" ::"l"(pn + (size_t)tid * 128));
              asm volatile("prefetch.global.L2 [%0];" ::"l"(pn + (size_t)(tid + kComputeThreads) * 128));
            }
          }
        }
      }
      const int nc = t_cnt;

      Decay cur{};
      float ld_next = 0.f;
      if (nc > 0) {
        cur = decay_of(0, load_ld(0), g0 & 1);
        ld_next = load_ld(1);
        state_copy(cur.eg);
      }

      for (int it = 0; it < nc; ++it) {
        const int gi = g0 + it;
        const int n = chunk_of(it);
        const int s = gi & 1;
        const uint32_t ph = (uint32_t)(gi >> 1) & 1u, par = (uint32_t)gi & 1u;
        const int L = min(kChunk, t_len - n * kChunk);
        uint8_t *stage = gbase + (size_t)s * kStageBytes;
        const float c_i = cur.c;

        // ---- decays of the next chunk, while the tensor cores are still on this one's X Y^T
        Decay nxt{};
        if (it + 1 < nc) {  // uniform over the CTA
          nxt = decay_of(it + 1, ld_next, (gi + 1) & 1);
          ld_next = load_ld(it + 2);
        }
        if (split) {
          // the epilogue dots the output with this row of xrow, read from global memory: start
          // that fetch now (one 128-byte line per thread) so that it is in cache by then
          if (F128 && i < L) {
            const char *xr = reinterpret_cast<const char *>(static_cast<const T *>(ap.xrow) + row_base +
                                                              (long long)n * kChunk * a.H * kChunk + 64 * wg);
            asm volatile("prefetch.global.L1 [%0];" ::"l"(xr));
          }
          state_copy_low(cur.eg, par);
        }
        // ---- Y <- Y (.) u in place (this warpgroup's 64 columns), once X Y^T has consumed Y
        mbar_wait(bar_full + 8 * s, ph, abort_flag, a.status, kStFull);
        mbar_wait(bar_p, par, abort_flag, a.status, kStP);
        tc_fence_after();
        if (split) {
          // high half in place, low half into the copy tile, once X T_lo has let go of it
          mbar_wait(bar_u, par, abort_flag, a.status, kStU);
          uint8_t *ybox = stage + kTileBytes + wg * kBoxBytes;
          uint8_t *lbox = gbase + kOffTb + wg * kBoxBytes;
          const float2 u2 = make_float2(cur.u, cur.u);
#pragma unroll 2
          for (int pc = 0; pc < 8; ++pc) {
            const uint32_t off = sw128_offset(i, pc);
            const uint4 y = *reinterpret_cast<const uint4 *>(ybox + off);
            const uint32_t yw[4] = {y.x, y.y, y.z, y.w};
            uint32_t hw[4], lw[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 p = mul2(Fmt<T>::unpack(yw[j]), u2);
              hw[j] = Fmt<T>::pack(p.x, p.y);
              const float2 hf = Fmt<T>::unpack(hw[j]);
              lw[j] = Fmt<T>::pack(p.x - hf.x, p.y - hf.y);
            }
            *reinterpret_cast<uint4 *>(ybox + off) = make_uint4(hw[0], hw[1], hw[2], hw[3]);
            *reinterpret_cast<uint4 *>(lbox + off) = make_uint4(lw[0], lw[1], lw[2], lw[3]);
          }
        } else {
          uint8_t *ybox = stage + kTileBytes + wg * kBoxBytes;
          uint4 v[8];
#pragma unroll
          for (int pc = 0; pc < 8; ++pc) v[pc] = *reinterpret_cast<const uint4 *>(ybox + sw128_offset(i, pc));
          // u as a 16-bit value plus its 16-bit remainder: two packed 16-bit operations per
          // pair of elements instead of unpack, fp32 multiply and pack
          const uint32_t uh = Fmt<T>::pack(cur.u, cur.u);
          const float urem = cur.u - Fmt<T>::unpack(uh).x;
          const uint32_t ul = Fmt<T>::pack(urem, urem);
#pragma unroll
          for (int pc = 0; pc < 8; ++pc) {
            v[pc].x = Fmt<T>::scale(v[pc].x, uh, ul);
            v[pc].y = Fmt<T>::scale(v[pc].y, uh, ul);
            v[pc].z = Fmt<T>::scale(v[pc].z, uh, ul);
            v[pc].w = Fmt<T>::scale(v[pc].w, uh, ul);
          }
#pragma unroll
          for (int pc = 0; pc < 8; ++pc) *reinterpret_cast<uint4 *>(ybox + sw128_offset(i, pc)) = v[pc];
        }
        fence_proxy_async();
        mbar_arrive(bar_y);

        // ---- masked 16-bit P~ (first 16 columns of each 32-column batch of P).  This thread's
        // batches are wg and wg + 2 ({0,2} / {1,3} balances the triangular work); both loads
        // are issued before the one wait.
        {
          const bool dead0 = rev ? (wg < q4) : (wg > q4);          // warp-uniform
          const bool dead1 = rev ? (wg + 2 < q4) : (wg + 2 > q4);
          uint32_t r0[32], r1[32];
          if (!dead0) tmem_ld32(tl + kColP + wg * 32, r0);
          if (!dead1) tmem_ld32(tl + kColP + (wg + 2) * 32, r1);
          tmem_wait_ld();
          auto mask_batch = [&](const int b2, uint32_t(&r)[32], const bool dead) {
            const int bt = wg + 2 * b2;
            uint32_t pk[16];
            if (dead) {
#pragma unroll
              for (int kk = 0; kk < 16; ++kk) pk[kk] = 0u;
            } else if (bt == q4 && cur.wide) {
              // diagonal batch whose decay range is too wide to factorise: one exponential per element
#pragma unroll
              for (int kk = 0; kk < 32; kk += 2) {
                const int j = bt * 32 + kk;
                const float2 cj = *reinterpret_cast<const float2 *>(&sm->cs[gi & 1][j]);
                float m0, m1;
                if (!rev) {
                  m0 = (j <= i) ? ex2(c_i - cj.x) : 0.f;
                  m1 = (j + 1 <= i) ? ex2(c_i - cj.y) : 0.f;
                } else {
                  m0 = (j >= i && j < L) ? ex2(cj.x - c_i) : 0.f;
                  m1 = (j + 1 >= i && j + 1 < L) ? ex2(cj.y - c_i) : 0.f;
                }
                pk[kk >> 1] = Fmt<T>::pack(__uint_as_float(r[kk]) * m0, __uint_as_float(r[kk + 1]) * m1);
              }
            } else {
              // weight = (row factor) x (column factor), both relative to the batch edge next to
              // the diagonal; on the diagonal batch the entries beyond the diagonal are dropped
              const float ai = b2 ? cur.a1 : cur.a0;
              const float2 ai2 = make_float2(ai, ai);
#pragma unroll
              for (int kk = 0; kk < 32; kk += 4) {
                const float4 bj = *reinterpret_cast<const float4 *>(&sm->bs[gi & 1][bt * 32 + kk]);
                const float2 p0 = mul2(f2(r[kk + 0], r[kk + 1]), mul2(ai2, make_float2(bj.x, bj.y)));
                const float2 p1 = mul2(f2(r[kk + 2], r[kk + 3]), mul2(ai2, make_float2(bj.z, bj.w)));
                r[kk + 0] = __float_as_uint(p0.x); r[kk + 1] = __float_as_uint(p0.y);
                r[kk + 2] = __float_as_uint(p1.x); r[kk + 3] = __float_as_uint(p1.y);
              }
              if (bt == q4) {
                const uint32_t keep = rev ? (0xffffffffu << lane) : (0xffffffffu >> (31 - lane));
#pragma unroll
                for (int kk = 0; kk < 32; ++kk) r[kk] = ((keep >> kk) & 1u) ? r[kk] : 0u;
              }
#pragma unroll
              for (int kk = 0; kk < 32; kk += 2)
                pk[kk >> 1] = Fmt<T>::pack(__uint_as_float(r[kk]), __uint_as_float(r[kk + 1]));
            }
            tmem_st16(tl + kColP + bt * 32, pk);
          };
          mask_batch(0, r0, dead0);
          mask_batch(1, r1, dead1);
        }
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(bar_f);

        // ---- while the tensor cores finish this chunk: state copy of the next one
        if (it + 1 < nc) {  // uniform over the CTA
          mbar_wait(bar_t, par, abort_flag, a.status, kStT);  // T holds this chunk's final state
          tc_fence_after();
          state_copy(nxt.eg);
        }

        // ---- epilogue W = W1 + s_i W2 (this warpgroup's 64 columns)
        mbar_wait(bar_w, par, abort_flag, a.status, kStW);
        tc_fence_after();
        const bool full_chunk = (L == kChunk);
        const int fz = F128 ? kChunk : ap.fz;
        const long long row_off = row_base + (long long)n * kChunk * a.H * fz;
        const float s_i = cur.s;
        float rd = 0.f;
#pragma unroll 1
        for (int b2 = 0; b2 < 2; ++b2) {
          const int c0 = 64 * wg + 32 * b2;
          uint32_t w1[32], w2[32];
          tmem_ld32(tl + kColW1 + c0, w1);
          tmem_ld32(tl + kColW2 + c0, w2);
          tmem_wait_ld();
          float w[32];
          const float2 s2 = make_float2(s_i, s_i);
#pragma unroll
          for (int kk = 0; kk < 32; kk += 2) {
            const float2 t2 = fma2(s2, f2(w2[kk], w2[kk + 1]), f2(w1[kk], w1[kk + 1]));
            w[kk] = t2.x;
            w[kk + 1] = t2.y;
          }
          if (split && i < L) {  // row-dot operand present (uniform over the CTA)
            const uint4 *xp = reinterpret_cast<const uint4 *>(static_cast<const T *>(ap.xrow) + row_off + c0);
#pragma unroll
            for (int pc = 0; pc < 4; ++pc) {
              if (!F128 && c0 + pc * 8 >= fz) break;  // features beyond the real width are zero
              const uint4 xv = xp[pc];
              float2 f;
              f = Fmt<T>::unpack(xv.x); rd = fmaf(f.x, w[pc * 8 + 0], rd); rd = fmaf(f.y, w[pc * 8 + 1], rd);
              f = Fmt<T>::unpack(xv.y); rd = fmaf(f.x, w[pc * 8 + 2], rd); rd = fmaf(f.y, w[pc * 8 + 3], rd);
              f = Fmt<T>::unpack(xv.z); rd = fmaf(f.x, w[pc * 8 + 4], rd); rd = fmaf(f.y, w[pc * 8 + 5], rd);
              f = Fmt<T>::unpack(xv.w); rd = fmaf(f.x, w[pc * 8 + 6], rd); rd = fmaf(f.y, w[pc * 8 + 7], rd);
            }
          }
#pragma unroll
          for (int pc = 0; pc < 4; ++pc) {
            uint4 v;
            v.x = Fmt<T>::pack(w[pc * 8 + 0], w[pc * 8 + 1]);
            v.y = Fmt<T>::pack(w[pc * 8 + 2], w[pc * 8 + 3]);
            v.z = Fmt<T>::pack(w[pc * 8 + 4], w[pc * 8 + 5]);
            v.w = Fmt<T>::pack(w[pc * 8 + 6], w[pc * 8 + 7]);
            if (full_chunk) {
              // staging = this stage's Z tile (dead once the MMAs above have completed)
              *reinterpret_cast<uint4 *>(stage + 2 * kTileBytes + wg * kBoxBytes + sw128_offset(i, b2 * 4 + pc)) = v;
            } else if (i < L && (F128 || c0 + pc * 8 < fz)) {
              reinterpret_cast<uint4 *>(static_cast<T *>(ap.out) + row_off + c0)[pc] = v;
            }
          }
        }
        if (split) {  // uniform over the CTA
          if (wg == 1) sm->rd[i] = rd;
          named_bar_sync(2, kComputeThreads);
          if (wg == 0 && i < L) ap.rowdot[F128 ? (row_off >> 7) : (row_off / fz)] = rd + sm->rd[i];
        }
        if (full_chunk) fence_proxy_async();
        tc_fence_before();
        mbar_arrive(bar_h);
        cur = nxt;
      }
      g0 += nc;

      // end state -> the caller's buffer, or the hand-off slot when the sequence continues on
      // the next CTA
      {
        const Task tk = task_of(a, range(), k, ntasks);
        if (tk.publishes || ap.tfinal != nullptr) {
          tc_fence_after();
          float *dst = tk.publishes ? sc.handoff + (size_t)blockIdx.x * (kChunk * kChunk)
                                    : ap.tfinal + ((long long)tk.seq * a.H + tk.h) *
                                                      (long long)(F128 ? kChunk * kChunk : ap.fx * ap.fz);
          const bool dst_tr = tk.publishes || ap.state_transposed != 0;
          const bool narrow_out = !F128 && !tk.publishes;
          for (int b2 = 0; b2 < 2; ++b2) {
            const int bt = 2 * wg + b2;
            uint32_t r[32];
            tmem_ld32(tl + kColT + bt * 32, r);
            tmem_wait_ld();
            if (narrow_out) {
              const int fx = ap.fx, fzs = ap.fz;
#pragma unroll
              for (int kk = 0; kk < 32; ++kk) {
                const int c = bt * 32 + kk;
                if (i < fx && c < fzs) dst[ap.state_transposed ? c * fx + i : i * fzs + c] = __uint_as_float(r[kk]);
              }
            } else if (dst_tr) {
#pragma unroll
              for (int kk = 0; kk < 32; ++kk) dst[(bt * 32 + kk) * kChunk + i] = __uint_as_float(r[kk]);
            } else {
              float4 *row = reinterpret_cast<float4 *>(dst + i * kChunk + bt * 32);
#pragma unroll
              for (int kk = 0; kk < 8; ++kk)
                row[kk] = make_float4(__uint_as_float(r[4 * kk]), __uint_as_float(r[4 * kk + 1]),
                                      __uint_as_float(r[4 * kk + 2]), __uint_as_float(r[4 * kk + 3]));
            }
          }
          if (tk.publishes) {
            __threadfence();
            named_bar_sync(3, kComputeThreads);
            if (tid == 0) st_release(sc.flags + blockIdx.x, 1);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kProducerWarp) {
    if (lane == 0 && sm->abort_flag != 0) {
      // loads that were issued but never consumed must land before the CTA's shared memory is
      // released; wait for them with a limit of their own
      int dummy = 0;
      for (int it = max(0, sm->issued - kStages); it < sm->issued; ++it)
        mbar_wait(bar_full + 8 * (it & 1), (uint32_t)(it >> 1) & 1u, &dummy, nullptr, 0, 1u << 20);
      for (int it = max(0, sm->issuedz - kStages); it < sm->issuedz; ++it)
        mbar_wait(bar_fullz + 8 * (it & 1), (uint32_t)(it >> 1) & 1u, &dummy, nullptr, 0, 1u << 20);
    }
    __syncwarp();
    tmem_dealloc(tmem, 512);
  }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
// wprefix[s] = sum over sequences before s of (chunks + kTaskUnits); one block
__global__ void weight_prefix_kernel(const long long *cu, int M, long long *wprefix) {
  __shared__ long long part[1024];
  const int tid = threadIdx.x, per = (M + 1023) / 1024;
  const int lo = min(M, tid * per), hi = min(M, lo + per);
  long long sum = 0;
  for (int s = lo; s < hi; ++s) {
    const long long len = cu[s + 1] - cu[s];
    sum += (len + kChunk - 1) / kChunk + kTaskUnits;
  }
  part[tid] = sum;
  __syncthreads();
  for (int off = 1; off < 1024; off <<= 1) {
    const long long v = tid >= off ? part[tid - off] : 0;
    __syncthreads();
    part[tid] += v;
    __syncthreads();
  }
  long long run = part[tid] - sum;
  for (int s = lo; s < hi; ++s) {
    wprefix[s] = run;
    const long long len = cu[s + 1] - cu[s];
    run += (len + kChunk - 1) / kChunk + kTaskUnits;
  }
  if (tid == 1023) wprefix[M] = part[1023];
}

struct DeviceInfo {
  bool ready = false, attr[8] = {false, false, false, false, false, false, false, false}, pool_tried = false;
  int sms = 0, dev = 0;
  cudaMemPool_t pool = nullptr;  // hand-off scratch; made on first need, null if that failed
};

std::mutex g_info_mu;

// per-device facts (no allocation of any kind)
DeviceInfo *device_info() {
  static DeviceInfo info[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(g_info_mu);
  DeviceInfo &d = info[dev];
  if (!d.ready) {
    if (cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return nullptr;
    d.dev = dev;
    d.ready = true;
  }
  return &d;
}

// The stream-ordered pool the hand-off scratch of the split schedule comes from; created by the
// first launch that takes that schedule (never by a launch with no_scratch set).
cudaMemPool_t handoff_pool(DeviceInfo *d) {
  std::lock_guard<std::mutex> lock(g_info_mu);
  if (!d->pool_tried) {
    d->pool_tried = true;
    cudaMemPoolProps props = {};
    props.allocType = cudaMemAllocationTypePinned;
    props.handleTypes = cudaMemHandleTypeNone;
    props.location.type = cudaMemLocationTypeDevice;
    props.location.id = d->dev;
    if (cudaMemPoolCreate(&d->pool, &props) == cudaSuccess) {
      uint64_t keep = ~0ull;  // freed scratch stays in the pool for the next launch
      cudaMemPoolSetAttribute(d->pool, cudaMemPoolAttrReleaseThreshold, &keep);
    } else {
      d->pool = nullptr;
      cudaGetLastError();
    }
  }
  return d->pool;
}

inline size_t round_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

template <typename T>
int fill_pass(const ChunkPass &p, int dtype, PassMaps &m, ChunkArgs &a) {
  int rc;
  if ((rc = make_map(&m.x, p.x, dtype, p.B, p.N, p.H, p.fx)) != LA_OK) return rc;
  if ((rc = make_map(&m.y, p.y, dtype, p.B, p.N, p.H, p.fx)) != LA_OK) return rc;
  if ((rc = make_map(&m.z, p.z, dtype, p.B, p.N, p.H, p.fz)) != LA_OK) return rc;
  if ((rc = make_map(&m.o, p.out, dtype, p.B, p.N, p.H, p.fz)) != LA_OK) return rc;
  if (p.xrow != nullptr && (reinterpret_cast<uintptr_t>(p.xrow) & 15u)) return LA_ERR_MISALIGNED;
  if ((reinterpret_cast<uintptr_t>(p.t0) | reinterpret_cast<uintptr_t>(p.tfinal)) & 15u) return LA_ERR_MISALIGNED;
  a.xrow = p.xrow; a.rowdot = p.xrow ? p.rowdot : nullptr; a.out = p.out;
  a.ld = p.ld; a.ld_sb = p.ld_sb; a.ld_sn = p.ld_sn; a.ld_sh = p.ld_sh;
  a.t0 = p.t0; a.tfinal = p.tfinal; a.state_transposed = p.state_transposed; a.reverse = p.reverse;
  a.cu = reinterpret_cast<const long long *>(p.cu);
  a.B = p.B; a.N = p.N; a.H = p.H; a.M = p.M;
  a.fx = p.fx; a.fz = p.fz;
  a.ld_act = p.ld_act;
  a.status = status_word_ptr();
  if (a.status == nullptr) return LA_ERR_CUDA;
  return LA_OK;
}

// One launch for one pass (q == nullptr) or for two passes over the same tokens.
template <typename T>
int launch_t(const ChunkPass &p, const ChunkPass *q, int dtype, cudaStream_t stream) {
  alignas(64) Maps maps;
  Launch lp;
  int rc;
  if ((rc = fill_pass<T>(p, dtype, maps.p[0], lp.a[0])) != LA_OK) return rc;
  if ((rc = fill_pass<T>(q ? *q : p, dtype, maps.p[1], lp.a[1])) != LA_OK) return rc;
  DeviceInfo *di = device_info();
  if (di == nullptr) return LA_ERR_CUDA;
  const bool f128 = p.fx == 128 && p.fz == 128 && (q == nullptr || (q->fx == 128 && q->fz == 128));
  const bool act = p.ld_act != 0;
  auto kern = f128 ? (act ? chunk_pass_kernel<T, true, true> : chunk_pass_kernel<T, true, false>)
                   : (act ? chunk_pass_kernel<T, false, true> : chunk_pass_kernel<T, false, false>);
  bool &attr = di->attr[(dtype == LA_BF16 ? 0 : 1) + (f128 ? 0 : 2) + (act ? 4 : 0)];  // the attribute is per device
  if (!attr) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess)
      return LA_ERR_CUDA;
    attr = true;
  }
  const int npass = q ? 2 : 1;
  const long long pairs = (long long)(p.cu ? p.M : p.B) * p.H;
  const int ranges = di->sms / npass;
  Sched &sc = lp.sc;
  sc.npass = npass;
  sc.balanced = 0;
  sc.total = 0;
  sc.wprefix = nullptr;
  sc.handoff = nullptr;
  sc.flags = nullptr;
  long long grid = pairs * npass;
  void *scratch = nullptr;
  // Worth it when whole pairs per CTA would leave SMs idle in the last wave (always the case
  // with ragged documents).
  if (!p.no_scratch && ranges > 0 && pairs > ranges && (p.cu != nullptr || pairs % ranges != 0)) {
    // even split of the chunk space over one CTA per SM
    grid = (long long)ranges * npass;
    const size_t flag_bytes = round_up((size_t)grid * sizeof(int), 256);
    const size_t prefix_bytes = p.cu ? round_up(((size_t)p.M + 1) * sizeof(long long), 256) : 0;
    const size_t bytes = flag_bytes + prefix_bytes + (size_t)grid * kChunk * kChunk * sizeof(float);
    cudaMemPool_t pool = handoff_pool(di);
    if (pool == nullptr || cudaMallocFromPoolAsync(&scratch, bytes, pool, stream) != cudaSuccess) {
      cudaGetLastError();
      scratch = nullptr;
      grid = pairs * npass;
    } else {
      uint8_t *base = static_cast<uint8_t *>(scratch);
      sc.balanced = 1;
      sc.flags = reinterpret_cast<int *>(base);
      sc.handoff = reinterpret_cast<float *>(base + flag_bytes + prefix_bytes);
      sc.total = pairs * (((long long)p.N + kChunk - 1) / kChunk);
      bool ok = cudaMemsetAsync(sc.flags, 0, flag_bytes, stream) == cudaSuccess;
      if (ok && p.cu) {
        long long *wp = reinterpret_cast<long long *>(base + flag_bytes);
        sc.wprefix = wp;
        weight_prefix_kernel<<<1, 1024, 0, stream>>>(reinterpret_cast<const long long *>(p.cu), p.M, wp);
        ok = cudaGetLastError() == cudaSuccess;
      }
      if (!ok) {
        cudaFreeAsync(scratch, stream);
        return LA_ERR_CUDA;
      }
    }
  }
  kern<<<(unsigned)grid, kThreads, kSmemBytes, stream>>>(maps, lp);
  rc = launch_status();
  if (scratch != nullptr && cudaFreeAsync(scratch, stream) != cudaSuccess && rc == LA_OK) rc = LA_ERR_CUDA;
  return rc;
}

// ------------------------------------------------------------------------------------------------
// Self-test of the tensor-core building blocks: one 128x128x128 product per variant, operands
// staged exactly as the chunk kernel stages them.
//   0: D = A B^T   (A, B K-major from TMA)            -- the X Y^T product
//   1: D = A B     (A K-major, B MN-major from TMA)   -- operand forms of X T and P~ Z
//   2: D = A B     (A through registers into tensor memory, B MN-major)
//   3: D = A^T B   (A, B MN-major from TMA)           -- the state update
//   4: D = A B     (B written to shared memory by threads in the swizzled layout)
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128, 1)
umma_probe_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                  const T *a_g, const T *b_g, float *d, int variant, int *status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t *gbase = smem_raw + (base - raw);
  Small *sm = reinterpret_cast<Small *>(gbase + 2 * kTileBytes);
  const int tid = threadIdx.x, warp = tid >> 5;
  const uint32_t bar_full = smem_u32(&sm->full[0]), bar_mma = smem_u32(&sm->bar_w);
  volatile int *abort_flag = &sm->abort_flag;
  if (tid == 0) {
    mbar_init(bar_full, 1);
    mbar_init(bar_mma, 1);
    sm->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(&sm->tmem_base), 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm->tmem_base;
  const uint32_t as = base, bs = base + kTileBytes;
  if (tid == 0) {
    mbar_arrive_expect_tx(bar_full, 2 * kTileBytes);
    tma_load_4d(as, &map_a, bar_full, 0, 0, 0, 0);
    tma_load_4d(as + kBoxBytes, &map_a, bar_full, 64, 0, 0, 0);
    tma_load_4d(bs, &map_b, bar_full, 0, 0, 0, 0);
    tma_load_4d(bs + kBoxBytes, &map_b, bar_full, 64, 0, 0, 0);
  }
  mbar_wait(bar_full, 0, abort_flag, status, kStFull);
  const uint32_t tl = tmem + ((uint32_t)(32 * warp) << 16);
  if (variant == 2) {
    for (int bt = 0; bt < 4; ++bt) {
      uint32_t pk[16];
      const uint32_t *src = reinterpret_cast<const uint32_t *>(a_g + tid * 128 + bt * 32);
#pragma unroll
      for (int k = 0; k < 16; ++k) pk[k] = src[k];
      tmem_st16(tl + 128 + bt * 16, pk);
    }
    tmem_wait_st();
  }
  if (variant == 4) {
    for (int pc = 0; pc < 16; ++pc) {
      const uint4 v = reinterpret_cast<const uint4 *>(b_g + tid * 128)[pc];
      *reinterpret_cast<uint4 *>(gbase + kTileBytes + (pc >> 3) * kBoxBytes + sw128_offset(tid, pc & 7)) = v;
    }
    fence_proxy_async();
  }
  tc_fence_before();
  __syncthreads();
  if (tid == 0) {
    tc_fence_after();
    for (int ks = 0; ks < 8; ++ks) {
      if (variant == 0)
        mma_ss(tmem, desc_kmajor(as + kslice(ks)), desc_kmajor(bs + kslice(ks)),
               instr_desc(Fmt<T>::kAB, 0, 0, 128, 128), ks > 0);
      else if (variant == 1 || variant == 4)
        mma_ss(tmem, desc_kmajor(as + kslice(ks)), desc_mnmajor(bs + ks * 2048, kBoxBytes),
               instr_desc(Fmt<T>::kAB, 0, 1, 128, 128), ks > 0);
      else if (variant == 2)
        mma_ts(tmem, tmem + 128 + ks * 8, desc_mnmajor(bs + ks * 2048, kBoxBytes),
               instr_desc(Fmt<T>::kAB, 0, 1, 128, 128), ks > 0);
      else
        mma_ss(tmem, desc_mnmajor(as + ks * 2048, kBoxBytes), desc_mnmajor(bs + ks * 2048, kBoxBytes),
               instr_desc(Fmt<T>::kAB, 1, 1, 128, 128), ks > 0);
    }
    mma_commit(bar_mma);
  }
  mbar_wait(bar_mma, 0, abort_flag, status, kStW);
  tc_fence_after();
  for (int bt = 0; bt < 4; ++bt) {
    uint32_t r[32];
    tmem_ld32(tl + bt * 32, r);
    tmem_wait_ld();
#pragma unroll
    for (int k = 0; k < 32; ++k) d[tid * 128 + bt * 32 + k] = __uint_as_float(r[k]);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 256);
}

// The give-up path of mbar_wait on its own: the barrier below is initialised and never arrived on,
// so the wait runs out after limit_us, raises the abort flag and records kStProbe; a second wait
// on the same barrier must then return at once.
constexpr int kStProbe = 199;
__global__ void wait_probe_kernel(uint32_t limit_us, int *status) {
  __shared__ unsigned long long bar;
  __shared__ int abort_flag;
  const uint32_t b = smem_u32(&bar);
  if (threadIdx.x == 0) {
    mbar_init(b, 1);
    abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();
  volatile int *af = &abort_flag;
  mbar_wait(b, 0, af, status, kStProbe, limit_us);
  mbar_wait(b, 0, af, status, kStProbe + 1, 1u << 22);  // returns at once: the CTA has given up
}

template <typename T>
int probe_t(int variant, const void *a, const void *b, float *d, int dtype, cudaStream_t stream) {
  alignas(64) CUtensorMap ma, mb;
  int rc;
  if ((rc = make_map(&ma, a, dtype, 1, 128, 1, 128)) != LA_OK) return rc;
  if ((rc = make_map(&mb, b, dtype, 1, 128, 1, 128)) != LA_OK) return rc;
  int *status = status_word_ptr();
  if (status == nullptr) return LA_ERR_CUDA;
  const int smem = 2 * kTileBytes + kSmallBytes + 1024;
  auto kern = umma_probe_kernel<T>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return LA_ERR_CUDA;
  kern<<<1, 128, smem, stream>>>(ma, mb, static_cast<const T *>(a), static_cast<const T *>(b), d, variant, status);
  return launch_status();
}

}  // namespace

int umma_probe(int variant, const void *a, const void *b, float *d, int dtype, cudaStream_t stream) {
  if (a == nullptr || b == nullptr || d == nullptr) return LA_ERR_NULL_POINTER;
  if (variant < 0 || variant > 4) return LA_ERR_BAD_SHAPE;
  if (dtype == LA_BF16) return probe_t<__nv_bfloat16>(variant, a, b, d, dtype, stream);
  if (dtype == LA_F16) return probe_t<__half>(variant, a, b, d, dtype, stream);
  return LA_ERR_UNSUPPORTED;
}

int wait_probe(uint32_t limit_us, cudaStream_t stream) {
  int *status = status_word_ptr();
  if (status == nullptr) return LA_ERR_CUDA;
  wait_probe_kernel<<<1, 64, 0, stream>>>(limit_us, status);
  return launch_status();
}

bool chunk_supported(int64_t N, int64_t D, int64_t E, int dtype) {
  // head dimensions up to 128 in multiples of 8 (a row of a tensor must stay 16-byte aligned)
  return (dtype == LA_BF16 || dtype == LA_F16) && D >= 8 && E >= 8 && D <= 128 && E <= 128 && D % 8 == 0 &&
         E % 8 == 0 && N >= 128;
}

namespace {
int check_pass(const ChunkPass &p) {
  if (p.x == nullptr || p.y == nullptr || p.z == nullptr || p.out == nullptr || p.ld == nullptr)
    return LA_ERR_NULL_POINTER;
  const int nb = p.cu ? p.M : p.B;
  if (nb <= 0 || p.H <= 0 || p.N <= 0) return LA_ERR_BAD_SHAPE;
  if (p.fx < 8 || p.fz < 8 || p.fx > 128 || p.fz > 128 || p.fx % 8 || p.fz % 8) return LA_ERR_UNSUPPORTED;
  if ((int64_t)nb * p.H * 2 > 0x7fffffff) return LA_ERR_TOO_LARGE;
  return LA_OK;
}
}  // namespace

int launch_chunk_pass(const ChunkPass &p, int dtype, cudaStream_t stream) {
  const int rc = check_pass(p);
  if (rc != LA_OK) return rc;
  if (dtype == LA_BF16) return launch_t<__nv_bfloat16>(p, nullptr, dtype, stream);
  if (dtype == LA_F16) return launch_t<__half>(p, nullptr, dtype, stream);
  return LA_ERR_UNSUPPORTED;
}

int launch_chunk_pass_pair(const ChunkPass &p, const ChunkPass &q, int dtype, cudaStream_t stream) {
  int rc = check_pass(p);
  if (rc == LA_OK) rc = check_pass(q);
  if (rc != LA_OK) return rc;
  if (p.B != q.B || p.N != q.N || p.H != q.H || p.M != q.M || p.cu != q.cu || p.reverse != q.reverse ||
      p.ld != q.ld || p.ld_sb != q.ld_sb || p.ld_sn != q.ld_sn || p.ld_sh != q.ld_sh || p.ld_act != q.ld_act)
    return LA_ERR_BAD_SHAPE;
  if (dtype == LA_BF16) return launch_t<__nv_bfloat16>(p, &q, dtype, stream);
  if (dtype == LA_F16) return launch_t<__half>(p, &q, dtype, stream);
  return LA_ERR_UNSUPPORTED;
}

}  // namespace la
