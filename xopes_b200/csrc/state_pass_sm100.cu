// State-only pass of scalar-decay linear attention on 5th-generation tensor cores (sm_100a).
//
// For every (sequence, head) it accumulates what the tokens of the sequence alone contribute to
// the running state, without producing any output rows:
//
//   forward  flow:  T = sum_j e^{G - c_j} y_j^T z_j      (state at the END of the sequence from a zero start)
//   reverse  flow:  T = sum_j e^{c_j}     y_j^T z_j      (state at the START, flowing backwards from a zero end)
//
// with c_j the inclusive cumulative log decay from the sequence's first token and G its total.
// (y, z) = (k, v) forward gives the KV state S; (q, do) reverse gives dS; (v, k) / (do, q) give
// their transposes.  This is the associative half of the recurrence
// (xopes/ops/lightning_attn/scalar_decay/README_CR_CN.md: S_out = e^g S_in + (K e^r)^T V): a long
// sequence cut into segments needs only these per-segment states and totals to know the state
// entering each segment (la_lasd_fold_states), after which all segments run in parallel from their
// true states.  It reads two of the operand tensors once (512 B per token and head) and writes
// 64 KB per segment.
//
// One CTA per (segment, head).  The forward flow walks the chunks LAST to FIRST and the reverse
// flow FIRST to LAST, so the decay of a row relative to the far end of the segment is a running
// sum that only ever decreases: every factor is <= 1 and the fp32 state in tensor memory is only
// ever added to (no rescaling of the accumulator between chunks).  Warps 0-3 (one row of the
// 128-token chunk per thread) scale Y in place, warp 4 issues TMA loads (3 stages, never
// multicast), warp 5 issues tcgen05.mma.  Every mbarrier wait is bounded.
#include <cuda.h>

#include "chunk.cuh"
#include "sm100_ptx.cuh"
#include "tile_common.cuh"

namespace la {
namespace {

using namespace ptx;
using namespace tile;

constexpr int kChunk = 128;
constexpr int kTileBytes = 32768, kBoxBytes = 16384;
constexpr int kStages = 3;
constexpr int kStageBytes = 2 * kTileBytes;
constexpr int kOffSmall = kStages * kStageBytes;
constexpr int kSmallBytes = 1024;
constexpr int kSmemBytes = kOffSmall + kSmallBytes;
constexpr int kComputeThreads = 128;
constexpr int kThreads = kComputeThreads + 64;
constexpr float kLog2e = 1.4426950408889634f;
constexpr int kStFull = 401, kStEmpty = 402, kStY = 403, kStDone = 404, kStAlign = 413;

struct Small {
  unsigned long long full[kStages], empty[kStages], bar_y[kStages], done;
  uint32_t tmem_base;
  int abort_flag;
  int issued;
  alignas(16) float wsum[2][4];
};
static_assert(sizeof(Small) <= kSmallBytes, "small area overflow");

struct StateArgs {
  const float *ld;
  long long ld_sb, ld_sn, ld_sh;
  const long long *cu;
  float *states;  // (nb, H, 128, 128): element (i, c) at i * 128 + c, i = feature of y, c = feature of z
  float *gsum;    // (nb, H) total log decay of each sequence (natural log), optional
  int B, N, H, M, reverse;
  int ranges;  // 1: cu holds M (begin, end) pairs instead of M + 1 boundaries
  int ld_act;  // 1: the log decay is logsigmoid(ld)
  int *status;
};

template <typename T>
__global__ void __launch_bounds__(kThreads, 1)
state_pass_kernel(const __grid_constant__ CUtensorMap map_y, const __grid_constant__ CUtensorMap map_z,
                  const StateArgs a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  uint8_t *gbase = smem_raw;
  Small *sm = reinterpret_cast<Small *>(gbase + kOffSmall);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (base & 1023u) {
    if (tid == 0) atomicCAS(a.status, 0, kStAlign);
    return;
  }
  const int seq = blockIdx.x / a.H, h = blockIdx.x - seq * a.H;
  long long t_begin = 0, t_end = a.N;
  int bidx = seq;
  if (a.cu != nullptr) {
    t_begin = a.ranges ? a.cu[2 * seq] : a.cu[seq];
    t_end = a.ranges ? a.cu[2 * seq + 1] : a.cu[seq + 1];
    bidx = 0;
  }
  const int len = (int)(t_end - t_begin);
  const int nc = (len + kChunk - 1) / kChunk;
  // forward flow visits the chunks last to first, reverse flow first to last
  const bool back = a.reverse == 0;

  const uint32_t bar_full = smem_u32(&sm->full[0]), bar_empty = smem_u32(&sm->empty[0]);
  const uint32_t bar_y = smem_u32(&sm->bar_y[0]), bar_done = smem_u32(&sm->done);
  volatile int *abort_flag = &sm->abort_flag;
  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
      mbar_init(bar_y + 8 * s, kComputeThreads);
    }
    mbar_init(bar_done, 1);
    sm->abort_flag = 0;
    sm->issued = 0;
    fence_barrier_init();
  }
  if (warp == 4) {
    tmem_alloc(smem_u32(&sm->tmem_base), 128);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm->tmem_base;

  if (warp == 4) {
    // ------------------------------------------------------------------ TMA loads
    if (lane == 0) {
      prefetch_tmap(&map_y);
      prefetch_tmap(&map_z);
      int n_issued = 0;
      for (int it = 0; it < nc; ++it) {
        const int n = back ? (nc - 1 - it) : it;
        const int s = it % kStages;
        const uint32_t ph = (uint32_t)(it / kStages) & 1u;
        const uint32_t dst = base + (uint32_t)s * kStageBytes;
        const int tok0 = (int)t_begin + n * kChunk;
        mbar_wait(bar_empty + 8 * s, ph ^ 1u, abort_flag, a.status, kStEmpty);
        if (*abort_flag) break;
        const uint32_t fb = bar_full + 8 * s;
        mbar_arrive_expect_tx(fb, 2 * kTileBytes);
        tma_load_4d(dst, &map_y, fb, 0, h, tok0, bidx);
        tma_load_4d(dst + kBoxBytes, &map_y, fb, 64, h, tok0, bidx);
        tma_load_4d(dst + kTileBytes, &map_z, fb, 0, h, tok0, bidx);
        tma_load_4d(dst + kTileBytes + kBoxBytes, &map_z, fb, 64, h, tok0, bidx);
        n_issued = it + 1;
      }
      sm->issued = n_issued;
    }
    __syncwarp();
  } else if (warp == 5) {
    // ------------------------------------------------------------------ tensor-core issue
    if (lane == 0) {
      const uint32_t idesc = instr_desc(Fmt<T>::kAB, 1, 1, 128, 128);
      for (int it = 0; it < nc; ++it) {
        const int s = it % kStages;
        const uint32_t ph = (uint32_t)(it / kStages) & 1u;
        const uint32_t ys = base + (uint32_t)s * kStageBytes, zs = ys + kTileBytes;
        const uint64_t d_y = desc_mnmajor(ys, kBoxBytes), d_z = desc_mnmajor(zs, kBoxBytes);
        mbar_wait(bar_y + 8 * s, ph, abort_flag, a.status, kStY);
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          mma_ss(tmem, d_y + (uint64_t)(ks * 128), d_z + (uint64_t)(ks * 128), idesc, (it > 0 || ks > 0) ? 1u : 0u);
        mma_commit(bar_empty + 8 * s);
      }
      mma_commit(bar_done);
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ compute warps: Y <- Y (.) u
    const int i = tid;  // row of the chunk
    const float *ld_row = a.ld + bidx * a.ld_sb + h * a.ld_sh + (t_begin + i) * a.ld_sn;
    auto load_ld = [&](int it) -> float {
      if (it >= nc) return 0.f;
      const int n = back ? (nc - 1 - it) : it;
      if (i >= len - n * kChunk) return 0.f;
      const float raw = ld_row[(long long)n * kChunk * a.ld_sn];
      return a.ld_act ? log2_sigmoid(raw) : raw * kLog2e;
    };
    float run = 0.f;          // log2 decay between this chunk and the far end of the sequence
    float ld_next = load_ld(0);
    for (int it = 0; it < nc; ++it) {
      const int n = back ? (nc - 1 - it) : it;
      const int s = it % kStages;
      const uint32_t ph = (uint32_t)(it / kStages) & 1u;
      const int L = min(kChunk, len - n * kChunk);
      const float ldv = ld_next;
      ld_next = load_ld(it + 1);
      // inclusive cumulative log2 decay of the chunk's rows
      float c = ldv;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const float nb = __shfl_up_sync(0xffffffffu, c, off);
        if (lane >= off) c += nb;
      }
      if (lane == 31) sm->wsum[it & 1][warp] = c;
      named_bar_sync(1, kComputeThreads);
      float w_lo = 0.f, g = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float ws = sm->wsum[it & 1][w];
        g += ws;
        if (w < warp) w_lo += ws;
      }
      c += w_lo;
      // forward flow: decay from row i (exclusive) to the end of the sequence; reverse flow: from
      // the start of the sequence to row i (inclusive).  Both exponents are <= 0.
      const float u = (i < L) ? ex2(run + (back ? (g - c) : c)) : 0.f;
      run += g;
      mbar_wait(bar_full + 8 * s, ph, abort_flag, a.status, kStFull);
      uint8_t *ytile = gbase + (size_t)s * kStageBytes;
      const uint32_t uh = Fmt<T>::pack(u, u);
      const float urem = u - Fmt<T>::unpack(uh).x;
      const uint32_t ul = Fmt<T>::pack(urem, urem);
#pragma unroll
      for (int bx = 0; bx < 2; ++bx) {
        uint4 v[8];
#pragma unroll
        for (int pc = 0; pc < 8; ++pc) v[pc] = *reinterpret_cast<const uint4 *>(ytile + bx * kBoxBytes + sw128_offset(i, pc));
#pragma unroll
        for (int pc = 0; pc < 8; ++pc) {
          v[pc].x = Fmt<T>::scale(v[pc].x, uh, ul);
          v[pc].y = Fmt<T>::scale(v[pc].y, uh, ul);
          v[pc].z = Fmt<T>::scale(v[pc].z, uh, ul);
          v[pc].w = Fmt<T>::scale(v[pc].w, uh, ul);
        }
#pragma unroll
        for (int pc = 0; pc < 8; ++pc) *reinterpret_cast<uint4 *>(ytile + bx * kBoxBytes + sw128_offset(i, pc)) = v[pc];
      }
      fence_proxy_async();
      mbar_arrive(bar_y + 8 * s);
    }
    // the state -> global memory (row i, 128 contiguous floats)
    if (nc > 0) mbar_wait(bar_done, 0, abort_flag, a.status, kStDone);
    tc_fence_after();
    float *dst = a.states + ((long long)seq * a.H + h) * (long long)(kChunk * kChunk) + (long long)i * kChunk;
    const uint32_t tl = tmem + ((uint32_t)(32 * warp) << 16);
    for (int bt = 0; bt < 4; ++bt) {
      uint32_t r[32];
      if (nc > 0) {
        tmem_ld32(tl + bt * 32, r);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int k = 0; k < 32; ++k) r[k] = 0u;
      }
      float4 *row = reinterpret_cast<float4 *>(dst + bt * 32);
#pragma unroll
      for (int k = 0; k < 8; ++k)
        row[k] = make_float4(__uint_as_float(r[4 * k]), __uint_as_float(r[4 * k + 1]), __uint_as_float(r[4 * k + 2]),
                             __uint_as_float(r[4 * k + 3]));
    }
    if (tid == 0 && a.gsum != nullptr) a.gsum[(long long)seq * a.H + h] = run * (1.f / kLog2e);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    if (lane == 0 && sm->abort_flag != 0) {
      int dummy = 0;
      for (int it = max(0, sm->issued - kStages); it < sm->issued; ++it)
        mbar_wait(bar_full + 8 * (it % kStages), (uint32_t)(it / kStages) & 1u, &dummy, nullptr, 0, 1u << 20);
    }
    __syncwarp();
    tmem_dealloc(tmem, 128);
  }
}

template <typename T>
int launch_t(const StatePass &p, int dtype, cudaStream_t stream) {
  alignas(64) CUtensorMap my, mz;
  int rc;
  if ((rc = make_map(&my, p.y, dtype, p.B, p.N, p.H)) != LA_OK) return rc;
  if ((rc = make_map(&mz, p.z, dtype, p.B, p.N, p.H)) != LA_OK) return rc;
  if (reinterpret_cast<uintptr_t>(p.states) & 15u) return LA_ERR_MISALIGNED;
  StateArgs a;
  a.ld = p.ld; a.ld_sb = p.ld_sb; a.ld_sn = p.ld_sn; a.ld_sh = p.ld_sh;
  a.cu = reinterpret_cast<const long long *>(p.cu);
  a.states = p.states; a.gsum = p.gsum;
  a.B = p.B; a.N = p.N; a.H = p.H; a.M = p.M; a.reverse = p.reverse; a.ranges = p.ranges;
  a.ld_act = p.ld_act;
  a.status = status_word_ptr();
  if (a.status == nullptr) return LA_ERR_CUDA;
  auto kern = state_pass_kernel<T>;
  const cudaError_t ea = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
  if (ea != cudaSuccess) {
    note_cuda_error(ea, "cudaFuncSetAttribute(state_pass_kernel)");
    return LA_ERR_CUDA;
  }
  const long long nb = p.cu ? p.M : p.B;
  kern<<<(unsigned)(nb * p.H), kThreads, kSmemBytes, stream>>>(my, mz, a);
  return launch_status();
}

// out[k] = state entering segment k (forward flow: at its first token; reverse flow: after its last),
// from the segments' own contributions local[k] and total log decays gsum[k]:
//   forward:  s = first(k) ? ext[doc(k)] : s ;  out[k] = s ;  s = local[k] + e^{gsum[k]} s   (k ascending)
//   reverse:  s = last(k)  ? ext[doc(k)] : s ;  out[k] = s ;  s = local[k] + e^{gsum[k]} s   (k descending)
// seg rows are {document, first-of-document, last-of-document, row of `local` holding the segment's
// own state or -1 if it was not computed (then it counts as zero: fine for a segment nothing
// follows)}.  ends[doc] (optional, one row per document) receives the state after the document's
// last segment in fold order: its end state (forward) or the state before its first token (reverse).
__global__ void fold_states_kernel(const float *__restrict__ local, const float *__restrict__ gsum,
                                   const int *__restrict__ seg, const int *__restrict__ emit,
                                   const float *__restrict__ ext, float *__restrict__ out,
                                   float *__restrict__ ends, int nseg, int H, int DE, int reverse) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long hde = (long long)H * DE;
  if (idx >= hde) return;
  const int h = (int)(idx / DE);
  float s = 0.f;
  for (int kk = 0; kk < nseg; ++kk) {
    const int k = reverse ? nseg - 1 - kk : kk;
    const bool fresh = seg[4 * k + (reverse ? 2 : 1)] != 0;
    if (fresh) s = ext != nullptr ? ext[(long long)seg[4 * k] * hde + idx] : 0.f;
    const int slot = emit != nullptr ? emit[k] : k;  // -1: nobody needs the state entering this piece
    if (slot >= 0 && out != nullptr) out[slot * hde + idx] = s;
    const int li = seg[4 * k + 3];
    s = li >= 0 ? local[li * hde + idx] + expf(gsum[(long long)li * H + h]) * s : 0.f;
    if (ends != nullptr && seg[4 * k + (reverse ? 1 : 2)] != 0) ends[(long long)seg[4 * k] * hde + idx] = s;
  }
}

}  // namespace

int launch_state_pass(const StatePass &p, int dtype, cudaStream_t stream) {
  if (p.y == nullptr || p.z == nullptr || p.ld == nullptr || p.states == nullptr) return LA_ERR_NULL_POINTER;
  const long long nb = p.cu ? p.M : p.B;
  if (nb <= 0 || p.H <= 0 || p.N <= 0) return LA_ERR_BAD_SHAPE;
  if (nb * p.H > 0x7fffffffLL) return LA_ERR_TOO_LARGE;
  if (dtype == LA_BF16) return launch_t<__nv_bfloat16>(p, dtype, stream);
  if (dtype == LA_F16) return launch_t<__half>(p, dtype, stream);
  return LA_ERR_UNSUPPORTED;
}

int launch_fold_states(const float *local, const float *gsum, const int *seg, const int *emit, const float *ext,
                       float *out, float *ends, int nseg, int H, int DE, int reverse, cudaStream_t st) {
  const long long hde = (long long)H * DE;
  const int threads = 256;
  fold_states_kernel<<<(unsigned)((hde + threads - 1) / threads), threads, 0, st>>>(local, gsum, seg, emit, ext, out, ends,
                                                                                   nseg, H, DE, reverse);
  return launch_status();
}

}  // namespace la

// ================================================================================================
// Vector decay (per-token, per-feature log decay on the features of y).
//
//   forward  flow:  T[d][e] = sum_j e^{G_d - c_jd} y_jd z_je        G_d = total, c_jd inclusive cumulative
//   reverse  flow:  T[d][e] = sum_j e^{c_jd}       y_jd z_je
//
// Same walk as the scalar kernel (forward flow last chunk first, reverse flow first chunk first),
// with a running per-feature sum, so every factor is <= 1 whatever the decay: unlike the chunk
// kernels this pass has no range limit.  Per chunk the fp32 decay tile (64 KB, TMA) is turned in
// place into the exponents of the factors by the cumulative-sum scheme of the vector-decay chunk
// kernel (thread = 4 features x 16 rows, segment totals through shared memory), then Y is scaled
// row by row.  256 compute threads, a TMA warp, a tensor-core issue warp; Y and Z double-buffered,
// the decay tile single-buffered.
// ================================================================================================
namespace la {
namespace {

namespace vec {
constexpr int kStagesV = 1;                                 // Y and Z: one stage (the product that reads them is short)
constexpr int kStagesCk = 2;                                // decay tile: two, the next one loads during this chunk's sums
constexpr int kOffYZ = 0;                                  // Y 32 KB + Z 32 KB
constexpr int kOffCk = kStagesV * 2 * kTileBytes;           // 2 x 64 KB fp32 decay tiles
constexpr int kCkBytes = 65536;
constexpr int kOffSeg = kOffCk + kStagesCk * kCkBytes;      // [8][128] segment totals
constexpr int kOffRun = kOffSeg + 8 * 128 * 4;              // [128] running per-feature log2 decay
constexpr int kOffSmallV = kOffRun + 512;
constexpr int kSmemBytesV = kOffSmallV + 1024;
constexpr int kComputeV = 256;
constexpr int kThreadsV = kComputeV + 64;
constexpr int kStFullV = 421, kStEmptyV = 422, kStYV = 423, kStDoneV = 424, kStAlignV = 433;

struct SmallV {
  unsigned long long full_ck[kStagesCk], empty_ck[kStagesCk], full_yz[kStagesV], empty_yz[kStagesV], bar_y[kStagesV], done;
  uint32_t tmem_base;
  int abort_flag;
  int issued_ck, issued_yz;
};

struct StateVecArgs {
  const long long *cu;
  float *states;  // (nb, H, 128, 128)
  float *gsum;    // (nb, H, 128) total log decay per feature (natural log)
  int B, N, H, M, reverse, ranges, ld_act, ld16;
  int *status;
};

__device__ __forceinline__ uint32_t ck_off(int i, int d) {
  return (uint32_t)(d >> 5) * kBoxBytes + (uint32_t)i * 128u + (uint32_t)((((d & 31) >> 2) ^ (i & 7)) << 4);
}
}  // namespace vec

template <typename T>
__global__ void __launch_bounds__(vec::kThreadsV, 1)
state_pass_vec_kernel(const __grid_constant__ CUtensorMap map_y, const __grid_constant__ CUtensorMap map_z,
                      const __grid_constant__ CUtensorMap map_ld, const vec::StateVecArgs a) {
  using namespace vec;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  uint8_t *gbase = smem_raw;
  SmallV *sm = reinterpret_cast<SmallV *>(gbase + kOffSmallV);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (base & 1023u) {
    if (tid == 0) atomicCAS(a.status, 0, kStAlignV);
    return;
  }
  const int seq = blockIdx.x / a.H, h = blockIdx.x - seq * a.H;
  long long t_begin = 0, t_end = a.N;
  int bidx = seq;
  if (a.cu != nullptr) {
    t_begin = a.ranges ? a.cu[2 * seq] : a.cu[seq];
    t_end = a.ranges ? a.cu[2 * seq + 1] : a.cu[seq + 1];
    bidx = 0;
  }
  const int len = (int)(t_end - t_begin);
  const int nc = (len + kChunk - 1) / kChunk;
  const bool back = a.reverse == 0;

  const uint32_t full_ck = smem_u32(&sm->full_ck[0]), empty_ck = smem_u32(&sm->empty_ck[0]);
  const uint32_t full_yz = smem_u32(&sm->full_yz[0]), empty_yz = smem_u32(&sm->empty_yz[0]);
  const uint32_t bar_y = smem_u32(&sm->bar_y[0]), bar_done = smem_u32(&sm->done);
  volatile int *abort_flag = &sm->abort_flag;
  if (tid == 0) {
    for (int s = 0; s < kStagesCk; ++s) {
      mbar_init(full_ck + 8 * s, 1);
      mbar_init(empty_ck + 8 * s, kComputeV);
    }
    for (int s = 0; s < kStagesV; ++s) {
      mbar_init(full_yz + 8 * s, 1);
      mbar_init(empty_yz + 8 * s, 1);
      mbar_init(bar_y + 8 * s, kComputeV);
    }
    mbar_init(bar_done, 1);
    sm->abort_flag = 0;
    sm->issued_ck = sm->issued_yz = 0;
    fence_barrier_init();
  }
  if (warp == 8) {
    tmem_alloc(smem_u32(&sm->tmem_base), 128);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm->tmem_base;

  if (warp == 8) {
    // ------------------------------------------------------------------ TMA loads
    if (lane == 0) {
      int n_ck = 0, n_yz = 0;
      for (int it = 0; it < nc; ++it) {
        const int n = back ? (nc - 1 - it) : it;
        const int s = it % kStagesV;
        const uint32_t ph = (uint32_t)(it / kStagesV) & 1u;
        const int sc = it % kStagesCk;
        const uint32_t phc = (uint32_t)(it / kStagesCk) & 1u;
        const int tok0 = (int)t_begin + n * kChunk;
        mbar_wait(empty_ck + 8 * sc, phc ^ 1u, abort_flag, a.status, kStEmptyV);
        if (*abort_flag) break;
        mbar_arrive_expect_tx(full_ck + 8 * sc, a.ld16 ? kCkBytes / 2 : kCkBytes);
        if (a.ld16) {  // two boxes of 64 16-bit features into the first half of the slot
          tma_load_4d(base + kOffCk + sc * kCkBytes, &map_ld, full_ck + 8 * sc, 0, h, tok0, bidx);
          tma_load_4d(base + kOffCk + sc * kCkBytes + kBoxBytes, &map_ld, full_ck + 8 * sc, 64, h, tok0, bidx);
        } else {
#pragma unroll
          for (int gq = 0; gq < 4; ++gq)
            tma_load_4d(base + kOffCk + sc * kCkBytes + gq * kBoxBytes, &map_ld, full_ck + 8 * sc, 32 * gq, h, tok0, bidx);
        }
        n_ck = it + 1;
        mbar_wait(empty_yz + 8 * s, ph ^ 1u, abort_flag, a.status, kStEmptyV);
        if (*abort_flag) break;
        const uint32_t dst = base + kOffYZ + (uint32_t)s * 2 * kTileBytes, fb = full_yz + 8 * s;
        mbar_arrive_expect_tx(fb, 2 * kTileBytes);
        tma_load_4d(dst, &map_y, fb, 0, h, tok0, bidx);
        tma_load_4d(dst + kBoxBytes, &map_y, fb, 64, h, tok0, bidx);
        tma_load_4d(dst + kTileBytes, &map_z, fb, 0, h, tok0, bidx);
        tma_load_4d(dst + kTileBytes + kBoxBytes, &map_z, fb, 64, h, tok0, bidx);
        n_yz = it + 1;
      }
      sm->issued_ck = n_ck;
      sm->issued_yz = n_yz;
    }
    __syncwarp();
  } else if (warp == 9) {
    // ------------------------------------------------------------------ tensor-core issue
    if (lane == 0) {
      const uint32_t idesc = instr_desc(Fmt<T>::kAB, 1, 1, 128, 128);
      for (int it = 0; it < nc; ++it) {
        const int s = it % kStagesV;
        const uint32_t ph = (uint32_t)(it / kStagesV) & 1u;
        const uint32_t ys = base + kOffYZ + (uint32_t)s * 2 * kTileBytes, zs = ys + kTileBytes;
        const uint64_t d_y = desc_mnmajor(ys, kBoxBytes), d_z = desc_mnmajor(zs, kBoxBytes);
        mbar_wait(bar_y + 8 * s, ph, abort_flag, a.status, kStYV);
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          mma_ss(tmem, d_y + (uint64_t)(ks * 128), d_z + (uint64_t)(ks * 128), idesc, (it > 0 || ks > 0) ? 1u : 0u);
        mma_commit(empty_yz + 8 * s);
      }
      mma_commit(bar_done);
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ compute warps
    const int wg = warp >> 2, q4 = warp & 3;
    const int i = q4 * 32 + lane;  // row for the scaling phase
    float *segtot = reinterpret_cast<float *>(gbase + kOffSeg);
    float *run = reinterpret_cast<float *>(gbase + kOffRun);
    if (tid < kChunk) run[tid] = 0.f;
    named_bar_sync(1, kComputeV);
    for (int it = 0; it < nc; ++it) {
      const int n = back ? (nc - 1 - it) : it;
      const int s = it % kStagesV;
      const uint32_t ph = (uint32_t)(it / kStagesV) & 1u;
      const int sc = it % kStagesCk;
      const uint32_t phc = (uint32_t)(it / kStagesCk) & 1u;
      uint8_t *ck = gbase + kOffCk + sc * kCkBytes;
      const int L = min(kChunk, len - n * kChunk);
      mbar_wait(full_ck + 8 * sc, phc, abort_flag, a.status, kStFullV);
      {
        const int dg = tid & 31, seg = tid >> 5, d0 = dg * 4;
        const uint32_t colbase = (uint32_t)(d0 >> 5) * kBoxBytes;
        const uint32_t c4 = (uint32_t)((d0 & 31) >> 2);
        float4 acc16[16];
        float4 runv = make_float4(0.f, 0.f, 0.f, 0.f);
        // one instantiation per (16-bit input, activation); a 16-bit tile fills the first half of
        // the slot, the second sweep overwrites the whole slot after every thread has read
        auto sweep = [&](auto mode) {
          constexpr int kMode = decltype(mode)::value;
#pragma unroll
          for (int r = 0; r < 16; ++r) {
            const int row = seg * 16 + r;
            if (row < L) {
              const float4 v = decay_quad<T, (kMode & 2) != 0>(ck, row, d0, kBoxBytes);
              if (kMode & 1) {  // the tile holds pre-activations of a logsigmoid
                runv.x += log2_sigmoid(v.x); runv.y += log2_sigmoid(v.y);
                runv.z += log2_sigmoid(v.z); runv.w += log2_sigmoid(v.w);
              } else {
                runv.x = fmaf(v.x, kLog2e, runv.x); runv.y = fmaf(v.y, kLog2e, runv.y);
                runv.z = fmaf(v.z, kLog2e, runv.z); runv.w = fmaf(v.w, kLog2e, runv.w);
              }
            }
            acc16[r] = runv;
          }
        };
        switch ((a.ld16 ? 2 : 0) | (a.ld_act ? 1 : 0)) {
          case 0: sweep(std::integral_constant<int, 0>{}); break;
          case 1: sweep(std::integral_constant<int, 1>{}); break;
          case 2: sweep(std::integral_constant<int, 2>{}); break;
          default: sweep(std::integral_constant<int, 3>{}); break;
        }
        *reinterpret_cast<float4 *>(&segtot[seg * 128 + d0]) = runv;
        const float4 far = *reinterpret_cast<const float4 *>(&run[d0]);  // decay between this chunk and the far end
        named_bar_sync(1, kComputeV);
        float4 pre = make_float4(0.f, 0.f, 0.f, 0.f), acc = pre;
#pragma unroll
        for (int sgl = 0; sgl < 8; ++sgl) {
          if (sgl == seg) pre = acc;
          const float4 t = *reinterpret_cast<const float4 *>(&segtot[sgl * 128 + d0]);
          acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
        }
        const float4 g = acc;
        // exponent of the factor of (row, feature): forward flow far + g - c, reverse flow far + c
        const float4 sh = back ? make_float4(far.x + g.x - pre.x, far.y + g.y - pre.y, far.z + g.z - pre.z, far.w + g.w - pre.w)
                               : make_float4(far.x + pre.x, far.y + pre.y, far.z + pre.z, far.w + pre.w);
#pragma unroll
        for (int r = 0; r < 16; ++r) {
          const int row = seg * 16 + r;
          float4 v = acc16[r];
          if (back) { v.x = sh.x - v.x; v.y = sh.y - v.y; v.z = sh.z - v.z; v.w = sh.w - v.w; }
          else { v.x += sh.x; v.y += sh.y; v.z += sh.z; v.w += sh.w; }
          *reinterpret_cast<float4 *>(ck + colbase + (uint32_t)row * 128u + ((c4 ^ (uint32_t)(r & 7)) << 4)) = v;
        }
        if (seg == 0)
          *reinterpret_cast<float4 *>(&run[d0]) = make_float4(far.x + g.x, far.y + g.y, far.z + g.z, far.w + g.w);
        named_bar_sync(1, kComputeV);
      }
      // ---- Y <- Y (.) 2^exponent (this thread's row, this warpgroup's 64 features)
      mbar_wait(full_yz + 8 * s, ph, abort_flag, a.status, kStFullV);
      uint8_t *ytile = gbase + kOffYZ + (size_t)s * 2 * kTileBytes;
#pragma unroll 2
      for (int pc = 0; pc < 8; ++pc) {
        const int d0 = wg * 64 + pc * 8;
        const float4 c0 = *reinterpret_cast<const float4 *>(ck + ck_off(i, d0));
        const float4 c1 = *reinterpret_cast<const float4 *>(ck + ck_off(i, d0 + 4));
        const float2 f01 = make_float2(ex2(c0.x), ex2(c0.y)), f23 = make_float2(ex2(c0.z), ex2(c0.w));
        const float2 f45 = make_float2(ex2(c1.x), ex2(c1.y)), f67 = make_float2(ex2(c1.z), ex2(c1.w));
        uint4 *py = reinterpret_cast<uint4 *>(ytile + wg * kBoxBytes + sw128_offset(i, pc));
        const uint4 y = *py;
        uint4 o;
        float2 p;
        p = mul2(Fmt<T>::unpack(y.x), f01); o.x = Fmt<T>::pack(p.x, p.y);
        p = mul2(Fmt<T>::unpack(y.y), f23); o.y = Fmt<T>::pack(p.x, p.y);
        p = mul2(Fmt<T>::unpack(y.z), f45); o.z = Fmt<T>::pack(p.x, p.y);
        p = mul2(Fmt<T>::unpack(y.w), f67); o.w = Fmt<T>::pack(p.x, p.y);
        *py = i < L ? o : make_uint4(0u, 0u, 0u, 0u);
      }
      fence_proxy_async();
      mbar_arrive(bar_y + 8 * s);
      mbar_arrive(empty_ck + 8 * sc);
    }
    // the state -> global memory; this warpgroup's 64 columns of row i
    if (nc > 0) mbar_wait(bar_done, 0, abort_flag, a.status, kStDoneV);
    tc_fence_after();
    float *dst = a.states + ((long long)seq * a.H + h) * (long long)(kChunk * kChunk) + (long long)i * kChunk;
    const uint32_t tl = tmem + ((uint32_t)(32 * q4) << 16);
    for (int b2 = 0; b2 < 2; ++b2) {
      const int bt = 2 * wg + b2;
      uint32_t r[32];
      if (nc > 0) {
        tmem_ld32(tl + bt * 32, r);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int k = 0; k < 32; ++k) r[k] = 0u;
      }
      float4 *row = reinterpret_cast<float4 *>(dst + bt * 32);
#pragma unroll
      for (int k = 0; k < 8; ++k)
        row[k] = make_float4(__uint_as_float(r[4 * k]), __uint_as_float(r[4 * k + 1]), __uint_as_float(r[4 * k + 2]),
                             __uint_as_float(r[4 * k + 3]));
    }
    if (tid < kChunk && a.gsum != nullptr)
      a.gsum[((long long)seq * a.H + h) * kChunk + tid] = run[tid] * (1.f / kLog2e);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 8) {
    if (lane == 0 && sm->abort_flag != 0) {
      int dummy = 0;
      for (int it = max(0, sm->issued_ck - kStagesCk); it < sm->issued_ck; ++it)
        mbar_wait(full_ck + 8 * (it % kStagesCk), (uint32_t)(it / kStagesCk) & 1u, &dummy, nullptr, 0, 1u << 20);
      for (int it = max(0, sm->issued_yz - kStagesV); it < sm->issued_yz; ++it)
        mbar_wait(full_yz + 8 * (it % kStagesV), (uint32_t)(it / kStagesV) & 1u, &dummy, nullptr, 0, 1u << 20);
    }
    __syncwarp();
    tmem_dealloc(tmem, 128);
  }
}

template <typename T>
int launch_vec_t(const StatePass &p, int dtype, cudaStream_t stream) {
  alignas(64) CUtensorMap my, mz, ml;
  int rc;
  if ((rc = make_map(&my, p.y, dtype, p.B, p.N, p.H)) != LA_OK) return rc;
  if ((rc = make_map(&mz, p.z, dtype, p.B, p.N, p.H)) != LA_OK) return rc;
  if ((rc = make_map(&ml, p.ldv, p.ld16 ? dtype : LA_F32, p.B, p.N, p.H)) != LA_OK) return rc;
  if (reinterpret_cast<uintptr_t>(p.states) & 15u) return LA_ERR_MISALIGNED;
  vec::StateVecArgs a;
  a.cu = reinterpret_cast<const long long *>(p.cu);
  a.states = p.states; a.gsum = p.gsum;
  a.B = p.B; a.N = p.N; a.H = p.H; a.M = p.M; a.reverse = p.reverse; a.ranges = p.ranges;
  a.ld_act = p.ld_act;
  a.ld16 = p.ld16;
  a.status = status_word_ptr();
  if (a.status == nullptr) return LA_ERR_CUDA;
  auto kern = state_pass_vec_kernel<T>;
  const cudaError_t ea = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, vec::kSmemBytesV);
  if (ea != cudaSuccess) {
    note_cuda_error(ea, "cudaFuncSetAttribute(state_pass_vec_kernel)");
    return LA_ERR_CUDA;
  }
  const long long nb = p.cu ? p.M : p.B;
  kern<<<(unsigned)(nb * p.H), vec::kThreadsV, vec::kSmemBytesV, stream>>>(my, mz, ml, a);
  return launch_status();
}

// Fold with a per-feature decay on the state's rows: s = local + e^{gsum[d]} (.) s, state (D, E).
__global__ void fold_states_vec_kernel(const float *__restrict__ local, const float *__restrict__ gsum,
                                       const int *__restrict__ seg, const int *__restrict__ emit,
                                       const float *__restrict__ ext, float *__restrict__ out, int nseg, int H, int D,
                                       int E, int reverse) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long hde = (long long)H * D * E;
  if (idx >= hde) return;
  const int h = (int)(idx / ((long long)D * E));
  const int d = (int)((idx / E) % D);
  float s = 0.f;
  for (int kk = 0; kk < nseg; ++kk) {
    const int k = reverse ? nseg - 1 - kk : kk;
    const bool fresh = seg[4 * k + (reverse ? 2 : 1)] != 0;
    if (fresh) s = ext != nullptr ? ext[(long long)seg[4 * k] * hde + idx] : 0.f;
    const int slot = emit != nullptr ? emit[k] : k;
    if (slot >= 0) out[slot * hde + idx] = s;
    const int li = seg[4 * k + 3];
    s = li >= 0 ? local[li * hde + idx] + expf(gsum[((long long)li * H + h) * D + d]) * s : 0.f;
  }
}

}  // namespace

int launch_state_pass_vec(const StatePass &p, int dtype, cudaStream_t stream) {
  if (p.y == nullptr || p.z == nullptr || p.ldv == nullptr || p.states == nullptr) return LA_ERR_NULL_POINTER;
  const long long nb = p.cu ? p.M : p.B;
  if (nb <= 0 || p.H <= 0 || p.N <= 0) return LA_ERR_BAD_SHAPE;
  if (nb * p.H > 0x7fffffffLL) return LA_ERR_TOO_LARGE;
  if (dtype == LA_BF16) return launch_vec_t<__nv_bfloat16>(p, dtype, stream);
  if (dtype == LA_F16) return launch_vec_t<__half>(p, dtype, stream);
  return LA_ERR_UNSUPPORTED;
}

int launch_fold_states_vec(const float *local, const float *gsum, const int *seg, const int *emit, const float *ext,
                           float *out, int nseg, int H, int D, int E, int reverse, cudaStream_t st) {
  const long long hde = (long long)H * D * E;
  const int threads = 256;
  fold_states_vec_kernel<<<(unsigned)((hde + threads - 1) / threads), threads, 0, st>>>(local, gsum, seg, emit, ext,
                                                                                       out, nseg, H, D, E, reverse);
  return launch_status();
}

}  // namespace la
