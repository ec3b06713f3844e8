// Correction pass of the sequence-parallel scalar-decay forward.
//
// A rank that starts in the middle of a document first runs the ordinary varlen forward with a
// zero incoming state.  Once the true incoming state S_in (H, D, E) of that document is known
// (folded from the preceding ranks' chunk-end states), every token t of the document's local part
// is missing the term
//
//     o_t += exp(cum_t) * q_t^T S_in ,   cum_t = sum of ld from the rank's first token to t.
//
// This file adds that term in place.  D = E = 128 with 16-bit tensors runs on tcgen05 (one
// 128-token tile of q per CTA via TMA, S_in as a 16-bit MN-major operand); anything else runs a
// plain fp32 kernel.
#include <cuda.h>

#include "chunk.cuh"
#include "sm100_ptx.cuh"
#include "tile_common.cuh"

namespace la {
namespace {

using namespace ptx;
using namespace tile;

// ------------------------------------------------------------------------------------------------
// generic fp32 path: one thread per (token, head, e)
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void seqpar_correct_generic(const T *__restrict__ q, T *o, const float *__restrict__ cum,
                                       const float *__restrict__ s_in, int T1, int H, int D, int E) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long total = (long long)T1 * H * E;
  if (idx >= total) return;
  const int e = (int)(idx % E);
  const int h = (int)((idx / E) % H);
  const long long t = idx / ((long long)E * H);
  const T *qr = q + (t * H + h) * (long long)D;
  const float *s = s_in + (long long)h * D * E + e;
  float acc = 0.f;
  for (int d = 0; d < D; ++d) acc = fmaf(Cvt<T>::to_f(qr[d]), s[(long long)d * E], acc);
  const float w = expf(cum[t * H + h]);
  o[idx] = Cvt<T>::from_f(Cvt<T>::to_f(o[idx]) + w * acc);
}

// ------------------------------------------------------------------------------------------------
// tensor-core path
// ------------------------------------------------------------------------------------------------
constexpr int kTile = 32768, kBox = 16384;

struct SmallC {
  unsigned long long full, done;
  uint32_t tmem_base;
  int abort_flag;
};

// grid (tiles, H); 128 threads.  q is (1, N, H, 128).  Without a segment table tokens [0, T1) are
// corrected with one S_in and cum[t]; with a table (nseg rows of {start, length, first tile,
// flag}) segment s covers tokens [start, start + length), uses s_in[s] and the weight
// exp(cum[t] - cum[start - 1]), cum being the inclusive cumulative log decay of the whole stream.
template <typename T>
__global__ void __launch_bounds__(128, 1)
seqpar_correct_tc(const __grid_constant__ CUtensorMap map_q, T *o, const float *__restrict__ cum,
                  const float *__restrict__ s_in, int T1, int H, const int *__restrict__ seg, int nseg,
                  int *status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t *gbase = smem_raw + (base - raw);
  SmallC *sm = reinterpret_cast<SmallC *>(gbase + 2 * kTile);
  const int tid = threadIdx.x, warp = tid >> 5;
  const int h = blockIdx.y;
  int tile = blockIdx.x, start = 0, slen = T1;
  if (seg != nullptr) {
    int sidx = 0;
    while (sidx + 1 < nseg && tile >= seg[4 * (sidx + 1) + 2]) ++sidx;
    start = seg[4 * sidx];
    slen = seg[4 * sidx + 1];
    tile -= seg[4 * sidx + 2];
    s_in += (long long)sidx * H * 128 * 128;
  }
  const int tok0 = start + tile * 128;
  const uint32_t bar_full = smem_u32(&sm->full), bar_done = smem_u32(&sm->done);
  volatile int *abort_flag = &sm->abort_flag;
  if (tid == 0) {
    mbar_init(bar_full, 1);
    mbar_init(bar_done, 1);
    sm->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(&sm->tmem_base), 128);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm->tmem_base;
  const uint32_t qs = base, ss = base + kTile;
  if (tid == 0) {
    mbar_arrive_expect_tx(bar_full, kTile);
    tma_load_4d(qs, &map_q, bar_full, 0, h, tok0, 0);
    tma_load_4d(qs + kBox, &map_q, bar_full, 64, h, tok0, 0);
  }
  // S_in[h] row d (= tid) -> 16-bit, MN-major swizzled tile [d][e]
  {
    const float4 *src = reinterpret_cast<const float4 *>(s_in + ((long long)h * 128 + tid) * 128);
#pragma unroll 4
    for (int pc = 0; pc < 16; ++pc) {
      const float4 a = src[pc * 2], b = src[pc * 2 + 1];
      uint4 v;
      v.x = Fmt<T>::pack(a.x, a.y); v.y = Fmt<T>::pack(a.z, a.w);
      v.z = Fmt<T>::pack(b.x, b.y); v.w = Fmt<T>::pack(b.z, b.w);
      *reinterpret_cast<uint4 *>(gbase + kTile + (pc >> 3) * kBox + sw128_offset(tid, pc & 7)) = v;
    }
  }
  fence_proxy_async();
  mbar_wait(bar_full, 0, abort_flag, status, 201);
  tc_fence_before();
  __syncthreads();
  if (tid == 0) {
    tc_fence_after();
    const uint32_t idesc = instr_desc(Fmt<T>::kAB, 0, 1, 128, 128);
#pragma unroll
    for (int ks = 0; ks < 8; ++ks)
      mma_ss(tmem, desc_kmajor(qs + (uint32_t)(ks >> 2) * kBox + (uint32_t)(ks & 3) * 32u),
             desc_mnmajor(ss + ks * 2048, kBox), idesc, ks > 0);
    mma_commit(bar_done);
  }
  mbar_wait(bar_done, 0, abort_flag, status, 202);
  tc_fence_after();
  const int t = tok0 + tid;
  const bool valid = tile * 128 + tid < slen;
  const uint32_t tl = tmem + ((uint32_t)(32 * warp) << 16);
  float w = 0.f;
  if (valid) {
    const float c0 = start > 0 ? cum[(long long)(start - 1) * H + h] : 0.f;
    w = expf(cum[(long long)t * H + h] - c0);
  }
  T *orow = o + ((long long)t * H + h) * 128;
  for (int bt = 0; bt < 4; ++bt) {
    uint32_t r[32];
    tmem_ld32(tl + bt * 32, r);
    tmem_wait_ld();
    if (valid) {
      uint4 *op = reinterpret_cast<uint4 *>(orow + bt * 32);
#pragma unroll
      for (int pc = 0; pc < 4; ++pc) {
        uint4 v = op[pc];
        float2 f;
        f = Fmt<T>::unpack(v.x); v.x = Fmt<T>::pack(fmaf(w, __uint_as_float(r[pc * 8 + 0]), f.x), fmaf(w, __uint_as_float(r[pc * 8 + 1]), f.y));
        f = Fmt<T>::unpack(v.y); v.y = Fmt<T>::pack(fmaf(w, __uint_as_float(r[pc * 8 + 2]), f.x), fmaf(w, __uint_as_float(r[pc * 8 + 3]), f.y));
        f = Fmt<T>::unpack(v.z); v.z = Fmt<T>::pack(fmaf(w, __uint_as_float(r[pc * 8 + 4]), f.x), fmaf(w, __uint_as_float(r[pc * 8 + 5]), f.y));
        f = Fmt<T>::unpack(v.w); v.w = Fmt<T>::pack(fmaf(w, __uint_as_float(r[pc * 8 + 6]), f.x), fmaf(w, __uint_as_float(r[pc * 8 + 7]), f.y));
        op[pc] = v;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 128);
}

template <typename T>
int launch_tc(const void *q, void *o, const float *cum, const float *s_in, int T1, int N, int H, int dtype,
              cudaStream_t st, const int *seg = nullptr, int nseg = 0, int total_tiles = 0) {
  alignas(64) CUtensorMap mq;
  int rc = make_map(&mq, q, dtype, 1, N, H);  // (1, N, H, 128) 16-bit, boxes of 128 tokens x 64 features
  if (rc != LA_OK) return rc;
  if ((reinterpret_cast<uintptr_t>(o) | reinterpret_cast<uintptr_t>(s_in)) & 15u) return LA_ERR_MISALIGNED;
  int *status = status_word_ptr();
  if (status == nullptr) return LA_ERR_CUDA;
  const int smem = 2 * kTile + 64 + 1024;
  auto kern = seqpar_correct_tc<T>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return LA_ERR_CUDA;
  dim3 grid(seg != nullptr ? total_tiles : (T1 + 127) / 128, H);
  kern<<<grid, 128, smem, st>>>(mq, static_cast<T *>(o), cum, s_in, T1, H, seg, nseg, status);
  return launch_status();
}

template <typename T>
int launch_generic(const void *q, void *o, const float *cum, const float *s_in, int T1, int H, int D, int E,
                   cudaStream_t st) {
  const long long total = (long long)T1 * H * E;
  const int threads = 256;
  const long long blocks = (total + threads - 1) / threads;
  if (blocks > 0x7fffffffLL) return LA_ERR_TOO_LARGE;
  seqpar_correct_generic<T><<<(unsigned)blocks, threads, 0, st>>>(static_cast<const T *>(q), static_cast<T *>(o),
                                                                  cum, s_in, T1, H, D, E);
  return launch_status();
}

// S_in of `rank` from the gathered per-rank summaries [S_loc (HDE) | G (H) | open_end | spans]:
//   S_in(r+1) = open_end(r) * (S_loc(r) + spans(r) * exp(G(r)) * S_in(r)),  S_in(0) = 0.
__global__ void seqpar_fold_kernel(const float *__restrict__ gathered, float *__restrict__ s_in, int rank, int H,
                                   int DE) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long hde = (long long)H * DE;
  if (idx >= hde) return;
  const int h = (int)(idx / DE);
  const long long row = hde + H + 2;
  float s = 0.f;
  for (int r = 0; r < rank; ++r) {
    const float *g = gathered + r * row;
    s = g[hde + H] * (g[idx] + g[hde + H + 1] * expf(g[hde + h]) * s);
  }
  s_in[idx] = s;
}

}  // namespace

// Stitch consecutive segments of the same document, all run with a zero incoming state:
//   s_in(k) = 0 if segment k starts a document, else the true end state of segment k-1;
//   states(k) <- states(k) + exp(G(k)) s_in(k)        (its true end state).
// seg rows are {start, length, first tile, starts-a-document}.
__global__ void seqpar_fold_segments_kernel(float *__restrict__ states, const float *__restrict__ G,
                                            const int *__restrict__ seg, float *__restrict__ s_in, int nseg, int H,
                                            int DE) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long hde = (long long)H * DE;
  if (idx >= hde) return;
  const int h = (int)(idx / DE);
  float s = 0.f;
  for (int k = 0; k < nseg; ++k) {
    if (seg[4 * k + 3] != 0) s = 0.f;
    s_in[k * hde + idx] = s;
    s = states[k * hde + idx] + expf(G[(long long)k * H + h]) * s;
    states[k * hde + idx] = s;
  }
}

int launch_seqpar_fold_segments(float *states, const float *G, const int *seg, float *s_in, int nseg, int H, int DE,
                                cudaStream_t st) {
  const long long hde = (long long)H * DE;
  const int threads = 256;
  seqpar_fold_segments_kernel<<<(unsigned)((hde + threads - 1) / threads), threads, 0, st>>>(states, G, seg, s_in,
                                                                                            nseg, H, DE);
  return launch_status();
}

int launch_seqpar_correct_multi(const void *q, void *o, const float *cum, const float *s_in, const int *seg,
                                int nseg, int total_tiles, int N, int H, int dtype, cudaStream_t st) {
  if (nseg <= 0 || total_tiles <= 0) return LA_OK;
  if (dtype == LA_BF16) return launch_tc<__nv_bfloat16>(q, o, cum, s_in, 0, N, H, dtype, st, seg, nseg, total_tiles);
  if (dtype == LA_F16) return launch_tc<__half>(q, o, cum, s_in, 0, N, H, dtype, st, seg, nseg, total_tiles);
  return LA_ERR_UNSUPPORTED;
}

int launch_seqpar_fold(const float *gathered, float *s_in, int rank, int H, int DE, cudaStream_t st) {
  const long long hde = (long long)H * DE;
  const int threads = 256;
  seqpar_fold_kernel<<<(unsigned)((hde + threads - 1) / threads), threads, 0, st>>>(gathered, s_in, rank, H, DE);
  return launch_status();
}

int launch_seqpar_correct(const void *q, void *o, const float *cum, const float *s_in, int T1, int N, int H,
                          int D, int E, int dtype, cudaStream_t st) {
  if (T1 <= 0) return LA_OK;
  if (D == 128 && E == 128 && N >= 128 && (dtype == LA_BF16 || dtype == LA_F16)) {
    return dtype == LA_BF16 ? launch_tc<__nv_bfloat16>(q, o, cum, s_in, T1, N, H, dtype, st)
                            : launch_tc<__half>(q, o, cum, s_in, T1, N, H, dtype, st);
  }
  switch (dtype) {
    case LA_F32: return launch_generic<float>(q, o, cum, s_in, T1, H, D, E, st);
    case LA_BF16: return launch_generic<__nv_bfloat16>(q, o, cum, s_in, T1, H, D, E, st);
    case LA_F16: return launch_generic<__half>(q, o, cum, s_in, T1, H, D, E, st);
  }
  return LA_ERR_UNSUPPORTED;
}

}  // namespace la
