// Chunk-parallel vector-decay (key-side decay ldk) pass on 5th-generation tensor cores (sm_100a).
//
// Per (sequence, head) and 128-token chunk, with ck[i][d] the in-chunk inclusive cumulative log
// decay of feature d, m[d] = ck at the middle row, g[d] = ck at the last row:
//
//   o  pass (X,Y,Z = q,k,v):   W = tril(Xs Ys^T) Z + Xs (diag(e^m) T) ;  T <- diag(e^g) T + (Ys e^{g-m})^T Z
//        with Xs = X (.) e^{ck-m},  Ys = Y (.) e^{m-ck}   ("N" mode: the decay sits on the contraction
//        dimension of X Y^T; the reverse-direction twin with (k,q,do) gives dv)
//   dq pass (X,Y,Z = do,v,k):  W = [tril(X Y^T) Zs + X (T diag(e^m))] (.) e^{ck-m} ; T <- T diag(e^g) + Y^T (Zs e^{g-m})
//        with Zs = Z (.) e^{m-ck}, T = S^T                ("T" mode: the decay sits on the output
//        dimension; the reverse twin with (v,do,q) gives dk)
//
// Referencing the exponentials to the middle of the chunk keeps every factor within
// e^{+-(half-chunk decay)}; masked-out products may overflow to inf and are removed by a select.
// A chunk whose half-chunk decay exceeds 2^64 (bf16; 2^10 for fp16) raises the "unsafe" flag; the caller then reruns
// the call on the fp32 scan kernels (predicated on that flag, no host round trip).
//
// Two references per chunk (REF2 instantiations).  With decays like logsigmoid(N(0,1)) half a
// chunk decays by ~2^-74, too much for one reference.  The REF2 kernels reference rows 0..63 to
// r1 = ck[31] and rows 64..127 to r3 = ck[95], so that every factor is within 2^(+-decay of 32
// rows); a pair (later row i, earlier row j) uses r1 when j < 64 and r3 when j >= 64 -- in every
// pass, so that the rounded operands of the dq and dk passes still agree term by term:
//   N mode, forward   X' = X e^{ck-r1} (all rows), Y' = Y e^{r3-ck} (all rows), and a third tile R
//                     with rows 0..63 = Y e^{r1-ck}, rows 64..127 = X e^{ck-r3};
//                     P[:, 0:64] = X' R[0:64]^T,  P[:, 64:128] = R Y'[64:128]^T  (rows 0..63 of the
//                     second product are dead under the causal mask);  W = tril(P) Z + X' (e^{r1} T),
//                     T <- e^{r3} T + Y'^T Z with e^{g-r3} owed.  The reverse twin mirrors it.
//   T mode, forward   Z' = Z e^{r(j)-ck_j} in place, Wa = P~[:, 0:64] Z'[0:64] + X (T e^{r1}) scaled
//                     by e^{ck_i-r1} on output, Wb = P~[:, 64:128] Z'[64:128] scaled by e^{ck_i-r3};
//                     the state update reads rows 0..63 of Z e^{r3-ck} from a spare tile.
//   T mode, reverse   Wa = P~[:, 0:64] Z'[0:64] + P~[:, 64:128] (Z e^{ck-r1})[64:128] for rows 0..63,
//                     Wb = P~bot[:, 64:128] Z'[64:128] + X (T e^{g-r3}), P~bot = P~ with rows 0..63
//                     zeroed (a second 16-bit copy in the unused half of each batch of P).
// The caller runs the one-reference kernels first; the REF2 kernels run only if those raised their
// flag, and the scan kernels only if a 32-row quarter decays by more than 2^-96 (bf16).
//
// The factor e^{g-m} of the state update is not multiplied into the operand: it is owed to the
// state (kept as T~ with T = T~ scaled per feature by the owed factor) and paid at the start of the
// next chunk together with that chunk's own factor, so one scaled value serves both as the 16-bit
// copy and as the state the update adds to.
//
// Structure as in chunk_sm100.cu (state resident in tensor memory, TMA producer / MMA issuer /
// TMA store warps, bounded mbarrier waits, no multicast), but single-stage: the chunk's operands
// are three 16-bit tiles plus the 64 KB fp32 decay tile, and one more tile holds the 16-bit state
// copy (and, before it is written, the segment totals of the cumulative sum).  In T mode Z lives in
// a further tile of its own and is loaded together with the next decay tile.  The stage goes back to the
// producer piece by piece (decay tile, Y and Z, X), each when its last reader is done, and the
// next chunk is pulled into L2 meanwhile, so that most of the load latency hides behind the rest
// of the current chunk.
#include <cuda.h>

#include <cstddef>

#include "chunk.cuh"
#include "sm100_ptx.cuh"
#include "tile_common.cuh"

namespace la {
namespace {

using namespace ptx;
using namespace tile;

constexpr int kChunk = 128;
constexpr int kTileBytes = 32768, kBoxBytes = 16384;
constexpr int kOffX = 0, kOffY = kTileBytes, kOffZ = 2 * kTileBytes, kOffCk = 3 * kTileBytes;
constexpr int kCkBytes = 65536;
constexpr int kOffTb = kOffCk + kCkBytes, kOffU = kOffTb + kTileBytes, kOffSmall = kOffU + kTileBytes;
constexpr int kSmallBytes = 3072;
// All of the 227 KB a CTA may have: the dynamic shared memory is declared 1024-byte aligned (the
// 128-byte swizzle needs that) and the kernel checks it, so there is no slack for rounding up.
constexpr int kSmemBytes = kOffSmall + kSmallBytes;
constexpr int kStAlign = 313;
constexpr int kComputeThreads = 256;
constexpr int kProducerWarp = 8, kMmaWarp = 9, kStoreWarp = 10;
constexpr int kThreads = kComputeThreads + 96;
constexpr float kLog2e = 1.4426950408889634f;
// Largest half-chunk decay, in bits, the mid-chunk reference handles: operands are scaled by up to
// 2^(+-bits) before they are rounded to 16 bit, so the element type's exponent range decides.
template <typename T> struct SafeBits;
template <> struct SafeBits<__nv_bfloat16> { static constexpr float value = 64.f; };
template <> struct SafeBits<__half> { static constexpr float value = 10.f; };
// the same per 32-row quarter for the two-reference kernels
template <typename T> struct SafeBits2;
template <> struct SafeBits2<__nv_bfloat16> { static constexpr float value = 96.f; };
template <> struct SafeBits2<__half> { static constexpr float value = 10.f; };

constexpr uint32_t kColT = 0, kColP = 128, kColW1 = 256, kColW2 = 384;
constexpr int kStFull = 301, kStEmpty = 302, kStP = 303, kStW = 304, kStD = 305, kStF = 306, kStH = 307, kStR = 308,
              kStX = 309, kStL = 310;

struct Small {
  // The single stage is handed back to the producer in three pieces, each as soon as its last
  // reader is done.  N mode: the decay tile after the rescale, Y and Z after the chunk's
  // products, X (which stages the output tile) once that has been stored.  T mode needs the decay
  // tile until the epilogue (it scales by it and then stages the gradient terms in it), so there
  // the two 64 KB regions -- decay tile, Y and Z -- swap roles from chunk to chunk: when the
  // chunk's products are done the next chunk's decay tile is loaded where Y and Z were, and after
  // the store the next chunk's Y and Z go where the decay tile was.
  unsigned long long full_ck, full_yz, full_x, empty_ck, empty_yz, empty_x;
  unsigned long long bar_p, bar_w, bar_r, bar_d, bar_f, bar_h;
  // two references, T mode, log-decay gradient requested: the state copy goes to the tensor cores
  // as a high and a low half through the one copy tile, one after the other
  unsigned long long bar_x;  // X T with the high half complete (MMA warp -> compute)
  unsigned long long bar_l;  // low half written (compute -> MMA warp)
  uint32_t tmem_base;
  int abort_flag;
  int issued[3];  // chunks whose decay tile / Y and Z / X loads were issued
  // The resident state is kept as T~ with T = T~ (.) uvec (per feature: per row in N mode, per
  // column in T mode): instead of scaling the update operand by uvec before the product, the
  // factor is owed to the state and paid at the start of the next chunk, together with that
  // chunk's own factor (cf = cvec (.) previous uvec scales both the 16-bit copy and T~ itself,
  // because e^g / uvec = cvec in either direction), and once more when the end state is written.
  alignas(16) float uvec[kChunk];  // factor owed to the state after this chunk's update
  alignas(16) float cf[kChunk];    // cvec (.) the factor owed from the previous chunk
  // two-reference kernels only: the resident state and its 16-bit copy take different factors
  alignas(16) float bfv[kChunk];   // factor of the resident state (cf is the copy's)
  alignas(16) float dl[kChunk];    // r3 - r1 in log2 units (<= 0)
};
static_assert(sizeof(Small) <= kSmallBytes, "small area overflow");

struct LavdArgs {
  void *out;
  const void *xrow;   // T mode: tensor multiplied into the output for the log-decay gradient
  float *dld;         // T mode: (B,N,H,128) fp32 accumulator, stored (dld_sub = 0) or decremented
  int dld_sub;
  int dld_add;        // both passes add to a zeroed buffer (TMA reduce / atomics): order-free
  const float *t0;
  float *tfinal;
  int state_transposed, reverse;
  const long long *cu;
  int B, N, H, M;
  int *status;
  int *unsafe;
  const int *enable;  // optional device word: the kernel does nothing while it reads 0
  int ld_act;         // 1: the decay tensor holds pre-activations x and the log decay is logsigmoid(x)
  int ld16;           // 1: the decay tensor has the 16-bit type of x, y, z (half the bytes per chunk)
};

// byte offset of the float4 holding features [d, d+4) of row i in the 128B-swizzled fp32 decay tile
__device__ __forceinline__ uint32_t ck_off(int i, int d) {
  return (uint32_t)(d >> 5) * kBoxBytes + (uint32_t)i * 128u + (uint32_t)((((d & 31) >> 2) ^ (i & 7)) << 4);
}
__device__ __forceinline__ uint32_t kslice(int ks) { return (uint32_t)(ks >> 2) * kBoxBytes + (uint32_t)(ks & 3) * 32u; }

// 2^(+-ckc) for the 8 features starting at d0 of row i.
template <bool NEG>
__device__ __forceinline__ void decay_factors(const uint8_t *ck, int i, int d0, float (&f)[8]) {
  const float4 c0 = *reinterpret_cast<const float4 *>(ck + ck_off(i, d0));
  const float4 c1 = *reinterpret_cast<const float4 *>(ck + ck_off(i, d0 + 4));
  if (NEG) {
    f[0] = ex2(-c0.x); f[1] = ex2(-c0.y); f[2] = ex2(-c0.z); f[3] = ex2(-c0.w);
    f[4] = ex2(-c1.x); f[5] = ex2(-c1.y); f[6] = ex2(-c1.z); f[7] = ex2(-c1.w);
  } else {
    f[0] = ex2(c0.x); f[1] = ex2(c0.y); f[2] = ex2(c0.z); f[3] = ex2(c0.w);
    f[4] = ex2(c1.x); f[5] = ex2(c1.y); f[6] = ex2(c1.z); f[7] = ex2(c1.w);
  }
}
// One 16-byte piece (8 16-bit features) times the factors f.
template <typename T>
__device__ __forceinline__ uint4 scale8(uint4 v, const float (&f)[8], float2 (&prod)[4]) {
  uint4 o;
  prod[0] = mul2(Fmt<T>::unpack(v.x), make_float2(f[0], f[1])); o.x = Fmt<T>::pack(prod[0].x, prod[0].y);
  prod[1] = mul2(Fmt<T>::unpack(v.y), make_float2(f[2], f[3])); o.y = Fmt<T>::pack(prod[1].x, prod[1].y);
  prod[2] = mul2(Fmt<T>::unpack(v.z), make_float2(f[4], f[5])); o.z = Fmt<T>::pack(prod[2].x, prod[2].y);
  prod[3] = mul2(Fmt<T>::unpack(v.w), make_float2(f[6], f[7])); o.w = Fmt<T>::pack(prod[3].x, prod[3].y);
  return o;
}
template <typename T, bool NEG>
__device__ __forceinline__ void rescale_xy(uint8_t *gbase, const uint8_t *ck, int i, int wg, int L) {
  // X <- X 2^(+-ckc), Y <- Y 2^(-+ckc) for this thread's row and 64 columns; rows past the end of
  // the sequence become zero in Y so that they add nothing to the state
#pragma unroll 2
  for (int pc = 0; pc < 8; ++pc) {
    const int d0 = wg * 64 + pc * 8;
    const uint32_t off = wg * kBoxBytes + sw128_offset(i, pc);
    float fx[8], fy[8];
    decay_factors<NEG>(ck, i, d0, fx);
    decay_factors<!NEG>(ck, i, d0, fy);
    float2 prod[4];
    uint4 *px = reinterpret_cast<uint4 *>(gbase + kOffX + off);
    *px = scale8<T>(*px, fx, prod);
    uint4 *py = reinterpret_cast<uint4 *>(gbase + kOffY + off);
    const uint4 ys = scale8<T>(*py, fy, prod);
    *py = i < L ? ys : make_uint4(0u, 0u, 0u, 0u);
  }
}
template <typename T, bool NEG>
__device__ __forceinline__ void rescale_z(uint8_t *gbase, uint32_t zoff, const uint8_t *ck, int i, int wg, int L) {
#pragma unroll 2
  for (int pc = 0; pc < 8; ++pc) {
    const int d0 = wg * 64 + pc * 8;
    const uint32_t off = wg * kBoxBytes + sw128_offset(i, pc);
    float fz[8];
    decay_factors<NEG>(ck, i, d0, fz);
    float2 prod[4];
    uint4 *pz = reinterpret_cast<uint4 *>(gbase + zoff + off);
    const uint4 zs = scale8<T>(*pz, fz, prod);
    *pz = i < L ? zs : make_uint4(0u, 0u, 0u, 0u);
  }
}


// ---- two-reference rescales.  t = decay tile value of (row i, feature d): ck - r1 for rows 0..63,
// ck - r3 for rows 64..127; dl[d] = r3 - r1.  The mixed factor 2^((top ? -t : t) + dl) is formed
// with that exact expression everywhere it appears (rescale and epilogue), so that the operand one
// pass feeds to the tensor cores is bit-identical to the factor its twin applies on output.
__device__ __forceinline__ void tile_vals(const uint8_t *ck, const float *dl, int i, int d0, float (&t)[8],
                                          float (&d)[8]) {
  const float4 c0 = *reinterpret_cast<const float4 *>(ck + ck_off(i, d0));
  const float4 c1 = *reinterpret_cast<const float4 *>(ck + ck_off(i, d0 + 4));
  const float4 e0 = *reinterpret_cast<const float4 *>(dl + d0);
  const float4 e1 = *reinterpret_cast<const float4 *>(dl + d0 + 4);
  t[0] = c0.x; t[1] = c0.y; t[2] = c0.z; t[3] = c0.w; t[4] = c1.x; t[5] = c1.y; t[6] = c1.z; t[7] = c1.w;
  d[0] = e0.x; d[1] = e0.y; d[2] = e0.z; d[3] = e0.w; d[4] = e1.x; d[5] = e1.y; d[6] = e1.z; d[7] = e1.w;
}
// N mode: X and Y in place, and the third tile R (see the file header).
template <typename T, bool REV>
__device__ __forceinline__ void rescale2_xy(uint8_t *gbase, const uint8_t *ck, const float *dl, int i, int wg,
                                            int L) {
  const bool top = i < 64;  // warp-uniform
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll 1
  for (int pc = 0; pc < 8; ++pc) {
    const int d0 = wg * 64 + pc * 8;
    const uint32_t off = wg * kBoxBytes + sw128_offset(i, pc);
    float t[8], d[8], fp[8], fn[8], fm[8];
    tile_vals(ck, dl, i, d0, t, d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      fp[j] = ex2(t[j]);
      fn[j] = ex2(-t[j]);
      fm[j] = ex2((top ? -t[j] : t[j]) + d[j]);
    }
    float2 prod[4];
    uint4 *px = reinterpret_cast<uint4 *>(gbase + kOffX + off);
    uint4 *py = reinterpret_cast<uint4 *>(gbase + kOffY + off);
    uint4 *pr = reinterpret_cast<uint4 *>(gbase + kOffU + off);
    const uint4 x = *px, y = *py;
    const bool live = i < L;
    if (!REV) {
      if (top) {  // X' = X 2^t, Y' = Y 2^(-t+dl), R = Y 2^-t
        *px = scale8<T>(x, fp, prod);
        *py = live ? scale8<T>(y, fm, prod) : zero;
        *pr = live ? scale8<T>(y, fn, prod) : zero;
      } else {    // X' = X 2^(t+dl), Y' = Y 2^-t, R = X 2^t
        *px = scale8<T>(x, fm, prod);
        *py = live ? scale8<T>(y, fn, prod) : zero;
        *pr = scale8<T>(x, fp, prod);
      }
    } else {
      if (top) {  // X' = X 2^(-t+dl), Y' = Y 2^t, R = X 2^-t
        *px = scale8<T>(x, fm, prod);
        *py = live ? scale8<T>(y, fp, prod) : zero;
        *pr = scale8<T>(x, fn, prod);
      } else {    // X' = X 2^-t, Y' = Y 2^(t+dl), R = Y 2^t
        *px = scale8<T>(x, fn, prod);
        *py = live ? scale8<T>(y, fm, prod) : zero;
        *pr = live ? scale8<T>(y, fp, prod) : zero;
      }
    }
  }
}
// T mode: Z in place (forward: 2^-t, reverse: 2^t) and, in the spare tile at foff, the rows the
// state update (and the reverse pass's first accumulator) need against the other reference:
// forward rows 0..63 = Z 2^(-t+dl), reverse rows 64..127 = Z 2^(t+dl).
template <typename T, bool REV>
__device__ __forceinline__ void rescale2_z(uint8_t *gbase, uint32_t zoff, uint32_t foff, const uint8_t *ck,
                                           const float *dl, int i, int wg, int L) {
  const bool top = i < 64;
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll 1
  for (int pc = 0; pc < 8; ++pc) {
    const int d0 = wg * 64 + pc * 8;
    const uint32_t off = wg * kBoxBytes + sw128_offset(i, pc);
    float t[8], d[8], f1[8], f2[8];
    tile_vals(ck, dl, i, d0, t, d);
    const bool second = REV ? !top : top;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      f1[j] = ex2(REV ? t[j] : -t[j]);
      f2[j] = ex2((top ? -t[j] : t[j]) + d[j]);
    }
    float2 prod[4];
    uint4 *pz = reinterpret_cast<uint4 *>(gbase + zoff + off);
    const uint4 z = *pz;
    const bool live = i < L;
    *pz = live ? scale8<T>(z, f1, prod) : zero;
    if (second) *reinterpret_cast<uint4 *>(gbase + foff + off) = live ? scale8<T>(z, f2, prod) : zero;
  }
}

template <typename T, bool TMODE, bool REF2>
__global__ void __launch_bounds__(kThreads, 1)
lavd_pass_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_y,
                 const __grid_constant__ CUtensorMap map_z, const __grid_constant__ CUtensorMap map_ld,
                 const __grid_constant__ CUtensorMap map_o, const __grid_constant__ CUtensorMap map_dld,
                 const LavdArgs a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  if (a.enable != nullptr && *a.enable == 0) return;  // uniform over the grid
  const uint32_t base = smem_u32(smem_raw);
  uint8_t *gbase = smem_raw;
  Small *sm = reinterpret_cast<Small *>(gbase + kOffSmall);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (base & 1023u) {  // uniform over the CTA; nothing has been set up yet
    if (tid == 0) atomicCAS(a.status, 0, kStAlign);
    return;
  }
  const int seq = blockIdx.x / a.H, h = blockIdx.x - seq * a.H;
  long long t_begin = 0, t_end = a.N;
  int bidx = seq;
  if (a.cu != nullptr) {
    t_begin = a.cu[seq];
    t_end = a.cu[seq + 1];
    bidx = 0;
  }
  const int len = (int)(t_end - t_begin);
  const int nc = (len + kChunk - 1) / kChunk;
  const bool rev = a.reverse != 0;

  const uint32_t full_ck = smem_u32(&sm->full_ck), full_yz = smem_u32(&sm->full_yz), full_x = smem_u32(&sm->full_x);
  const uint32_t empty_ck = smem_u32(&sm->empty_ck), empty_yz = smem_u32(&sm->empty_yz), empty_x = smem_u32(&sm->empty_x);
  const uint32_t bar_p = smem_u32(&sm->bar_p), bar_w = smem_u32(&sm->bar_w), bar_r = smem_u32(&sm->bar_r);
  const uint32_t bar_d = smem_u32(&sm->bar_d), bar_f = smem_u32(&sm->bar_f), bar_h = smem_u32(&sm->bar_h);
  const uint32_t bar_x = smem_u32(&sm->bar_x), bar_l = smem_u32(&sm->bar_l);
  volatile int *abort_flag = &sm->abort_flag;

  if (tid == 0) {
    mbar_init(full_ck, 1);
    mbar_init(full_yz, 1);
    mbar_init(full_x, 1);
    mbar_init(empty_ck, TMODE ? 1 : kComputeThreads);
    mbar_init(empty_yz, 1);
    mbar_init(empty_x, 1);
    mbar_init(bar_p, 1);
    mbar_init(bar_w, 1);
    mbar_init(bar_r, kComputeThreads);
    mbar_init(bar_d, kComputeThreads);
    mbar_init(bar_f, kComputeThreads);
    mbar_init(bar_h, kComputeThreads);
    mbar_init(bar_x, 1);
    mbar_init(bar_l, kComputeThreads);
    sm->abort_flag = 0;
    sm->issued[0] = sm->issued[1] = sm->issued[2] = 0;
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
  const uint32_t xs = base + kOffX, ys = base + kOffY, zs = base + kOffZ, cks = base + kOffCk;
  const uint32_t tbs = base + kOffTb, zts = base + kOffU;  // zts: T mode's Z tile

  if (warp == kProducerWarp) {
    // ------------------------------------------------------------------ TMA loads (single stage)
    if (lane == 0) {
      int n_ck = 0, n_yz = 0, n_x = 0;
      auto load_ck = [&](int tok0, uint32_t par, uint32_t dst) {
        mbar_wait(empty_ck, par ^ 1u, abort_flag, a.status, kStEmpty);
        if (*abort_flag) return false;
        const int ck_bytes = a.ld16 ? kCkBytes / 2 : kCkBytes;
        mbar_arrive_expect_tx(full_ck, TMODE ? ck_bytes + kTileBytes : ck_bytes);
        if (a.ld16) {  // two boxes of 64 16-bit features into the first half of the slot
          tma_load_4d(dst, &map_ld, full_ck, 0, h, tok0, bidx);
          tma_load_4d(dst + kBoxBytes, &map_ld, full_ck, 64, h, tok0, bidx);
        } else {
#pragma unroll
          for (int gq = 0; gq < 4; ++gq) tma_load_4d(dst + gq * kBoxBytes, &map_ld, full_ck, 32 * gq, h, tok0, bidx);
        }
        if (TMODE) {
          // T mode keeps Z in a tile of its own (free like the decay slot once the previous
          // chunk's products are done), so the rescale of the next chunk never waits for the store
          tma_load_4d(zts, &map_z, full_ck, 0, h, tok0, bidx);
          tma_load_4d(zts + kBoxBytes, &map_z, full_ck, 64, h, tok0, bidx);
        }
        ++n_ck;
        return true;
      };
      for (int it = 0; it < nc; ++it) {
        const int n = rev ? (nc - 1 - it) : it;
        const uint32_t par = (uint32_t)it & 1u;
        const int tok0 = (int)t_begin + n * kChunk;
        const bool swap = TMODE && (it & 1);  // T mode: the two 64 KB regions swap roles every chunk
        const uint32_t ck_dst = swap ? ys : cks, y_dst = swap ? cks : ys, z_dst = y_dst + kTileBytes;
        // in the order in which the pieces come free
        if (!load_ck(tok0, par, ck_dst)) break;
        mbar_wait(empty_yz, par ^ 1u, abort_flag, a.status, kStEmpty);
        if (*abort_flag) break;
        mbar_arrive_expect_tx(full_yz, TMODE ? kTileBytes : 2 * kTileBytes);
        tma_load_4d(y_dst, &map_y, full_yz, 0, h, tok0, bidx);
        tma_load_4d(y_dst + kBoxBytes, &map_y, full_yz, 64, h, tok0, bidx);
        if (!TMODE) {
          tma_load_4d(z_dst, &map_z, full_yz, 0, h, tok0, bidx);
          tma_load_4d(z_dst + kBoxBytes, &map_z, full_yz, 64, h, tok0, bidx);
        }
        ++n_yz;
        mbar_wait(empty_x, par ^ 1u, abort_flag, a.status, kStEmpty);
        if (*abort_flag) break;
        mbar_arrive_expect_tx(full_x, kTileBytes);
        tma_load_4d(xs, &map_x, full_x, 0, h, tok0, bidx);
        tma_load_4d(xs + kBoxBytes, &map_x, full_x, 64, h, tok0, bidx);
        ++n_x;
        // The stage is single-buffered, so the next chunk's loads start only as its pieces come
        // free and the CTA then waits out their latency; pulling that chunk into L2 now shortens
        // the wait (the pass uses a fraction of the HBM bandwidth, so this costs nothing).
        if (it + 1 < nc) {
          const int tokp = (int)t_begin + (rev ? (n - 1) : (n + 1)) * kChunk;
          tma_prefetch_4d(&map_x, 0, h, tokp, bidx);
          tma_prefetch_4d(&map_x, 64, h, tokp, bidx);
          tma_prefetch_4d(&map_y, 0, h, tokp, bidx);
          tma_prefetch_4d(&map_y, 64, h, tokp, bidx);
          tma_prefetch_4d(&map_z, 0, h, tokp, bidx);
          tma_prefetch_4d(&map_z, 64, h, tokp, bidx);
          if (a.ld16) {
            tma_prefetch_4d(&map_ld, 0, h, tokp, bidx);
            tma_prefetch_4d(&map_ld, 64, h, tokp, bidx);
          } else {
#pragma unroll
            for (int gq = 0; gq < 4; ++gq) tma_prefetch_4d(&map_ld, 32 * gq, h, tokp, bidx);
          }
        }
      }
      sm->issued[0] = n_ck;
      sm->issued[1] = n_yz;
      sm->issued[2] = n_x;
    }
    __syncwarp();
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------------ tensor-core issue
    if (lane == 0) {
      const uint32_t idesc_kk = instr_desc(Fmt<T>::kAB, 0, 0, 128, 128);
      const uint32_t idesc_kk64 = instr_desc(Fmt<T>::kAB, 0, 0, 128, 64);
      const uint32_t idesc_kmn = instr_desc(Fmt<T>::kAB, 0, 1, 128, 128);
      const uint32_t idesc_mnmn = instr_desc(Fmt<T>::kAB, 1, 1, 128, 128);
      const uint64_t d_xk = desc_kmajor(xs), d_tb = desc_mnmajor(tbs, kBoxBytes);
      const uint64_t d_rk = desc_kmajor(zts);  // N mode, two references: the third tile R
      constexpr uint64_t kRow64 = (64 * 128) >> 4;  // rows 64..127 of a K-major tile, in descriptor units
      for (int it = 0; it < nc; ++it) {
        const uint32_t par = (uint32_t)it & 1u;
        const uint32_t y_at = (TMODE && (it & 1)) ? cks : ys, z_at = TMODE ? zts : y_at + kTileBytes;
        const uint64_t d_yk = desc_kmajor(y_at), d_ymn = desc_mnmajor(y_at, kBoxBytes);
        const uint64_t d_zmn = desc_mnmajor(z_at, kBoxBytes);
        const uint64_t d_fmn = desc_mnmajor(y_at + kTileBytes, kBoxBytes);  // T mode, two references: spare tile
        mbar_wait(full_x, par, abort_flag, a.status, kStFull);
        mbar_wait(full_yz, par, abort_flag, a.status, kStFull);
        // N mode multiplies the rescaled X and Y; T mode the tiles as loaded
        if (!TMODE) mbar_wait(bar_r, par, abort_flag, a.status, kStR);
        tc_fence_after();
        if (!TMODE && REF2) {
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            const uint64_t ko = (uint64_t)((ks >> 2) * (kBoxBytes >> 4) + (ks & 3) * 2);
            if (!rev) {  // P[:, 0:64] = X' R[0:64]^T ; P[:, 64:128] = R Y'[64:128]^T
              mma_ss(tmem + kColP, d_xk + ko, d_rk + ko, idesc_kk64, ks > 0);
              mma_ss(tmem + kColP + 64, d_rk + ko, d_yk + ko + kRow64, idesc_kk64, ks > 0);
            } else {     // P[:, 0:64] = R Y'[0:64]^T ; P[:, 64:128] = X' R[64:128]^T
              mma_ss(tmem + kColP, d_rk + ko, d_yk + ko, idesc_kk64, ks > 0);
              mma_ss(tmem + kColP + 64, d_xk + ko, d_rk + ko + kRow64, idesc_kk64, ks > 0);
            }
          }
        } else {
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            const uint64_t ko = (uint64_t)((ks >> 2) * (kBoxBytes >> 4) + (ks & 3) * 2);
            mma_ss(tmem + kColP, d_xk + ko, d_yk + ko, idesc_kk, ks > 0);
          }
        }
        mma_commit(bar_p);
        mbar_wait(bar_d, par, abort_flag, a.status, kStD);
        if (TMODE) mbar_wait(bar_r, par, abort_flag, a.status, kStR);
        tc_fence_after();
        // X * (scaled 16-bit state copy).  One reference: its own accumulator W2, added to W1 in the
        // epilogue.  T mode with two references: it shares the accumulator whose output scale it
        // has (forward: Wa = columns W1, reverse: Wb = columns W2).
        const uint32_t col_xt = (TMODE && REF2 && !rev) ? kColW1 : kColW2;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint64_t ko = (uint64_t)((ks >> 2) * (kBoxBytes >> 4) + (ks & 3) * 2);
          mma_ss(tmem + col_xt, d_xk + ko, d_tb + (uint64_t)(ks * 128), idesc_kmn, ks > 0);
        }
        if (TMODE && REF2 && a.dld != nullptr) {   // low half of the split state copy (same tile, in turn)
          mma_commit(bar_x);
          mbar_wait(bar_l, par, abort_flag, a.status, kStL);
          tc_fence_after();
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            const uint64_t ko = (uint64_t)((ks >> 2) * (kBoxBytes >> 4) + (ks & 3) * 2);
            mma_ss(tmem + col_xt, d_xk + ko, d_tb + (uint64_t)(ks * 128), idesc_kmn, 1);
          }
        }
        if (TMODE && !REF2 && a.dld != nullptr) {  // low half of the split state copy (spare tile)
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            const uint64_t ko = (uint64_t)((ks >> 2) * (kBoxBytes >> 4) + (ks & 3) * 2);
            mma_ss(tmem + col_xt, d_xk + ko, d_fmn + (uint64_t)(ks * 128), idesc_kmn, 1);
          }
        }
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {  // state update Y^T Z (N mode: Y rescaled; T mode: Z rescaled)
          uint64_t zb = d_zmn;
          if (TMODE && REF2 && ((ks < 4) != rev)) zb = d_fmn;  // rows against the other reference
          mma_ss(tmem + kColT, d_ymn + (uint64_t)(ks * 128), zb + (uint64_t)(ks * 128), idesc_mnmn, 1);
        }
        mbar_wait(bar_f, par, abort_flag, a.status, kStF);
        tc_fence_after();
        if (TMODE && REF2) {
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            const uint32_t pa = tmem + kColP + (ks >> 1) * 32 + (ks & 1) * 8;
            const uint64_t zk = d_zmn + (uint64_t)(ks * 128), fk = d_fmn + (uint64_t)(ks * 128);
            if (!rev) {
              // Wa += P~[:, 0:64] Z'[0:64] (on top of X T) ; Wb = P~[:, 64:128] Z'[64:128]
              if (ks < 4) mma_ts(tmem + kColW1, pa, zk, idesc_kmn, 1);
              else mma_ts(tmem + kColW2, pa, zk, idesc_kmn, ks > 4);
            } else {
              // Wa = P~[:, 0:64] Z'[0:64] + P~[:, 64:128] F[64:128] ; Wb += P~bot[:, 64:128] Z'[64:128]
              mma_ts(tmem + kColW1, pa, ks < 4 ? zk : fk, idesc_kmn, ks > 0);
              if (ks >= 4) mma_ts(tmem + kColW2, pa + 16, zk, idesc_kmn, 1);
            }
          }
        } else {
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)  // W1 = P~ Z (T mode: Z is the rescaled tile)
            mma_ts(tmem + kColW1, tmem + kColP + (ks >> 1) * 32 + (ks & 1) * 8, d_zmn + (uint64_t)(ks * 128),
                   idesc_kmn, ks > 0);
        }
        mma_commit(bar_w);
        // Y and Z have no reader left once the products above are done: in N mode they go back
        // to the producer for the next chunk's Y and Z, in T mode for its decay tile
        mma_commit(TMODE ? empty_ck : empty_yz);
        mbar_wait(bar_w, par, abort_flag, a.status, kStW);
      }
    }
    __syncwarp();
  } else if (warp == kStoreWarp) {
    // ------------------------------------------------------------------ TMA stores
    if (lane == 0) {
      for (int it = 0; it < nc; ++it) {
        const int n = rev ? (nc - 1 - it) : it;
        const uint32_t par = (uint32_t)it & 1u;
        const int L = min(kChunk, len - n * kChunk);
        mbar_wait(bar_h, par, abort_flag, a.status, kStH);
        if (L == kChunk) {
          const int tok0 = (int)t_begin + n * kChunk;
          tma_store_4d(&map_o, xs, 0, h, tok0, bidx);
          tma_store_4d(&map_o, xs + kBoxBytes, 64, h, tok0, bidx);
          if (TMODE && a.dld != nullptr) {
            // the decay tile now holds this chunk's log-decay-gradient terms: store (dq pass) or
            // add the (negated) terms as four fp32 boxes
            const uint32_t stg = (it & 1) ? ys : cks;
#pragma unroll
            for (int gq = 0; gq < 4; ++gq) {
              if (a.dld_sub || a.dld_add) tma_reduce_add_4d(&map_dld, stg + gq * kBoxBytes, 32 * gq, h, tok0, bidx);
              else tma_store_4d(&map_dld, stg + gq * kBoxBytes, 32 * gq, h, tok0, bidx);
            }
          }
          tma_store_commit();
          tma_store_wait_read();
        }
        mbar_arrive(empty_x);
        if (TMODE) mbar_arrive(empty_yz);
      }
      tma_store_wait_all();
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ compute warps
    const int wg = warp >> 2, q4 = warp & 3;
    const int i = q4 * 32 + lane;  // tile row / tensor-memory lane
    const uint32_t tl = tmem + ((uint32_t)(32 * q4) << 16);
    const long long st_base = ((long long)seq * a.H + h) * (long long)(kChunk * kChunk);
    uint8_t *ck = gbase + kOffCk;  // T mode: re-pointed every chunk
    // [8][128] segment totals of the cumulative sum, in the state-copy tile: the copy's last
    // reader (X T of the previous chunk) is done before the previous epilogue, and the next copy is
    // written after the cumulative sum
    float *segtot = reinterpret_cast<float *>(gbase + kOffTb);

    for (int b2 = 0; b2 < 2; ++b2) {  // starting state -> tensor memory
      const int bt = 2 * wg + b2;
      uint32_t r[32];
#pragma unroll
      for (int k = 0; k < 32; ++k) {
        const int c = bt * 32 + k;
        float v = 0.f;
        if (a.t0 != nullptr) v = a.t0[st_base + (a.state_transposed ? (c * kChunk + i) : (i * kChunk + c))];
        r[k] = __float_as_uint(v);
      }
      tmem_st32(tl + kColT + bt * 32, r);
    }
    tmem_wait_st();
    if (tid < kChunk) sm->uvec[tid] = 1.f;  // nothing is owed to the starting state

    for (int it = 0; it < nc; ++it) {
      const int n = rev ? (nc - 1 - it) : it;
      const uint32_t par = (uint32_t)it & 1u;
      const int L = min(kChunk, len - n * kChunk);
      const long long tok = t_begin + (long long)n * kChunk + i;

      const uint32_t z_off = TMODE ? kOffU : kOffZ;
      if (TMODE) ck = gbase + ((it & 1) ? kOffY : kOffCk);
      if (TMODE && a.dld != nullptr && i < L) {
        // the epilogue multiplies the output by this row of xrow, read from global memory: pull
        // it into L2 now (one 128-byte line per thread; L1 is too small beside 227 KB of shared
        // memory to hold it until then)
        const char *xr = reinterpret_cast<const char *>(static_cast<const T *>(a.xrow) +
                                                          ((bidx * (long long)a.N + tok) * a.H + h) * (long long)kChunk + wg * 64);
        asm volatile("prefetch.global.L2 [%0];" ::"l"(xr));
      }
      mbar_wait(full_ck, par, abort_flag, a.status, kStFull);

      // ---- S: per-feature inclusive cumulative log2 decay down the 128 rows, centred on row 63.
      // Thread (dg = tid % 32, seg = tid / 32) scans the four features [4 dg, 4 dg + 4) over the
      // sixteen rows of segment seg with 128-bit accesses; segment totals meet in shared memory.
      {
        const int dg = tid & 31, seg = tid >> 5, d0 = dg * 4;
        const uint32_t colbase = (uint32_t)(d0 >> 5) * kBoxBytes;
        const uint32_t c4 = (uint32_t)((d0 & 31) >> 2);
        // the sixteen running sums stay in registers between the two sweeps: one load and one
        // store per row and no read-back
        float4 acc16[16];
        float4 run = make_float4(0.f, 0.f, 0.f, 0.f);
        // first sweep, one instantiation per (16-bit input, activation): the plain fp32 path keeps
        // its two instructions per value.  A 16-bit tile fills the first half of the slot only; the
        // second sweep below overwrites the whole slot with fp32 sums after every thread has read.
        auto sweep = [&](auto mode) {
          constexpr int kMode = decltype(mode)::value;
#pragma unroll
          for (int r = 0; r < 16; ++r) {
            const int row = seg * 16 + r;  // row & 7 == r & 7
            if (row < L) {
              const float4 v = decay_quad<T, (kMode & 2) != 0>(ck, row, d0, kBoxBytes);
              if (kMode & 1) {  // the tile holds pre-activations of a logsigmoid
                run.x += log2_sigmoid(v.x); run.y += log2_sigmoid(v.y);
                run.z += log2_sigmoid(v.z); run.w += log2_sigmoid(v.w);
              } else {
                run.x = fmaf(v.x, kLog2e, run.x); run.y = fmaf(v.y, kLog2e, run.y);
                run.z = fmaf(v.z, kLog2e, run.z); run.w = fmaf(v.w, kLog2e, run.w);
              }
            }
            acc16[r] = run;
          }
        };
        switch ((a.ld16 ? 2 : 0) | (a.ld_act ? 1 : 0)) {
          case 0: sweep(std::integral_constant<int, 0>{}); break;
          case 1: sweep(std::integral_constant<int, 1>{}); break;
          case 2: sweep(std::integral_constant<int, 2>{}); break;
          default: sweep(std::integral_constant<int, 3>{}); break;
        }
        *reinterpret_cast<float4 *>(&segtot[seg * 128 + d0]) = run;
        named_bar_sync(1, kComputeThreads);
        float4 pre = make_float4(0.f, 0.f, 0.f, 0.f), m = pre, acc = pre, r1 = pre, r3 = pre;
#pragma unroll
        for (int sgl = 0; sgl < 8; ++sgl) {
          if (sgl == seg) pre = acc;
          if (sgl == 2) r1 = acc;
          if (sgl == 4) m = acc;
          if (sgl == 6) r3 = acc;
          const float4 t = *reinterpret_cast<const float4 *>(&segtot[sgl * 128 + d0]);
          acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
        }
        const float4 g = acc;  // r1, m, r3, g: ck at rows 31, 63, 95, 127
        // the tile is centred on row 63, or (two references) its halves on rows 31 and 95
        const float4 ref = REF2 ? (seg < 4 ? r1 : r3) : m;
        const float4 sh = make_float4(pre.x - ref.x, pre.y - ref.y, pre.z - ref.z, pre.w - ref.w);
#pragma unroll
        for (int r = 0; r < 16; ++r) {
          const int row = seg * 16 + r;
          float4 v = acc16[r];
          v.x += sh.x; v.y += sh.y; v.z += sh.z; v.w += sh.w;
          *reinterpret_cast<float4 *>(ck + colbase + (uint32_t)row * 128u + ((c4 ^ (uint32_t)(r & 7)) << 4)) = v;
        }
        if (seg == 0) {
          const float mm[4] = {m.x, m.y, m.z, m.w}, gg[4] = {g.x, g.y, g.z, g.w};
          const float q1[4] = {r1.x, r1.y, r1.z, r1.w}, q3[4] = {r3.x, r3.y, r3.z, r3.w};
          bool bad = false;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const float u_old = sm->uvec[d0 + c];  // still the previous chunk's
            if (!REF2) {
              const float u_new = rev ? ex2(mm[c]) : ex2(gg[c] - mm[c]);
              const float c_new = rev ? ex2(gg[c] - mm[c]) : ex2(mm[c]);
              sm->cf[d0 + c] = c_new * u_old;
              sm->uvec[d0 + c] = u_new;
              bad = bad || (-mm[c] > SafeBits<T>::value) || (-(gg[c] - mm[c]) > SafeBits<T>::value);
            } else {
              // forward: copy T e^{r1}, resident e^{r3} T + update, e^{g-r3} owed;
              // reverse: copy T e^{g-r3}, resident e^{g-r1} T + update, e^{r1} owed
              sm->cf[d0 + c] = (rev ? ex2(gg[c] - q3[c]) : ex2(q1[c])) * u_old;
              sm->bfv[d0 + c] = (rev ? ex2(gg[c] - q1[c]) : ex2(q3[c])) * u_old;
              sm->uvec[d0 + c] = rev ? ex2(q1[c]) : ex2(gg[c] - q3[c]);
              sm->dl[d0 + c] = q3[c] - q1[c];
              const float lim = SafeBits2<T>::value;
              bad = bad || (-q1[c] > lim) || (q1[c] - mm[c] > lim) || (mm[c] - q3[c] > lim) || (q3[c] - gg[c] > lim);
            }
          }
          if (bad) atomicExch(a.unsafe, 1);
        }
        named_bar_sync(1, kComputeThreads);
      }

      // ---- R: rescale operands in place
      if (!TMODE) {  // T mode rescales Z only, which came with the decay tile
        mbar_wait(full_yz, par, abort_flag, a.status, kStFull);
        mbar_wait(full_x, par, abort_flag, a.status, kStFull);
      }
      if (REF2) {
        if (!TMODE) {
          if (rev) rescale2_xy<T, true>(gbase, ck, sm->dl, i, wg, L);
          else rescale2_xy<T, false>(gbase, ck, sm->dl, i, wg, L);
        } else {
          // the spare tile is the unused half of the region Y was loaded into; that region staged
          // the previous chunk's gradient terms, and Y's arrival says the store has let go of it
          mbar_wait(full_yz, par, abort_flag, a.status, kStFull);
          const uint32_t f_off = ((it & 1) ? kOffCk : kOffY) + kTileBytes;
          if (rev) rescale2_z<T, true>(gbase, z_off, f_off, ck, sm->dl, i, wg, L);
          else rescale2_z<T, false>(gbase, z_off, f_off, ck, sm->dl, i, wg, L);
        }
      } else if (!TMODE) {
        if (rev) rescale_xy<T, true>(gbase, ck, i, wg, L);   // dv: X = k 2^(m-ck), Y = q 2^(ck-m)
        else rescale_xy<T, false>(gbase, ck, i, wg, L);      // o:  X = q 2^(ck-m), Y = k 2^(m-ck)
      } else {
        if (rev) rescale_z<T, false>(gbase, z_off, ck, i, wg, L);   // dk: Z = q 2^(ck-m)
        else rescale_z<T, true>(gbase, z_off, ck, i, wg, L);        // dq: Z = k 2^(m-ck)
      }
      fence_proxy_async();
      mbar_arrive(bar_r);
      if (!TMODE) mbar_arrive(empty_ck);  // N mode reads the decay tile for the last time above

      // ---- D: scaled 16-bit state copy (B operand of X T), decay of the resident state
      {
        uint32_t r0[32], r1[32];
        tmem_ld32(tl + kColT + (2 * wg) * 32, r0);
        tmem_ld32(tl + kColT + (2 * wg + 1) * 32, r1);
        tmem_wait_ld();
        uint8_t *box = gbase + kOffTb + wg * kBoxBytes;
        // With a log-decay gradient requested (one reference) the copy is written as a high and a
        // low 16-bit half: the inter-chunk parts of q*dq and k*dk cancel only as far as the forward
        // and reverse states agree, and a single 16-bit rounding of the copy is what limits that.
        // The low half goes to the unused half of the region Y was loaded into (that region staged
        // the previous chunk's gradient terms; Y's arrival says the store has let go of it).
        const bool splitc = TMODE && !REF2 && a.dld != nullptr;
        // two references: no spare tile; the low half waits in registers until X T_hi is done
        const bool splits = TMODE && REF2 && a.dld != nullptr;
        uint32_t lo_keep[32];
        uint8_t *lbox = gbase + ((it & 1) ? kOffCk : kOffY) + kTileBytes + wg * kBoxBytes;
        if (splitc) mbar_wait(full_yz, par, abort_flag, a.status, kStFull);
        const float cf_row = sm->cf[i], bf_row = REF2 ? sm->bfv[i] : 0.f;
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          uint32_t(&r)[32] = hf ? r1 : r0;
#pragma unroll
          for (int pc = 0; pc < 4; ++pc) {
            float2 c01, c23, c45, c67;
            const int d0 = wg * 64 + hf * 32 + pc * 8;
            if (TMODE) {
              const float4 ca = *reinterpret_cast<const float4 *>(&sm->cf[d0]);
              const float4 cb = *reinterpret_cast<const float4 *>(&sm->cf[d0 + 4]);
              c01 = make_float2(ca.x, ca.y); c23 = make_float2(ca.z, ca.w);
              c45 = make_float2(cb.x, cb.y); c67 = make_float2(cb.z, cb.w);
            } else {
              c01 = c23 = c45 = c67 = make_float2(cf_row, cf_row);
            }
            // one scaled value serves as the 16-bit copy and as the state the update adds to
            // (two references: the copy and the resident state take different factors)
            const float2 s01 = mul2(f2(r[pc * 8 + 0], r[pc * 8 + 1]), c01), s23 = mul2(f2(r[pc * 8 + 2], r[pc * 8 + 3]), c23);
            const float2 s45 = mul2(f2(r[pc * 8 + 4], r[pc * 8 + 5]), c45), s67 = mul2(f2(r[pc * 8 + 6], r[pc * 8 + 7]), c67);
            uint4 v;
            v.x = Fmt<T>::pack(s01.x, s01.y); v.y = Fmt<T>::pack(s23.x, s23.y);
            v.z = Fmt<T>::pack(s45.x, s45.y); v.w = Fmt<T>::pack(s67.x, s67.y);
            *reinterpret_cast<uint4 *>(box + sw128_offset(i, hf * 4 + pc)) = v;
            if (splitc || splits) {
              const float2 h01 = Fmt<T>::unpack(v.x), h23 = Fmt<T>::unpack(v.y), h45 = Fmt<T>::unpack(v.z), h67 = Fmt<T>::unpack(v.w);
              uint4 l;
              l.x = Fmt<T>::pack(s01.x - h01.x, s01.y - h01.y); l.y = Fmt<T>::pack(s23.x - h23.x, s23.y - h23.y);
              l.z = Fmt<T>::pack(s45.x - h45.x, s45.y - h45.y); l.w = Fmt<T>::pack(s67.x - h67.x, s67.y - h67.y);
              if (splitc) {
                *reinterpret_cast<uint4 *>(lbox + sw128_offset(i, hf * 4 + pc)) = l;
              } else {
                lo_keep[hf * 16 + pc * 4 + 0] = l.x; lo_keep[hf * 16 + pc * 4 + 1] = l.y;
                lo_keep[hf * 16 + pc * 4 + 2] = l.z; lo_keep[hf * 16 + pc * 4 + 3] = l.w;
              }
            }
            if (!REF2) {
              r[pc * 8 + 0] = __float_as_uint(s01.x); r[pc * 8 + 1] = __float_as_uint(s01.y);
              r[pc * 8 + 2] = __float_as_uint(s23.x); r[pc * 8 + 3] = __float_as_uint(s23.y);
              r[pc * 8 + 4] = __float_as_uint(s45.x); r[pc * 8 + 5] = __float_as_uint(s45.y);
              r[pc * 8 + 6] = __float_as_uint(s67.x); r[pc * 8 + 7] = __float_as_uint(s67.y);
            } else {
              float2 b01, b23, b45, b67;
              if (TMODE) {
                const float4 ba = *reinterpret_cast<const float4 *>(&sm->bfv[d0]);
                const float4 bb = *reinterpret_cast<const float4 *>(&sm->bfv[d0 + 4]);
                b01 = make_float2(ba.x, ba.y); b23 = make_float2(ba.z, ba.w);
                b45 = make_float2(bb.x, bb.y); b67 = make_float2(bb.z, bb.w);
              } else {
                b01 = b23 = b45 = b67 = make_float2(bf_row, bf_row);
              }
              const float2 t01 = mul2(f2(r[pc * 8 + 0], r[pc * 8 + 1]), b01), t23 = mul2(f2(r[pc * 8 + 2], r[pc * 8 + 3]), b23);
              const float2 t45 = mul2(f2(r[pc * 8 + 4], r[pc * 8 + 5]), b45), t67 = mul2(f2(r[pc * 8 + 6], r[pc * 8 + 7]), b67);
              r[pc * 8 + 0] = __float_as_uint(t01.x); r[pc * 8 + 1] = __float_as_uint(t01.y);
              r[pc * 8 + 2] = __float_as_uint(t23.x); r[pc * 8 + 3] = __float_as_uint(t23.y);
              r[pc * 8 + 4] = __float_as_uint(t45.x); r[pc * 8 + 5] = __float_as_uint(t45.y);
              r[pc * 8 + 6] = __float_as_uint(t67.x); r[pc * 8 + 7] = __float_as_uint(t67.y);
            }
          }
        }
        tmem_st32(tl + kColT + (2 * wg) * 32, r0);
        tmem_st32(tl + kColT + (2 * wg + 1) * 32, r1);
        tmem_wait_st();
        fence_proxy_async();
        tc_fence_before();
        mbar_arrive(bar_d);
        if (splits) {
          mbar_wait(bar_x, par, abort_flag, a.status, kStX);
#pragma unroll
          for (int pc8 = 0; pc8 < 8; ++pc8)
            *reinterpret_cast<uint4 *>(box + sw128_offset(i, pc8)) =
                make_uint4(lo_keep[pc8 * 4], lo_keep[pc8 * 4 + 1], lo_keep[pc8 * 4 + 2], lo_keep[pc8 * 4 + 3]);
          fence_proxy_async();
          mbar_arrive(bar_l);
        }
      }

      // ---- F: causal (or reverse-causal) 16-bit P~ in the first 16 columns of each 32-column batch
      mbar_wait(bar_p, par, abort_flag, a.status, kStP);
      tc_fence_after();
#pragma unroll 1
      for (int b2 = 0; b2 < 2; ++b2) {
        const int bt = wg + 2 * b2;
        uint32_t pk[16];
        const bool dead = rev ? (bt < q4) : (bt > q4);
        if (dead) {
#pragma unroll
          for (int k = 0; k < 16; ++k) pk[k] = 0u;
        } else {
          uint32_t r[32];
          tmem_ld32(tl + kColP + bt * 32, r);
          tmem_wait_ld();
          // bit k of `keep`: column 32 bt + k of this row survives the (reverse-)causal mask
          const int lo = i - bt * 32;      // forward: columns k <= lo; reverse: columns k >= lo ...
          const int hi = L - bt * 32;      // ... and k < hi (end of the sequence)
          uint32_t keep;
          if (!rev) keep = lo >= 31 ? 0xffffffffu : (lo < 0 ? 0u : (0xffffffffu >> (31 - lo)));
          else {
            keep = lo <= 0 ? 0xffffffffu : (lo > 31 ? 0u : (0xffffffffu << lo));
            if (hi < 32) keep &= hi <= 0 ? 0u : (0xffffffffu >> (32 - hi));
          }
#pragma unroll
          for (int k = 0; k < 32; k += 2) {
            // select, not multiply: masked-out entries may be inf or NaN
            pk[k >> 1] = Fmt<T>::pack(((keep >> k) & 1u) ? __uint_as_float(r[k]) : 0.f,
                                      ((keep >> (k + 1)) & 1u) ? __uint_as_float(r[k + 1]) : 0.f);
          }
        }
        tmem_st16(tl + kColP + bt * 32, pk);
        if (TMODE && REF2 && rev && bt >= 2) {
          // second copy of the batch with rows 0..63 zeroed, in the half of the batch the 16-bit
          // values leave free (this thread read those columns above, or the batch is dead)
          if (i < 64) {
#pragma unroll
            for (int k = 0; k < 16; ++k) pk[k] = 0u;
          }
          tmem_st16(tl + kColP + bt * 32 + 16, pk);
        }
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bar_f);

      // ---- H: epilogue
      mbar_wait(bar_w, par, abort_flag, a.status, kStW);
      tc_fence_after();
      const bool full_chunk = (L == kChunk);
      const long long row_off = ((bidx * (long long)a.N + tok) * a.H + h) * (long long)kChunk;
      // packed fp32x2 arithmetic throughout: every product below is an fp32 multiply rounded to
      // nearest, exactly as its scalar form
      if (TMODE && REF2) {
        // Two accumulators with different output scales (see the file header): rows 0..63 take
        // Wa, rows 64..127 take Wb, each times 2^(+-t); the rows that reach across the middle
        // (forward: 64..127, reverse: 0..63) add the other accumulator times the mixed factor.
        const bool top = i < 64;              // warp-uniform
        const bool two = rev ? top : !top;
        const bool want_dld = a.dld != nullptr && i < L;
        const uint32_t colA = top ? kColW1 : kColW2, colB = top ? kColW2 : kColW1;
#pragma unroll 1
        for (int cb = 0; cb < 4; ++cb) {      // this warpgroup's 64 columns, 16 at a time
          const int c0 = wg * 64 + cb * 16;
          uint4 xv2[2] = {};
          if (want_dld) {
            const uint4 *xp = reinterpret_cast<const uint4 *>(static_cast<const T *>(a.xrow) + row_off + c0);
            xv2[0] = __ldg(xp);
            xv2[1] = __ldg(xp + 1);
          }
          uint32_t wa[16], wb[16];
          tmem_ld16(tl + colA + c0, wa);
          if (two) tmem_ld16(tl + colB + c0, wb);
          tmem_wait_ld();
          const uint32_t flip = (full_chunk && a.dld_sub) ? 0x80008000u : 0u;
#pragma unroll
          for (int pc = 0; pc < 2; ++pc) {
            const int d0 = c0 + pc * 8;
            float t[8], dd[8];
            tile_vals(ck, sm->dl, i, d0, t, dd);
            float2 ov[4], pr[4];
            const uint32_t xw[4] = {xv2[pc].x ^ flip, xv2[pc].y ^ flip, xv2[pc].z ^ flip, xv2[pc].w ^ flip};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float e0 = rev ? -t[2 * j] : t[2 * j], e1 = rev ? -t[2 * j + 1] : t[2 * j + 1];
              const float2 sA = make_float2(ex2(e0), ex2(e1));
              const float2 wA = f2(wa[pc * 8 + 2 * j], wa[pc * 8 + 2 * j + 1]);
              ov[j] = mul2(wA, sA);
              const float2 xa = mul2(Fmt<T>::unpack(xw[j]), sA);
              pr[j] = mul2(Fmt<T>::unpack(Fmt<T>::pack(xa.x, xa.y)), wA);
              if (two) {
                const float2 sB = make_float2(ex2(e0 + dd[2 * j]), ex2(e1 + dd[2 * j + 1]));
                const float2 wB = f2(wb[pc * 8 + 2 * j], wb[pc * 8 + 2 * j + 1]);
                ov[j] = fma2(wB, sB, ov[j]);
                const float2 xb = mul2(Fmt<T>::unpack(xw[j]), sB);
                pr[j] = fma2(Fmt<T>::unpack(Fmt<T>::pack(xb.x, xb.y)), wB, pr[j]);
              }
            }
            if (want_dld) {
              float4 lo = make_float4(pr[0].x, pr[0].y, pr[1].x, pr[1].y);
              float4 hi = make_float4(pr[2].x, pr[2].y, pr[3].x, pr[3].y);
              float4 *dp = reinterpret_cast<float4 *>(a.dld + row_off + d0);
              if (full_chunk) {
                *reinterpret_cast<float4 *>(ck + ck_off(i, d0)) = lo;
                *reinterpret_cast<float4 *>(ck + ck_off(i, d0 + 4)) = hi;
              } else if (a.dld_add) {
                const float sg = a.dld_sub ? -1.f : 1.f;
                float *dpf = reinterpret_cast<float *>(dp);
                atomicAdd(dpf + 0, sg * lo.x); atomicAdd(dpf + 1, sg * lo.y); atomicAdd(dpf + 2, sg * lo.z); atomicAdd(dpf + 3, sg * lo.w);
                atomicAdd(dpf + 4, sg * hi.x); atomicAdd(dpf + 5, sg * hi.y); atomicAdd(dpf + 6, sg * hi.z); atomicAdd(dpf + 7, sg * hi.w);
              } else {
                if (a.dld_sub) {
                  const float4 ol = dp[0], oh = dp[1];
                  lo = make_float4(ol.x - lo.x, ol.y - lo.y, ol.z - lo.z, ol.w - lo.w);
                  hi = make_float4(oh.x - hi.x, oh.y - hi.y, oh.z - hi.z, oh.w - hi.w);
                }
                dp[0] = lo;
                dp[1] = hi;
              }
            }
            uint4 v;
            v.x = Fmt<T>::pack(ov[0].x, ov[0].y); v.y = Fmt<T>::pack(ov[1].x, ov[1].y);
            v.z = Fmt<T>::pack(ov[2].x, ov[2].y); v.w = Fmt<T>::pack(ov[3].x, ov[3].y);
            if (full_chunk) {
              *reinterpret_cast<uint4 *>(gbase + kOffX + wg * kBoxBytes + sw128_offset(i, cb * 2 + pc)) = v;
            } else if (i < L) {
              reinterpret_cast<uint4 *>(static_cast<T *>(a.out) + row_off + d0)[0] = v;
            }
          }
        }
      } else
#pragma unroll 1
      for (int b2 = 0; b2 < 2; ++b2) {
        const int bt = 2 * wg + b2;
        // the row of xrow for the gradient terms: in flight while the accumulators are read and
        // the scale factors computed
        const bool want_dld = TMODE && a.dld != nullptr && i < L;
        uint4 xv4[4] = {};
        if (want_dld) {
          const uint4 *xp = reinterpret_cast<const uint4 *>(static_cast<const T *>(a.xrow) + row_off + bt * 32);
#pragma unroll
          for (int pc = 0; pc < 4; ++pc) xv4[pc] = __ldg(xp + pc);
        }
        uint32_t w1[32], w2[32];
        tmem_ld32(tl + kColW1 + bt * 32, w1);
        tmem_ld32(tl + kColW2 + bt * 32, w2);
        tmem_wait_ld();
        float2 w[16], scl[16];  // pairs of adjacent columns
#pragma unroll
        for (int k = 0; k < 32; k += 4) {
          float2 s0 = make_float2(1.f, 1.f), s1 = s0;
          if (TMODE) {
            const float4 c = *reinterpret_cast<const float4 *>(ck + ck_off(i, bt * 32 + k));
            if (rev) { s0 = make_float2(ex2(-c.x), ex2(-c.y)); s1 = make_float2(ex2(-c.z), ex2(-c.w)); }
            else { s0 = make_float2(ex2(c.x), ex2(c.y)); s1 = make_float2(ex2(c.z), ex2(c.w)); }
          }
          w[(k >> 1) + 0] = __fadd2_rn(f2(w1[k + 0], w1[k + 1]), f2(w2[k + 0], w2[k + 1]));
          w[(k >> 1) + 1] = __fadd2_rn(f2(w1[k + 2], w1[k + 3]), f2(w2[k + 2], w2[k + 3]));
          scl[(k >> 1) + 0] = s0;
          scl[(k >> 1) + 1] = s1;
        }
        if (want_dld) {
          // Log-decay gradient term x * W.  W = w * scl, but the product is formed as
          // round16(x * scl) * w: round16(x * scl) is exactly the rescaled operand the twin pass
          // feeds to the tensor cores, so the intra-chunk parts of q*dq and k*dk cancel term by term
          // as they do in exact arithmetic.  The sign of the dk pass goes onto x (a bit flip).
          float4 *dp = reinterpret_cast<float4 *>(a.dld + row_off + bt * 32);
          const uint32_t flip = (full_chunk && a.dld_sub) ? 0x80008000u : 0u;
#pragma unroll
          for (int pc = 0; pc < 4; ++pc) {
            const uint4 xv = xv4[pc];
            const uint32_t xw[4] = {xv.x ^ flip, xv.y ^ flip, xv.z ^ flip, xv.w ^ flip};
            float2 pr[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 t = mul2(Fmt<T>::unpack(xw[j]), scl[pc * 4 + j]);
              pr[j] = mul2(Fmt<T>::unpack(Fmt<T>::pack(t.x, t.y)), w[pc * 4 + j]);
            }
            float4 lo = make_float4(pr[0].x, pr[0].y, pr[1].x, pr[1].y);
            float4 hi = make_float4(pr[2].x, pr[2].y, pr[3].x, pr[3].y);
            if (full_chunk) {
              // stage in the decay tile (this thread's row, columns already consumed above); the
              // store warp writes the tile out with TMA
              const int d0 = bt * 32 + pc * 8;
              *reinterpret_cast<float4 *>(ck + ck_off(i, d0)) = lo;
              *reinterpret_cast<float4 *>(ck + ck_off(i, d0 + 4)) = hi;
              continue;
            }
            if (a.dld_add) {  // the twin pass may be on this tile too
              const float sg = a.dld_sub ? -1.f : 1.f;
              float *dpf = reinterpret_cast<float *>(dp + pc * 2);
              atomicAdd(dpf + 0, sg * lo.x); atomicAdd(dpf + 1, sg * lo.y); atomicAdd(dpf + 2, sg * lo.z); atomicAdd(dpf + 3, sg * lo.w);
              atomicAdd(dpf + 4, sg * hi.x); atomicAdd(dpf + 5, sg * hi.y); atomicAdd(dpf + 6, sg * hi.z); atomicAdd(dpf + 7, sg * hi.w);
              continue;
            }
            if (a.dld_sub) {
              const float4 ol = dp[pc * 2], oh = dp[pc * 2 + 1];
              lo = make_float4(ol.x - lo.x, ol.y - lo.y, ol.z - lo.z, ol.w - lo.w);
              hi = make_float4(oh.x - hi.x, oh.y - hi.y, oh.z - hi.z, oh.w - hi.w);
            }
            dp[pc * 2] = lo;
            dp[pc * 2 + 1] = hi;
          }
        }
#pragma unroll
        for (int pc = 0; pc < 4; ++pc) {
          uint4 v;
          float2 t;
          t = mul2(w[pc * 4 + 0], scl[pc * 4 + 0]); v.x = Fmt<T>::pack(t.x, t.y);
          t = mul2(w[pc * 4 + 1], scl[pc * 4 + 1]); v.y = Fmt<T>::pack(t.x, t.y);
          t = mul2(w[pc * 4 + 2], scl[pc * 4 + 2]); v.z = Fmt<T>::pack(t.x, t.y);
          t = mul2(w[pc * 4 + 3], scl[pc * 4 + 3]); v.w = Fmt<T>::pack(t.x, t.y);
          if (full_chunk) {
            *reinterpret_cast<uint4 *>(gbase + kOffX + wg * kBoxBytes + sw128_offset(i, b2 * 4 + pc)) = v;
          } else if (i < L) {
            reinterpret_cast<uint4 *>(static_cast<T *>(a.out) + row_off + bt * 32)[pc] = v;
          }
        }
      }
      if (full_chunk) fence_proxy_async();
      tc_fence_before();
      mbar_arrive(bar_h);
    }

    if (a.tfinal != nullptr) {  // end state -> global, with the factor still owed to it
      named_bar_sync(1, kComputeThreads);  // uvec of the last chunk (or its initial ones) is in place
      tc_fence_after();
      const float u_row = sm->uvec[i];
      for (int b2 = 0; b2 < 2; ++b2) {
        const int bt = 2 * wg + b2;
        uint32_t r[32];
        tmem_ld32(tl + kColT + bt * 32, r);
        tmem_wait_ld();
#pragma unroll
        for (int k = 0; k < 32; ++k) {
          const int c = bt * 32 + k;
          const float u = TMODE ? sm->uvec[c] : u_row;
          a.tfinal[st_base + (a.state_transposed ? (c * kChunk + i) : (i * kChunk + c))] = __uint_as_float(r[k]) * u;
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kProducerWarp) {
    if (lane == 0 && sm->abort_flag != 0) {
      int dummy = 0;
      const uint32_t fulls[3] = {full_ck, full_yz, full_x};
      for (int gq = 0; gq < 3; ++gq)
        if (sm->issued[gq] > 0)
          mbar_wait(fulls[gq], (uint32_t)(sm->issued[gq] - 1) & 1u, &dummy, nullptr, 0, 1u << 20);
    }
    __syncwarp();
    tmem_dealloc(tmem, 512);
  }
}

template <typename T, bool TMODE, bool REF2>
int launch_t(const LavdPass &p, int dtype, cudaStream_t stream) {
  alignas(64) CUtensorMap mx, my, mz, ml, mo, md;
  int rc;
  if ((rc = make_map(&mx, p.x, dtype, p.B, p.N, p.H)) != LA_OK) return rc;
  if ((rc = make_map(&my, p.y, dtype, p.B, p.N, p.H)) != LA_OK) return rc;
  if ((rc = make_map(&mz, p.z, dtype, p.B, p.N, p.H)) != LA_OK) return rc;
  if ((rc = make_map(&ml, p.ldk, p.ld16 ? dtype : LA_F32, p.B, p.N, p.H)) != LA_OK) return rc;
  if ((rc = make_map(&mo, p.out, dtype, p.B, p.N, p.H)) != LA_OK) return rc;
  if (p.dld != nullptr && ((reinterpret_cast<uintptr_t>(p.xrow) | reinterpret_cast<uintptr_t>(p.dld)) & 15u))
    return LA_ERR_MISALIGNED;
  // without a gradient buffer the map is never used; point it at the decay tensor to keep it valid
  if ((rc = make_map(&md, p.dld != nullptr ? static_cast<const void *>(p.dld) : static_cast<const void *>(p.ldk),
                     LA_F32, p.B, p.N, p.H)) != LA_OK)
    return rc;
  LavdArgs a;
  a.out = p.out; a.xrow = p.xrow; a.dld = p.xrow ? p.dld : nullptr; a.dld_sub = p.dld_sub; a.dld_add = p.dld_add;
  a.t0 = p.t0; a.tfinal = p.tfinal; a.state_transposed = p.state_transposed; a.reverse = p.reverse;
  a.cu = reinterpret_cast<const long long *>(p.cu);
  a.B = p.B; a.N = p.N; a.H = p.H; a.M = p.M;
  a.status = status_word_ptr();
  a.unsafe = p.unsafe;
  a.enable = p.enable;
  a.ld_act = p.ld_act;
  a.ld16 = p.ld16;
  if (a.status == nullptr || a.unsafe == nullptr) return LA_ERR_CUDA;
  auto kern = lavd_pass_kernel<T, TMODE, REF2>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess)
    return LA_ERR_CUDA;
  const int nb = p.cu ? p.M : p.B;
  kern<<<nb * p.H, kThreads, kSmemBytes, stream>>>(mx, my, mz, ml, mo, md, a);
  return launch_status();
}

}  // namespace

bool lavd_chunk_supported(int64_t N, int64_t D, int64_t E, int dtype, bool has_ldk, bool has_ldv) {
  // exactly one decay: on the key features (ldk) or, by exchanging the roles of the passes, on the
  // value features (ldv); both at once would need a second 64 KB decay tile per chunk
  return (has_ldk != has_ldv) && (dtype == LA_BF16 || dtype == LA_F16) && D == 128 && E == 128 && N >= 128;
}

int launch_lavd_pass(const LavdPass &p, int dtype, cudaStream_t stream) {
  if (p.x == nullptr || p.y == nullptr || p.z == nullptr || p.out == nullptr || p.ldk == nullptr)
    return LA_ERR_NULL_POINTER;
  const int nb = p.cu ? p.M : p.B;
  if (nb <= 0 || p.H <= 0 || p.N <= 0) return LA_ERR_BAD_SHAPE;
  if (dtype == LA_BF16) {
    if (p.ref2)
      return p.tmode ? launch_t<__nv_bfloat16, true, true>(p, dtype, stream)
                     : launch_t<__nv_bfloat16, false, true>(p, dtype, stream);
    return p.tmode ? launch_t<__nv_bfloat16, true, false>(p, dtype, stream)
                   : launch_t<__nv_bfloat16, false, false>(p, dtype, stream);
  }
  if (dtype == LA_F16) {
    if (p.ref2)
      return p.tmode ? launch_t<__half, true, true>(p, dtype, stream) : launch_t<__half, false, true>(p, dtype, stream);
    return p.tmode ? launch_t<__half, true, false>(p, dtype, stream) : launch_t<__half, false, false>(p, dtype, stream);
  }
  return LA_ERR_UNSUPPORTED;
}

}  // namespace la
