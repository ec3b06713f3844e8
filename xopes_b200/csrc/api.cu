// extern "C" entry points: argument checks, choice of kernel family, pass orchestration.
#include <mutex>

#include "chunk.cuh"
#include "scan.cuh"

namespace la {

__device__ int g_status_word = 0;

char *last_cuda_error_buf() {
  static thread_local char buf[256] = "";
  return buf;
}

int *status_word_ptr() {
  static int *ptrs[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (ptrs[dev] == nullptr) {
    void *p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) return nullptr;
    ptrs[dev] = static_cast<int *>(p);
  }
  return ptrs[dev];
}

// [0]: raised by the one-reference vector-decay chunk kernels when a chunk leaves their safe range
// (the two-reference kernels then run); [1]: raised by those in turn (the scan kernels then run)
__device__ int g_lavd_unsafe[2] = {0, 0};

static int *lavd_unsafe_ptr() {
  static int *ptrs[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (ptrs[dev] == nullptr) {
    void *p = nullptr;
    if (cudaGetSymbolAddress(&p, g_lavd_unsafe) != cudaSuccess) return nullptr;
    ptrs[dev] = static_cast<int *>(p);
  }
  return ptrs[dev];
}

namespace {

// A second stream per device for passes of one call that do not depend on each other (a gradient
// pass that would leave SMs idle runs beside the next one).  fork() makes the side stream wait for
// everything already queued on the caller's stream, join() makes the caller's stream wait for the
// side stream.  One caller at a time per device: the lock is held from fork to join.
struct SideStream {
  cudaStream_t stream = nullptr, stream2 = nullptr;
  cudaEvent_t fork_ev = nullptr, join_ev = nullptr, join_ev2 = nullptr;
  std::mutex mu;
  bool ready = false, failed = false;
};

SideStream *side_stream() {
  static SideStream side[64];
  static std::mutex init_mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(init_mu);
  SideStream &s = side[dev];
  if (!s.ready && !s.failed) {
    if (cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaStreamCreateWithFlags(&s.stream2, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&s.fork_ev, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&s.join_ev, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&s.join_ev2, cudaEventDisableTiming) != cudaSuccess) {
      s.failed = true;
      cudaGetLastError();
    } else {
      s.ready = true;
    }
  }
  return s.ready ? &s : nullptr;
}

bool side_fork(SideStream *s, cudaStream_t st) {
  return cudaEventRecord(s->fork_ev, st) == cudaSuccess && cudaStreamWaitEvent(s->stream, s->fork_ev, 0) == cudaSuccess;
}
bool side_join(SideStream *s, cudaStream_t st) {
  return cudaEventRecord(s->join_ev, s->stream) == cudaSuccess && cudaStreamWaitEvent(st, s->join_ev, 0) == cudaSuccess;
}
// the second side stream, forked from the same event (call side_fork first)
bool side_fork2(SideStream *s) { return cudaStreamWaitEvent(s->stream2, s->fork_ev, 0) == cudaSuccess; }
bool side_join2(SideStream *s, cudaStream_t st) {
  return cudaEventRecord(s->join_ev2, s->stream2) == cudaSuccess && cudaStreamWaitEvent(st, s->join_ev2, 0) == cudaSuccess;
}

int sm_count() {
  static int sms[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (sms[dev] == 0 && cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
  return sms[dev];
}

bool dtype_ok(int dtype) { return dtype == LA_F32 || dtype == LA_BF16 || dtype == LA_F16; }

int check_common(const void *q, const void *k, const void *v, int64_t B, int64_t N, int64_t H,
                 int64_t D, int64_t E, int64_t M, const int64_t *cu, int dtype) {
  // An error another library left behind on this thread (the runtime keeps the last one until it is
  // read) must not be taken for a failure of the launches that follow.
  cudaGetLastError();
  if (q == nullptr || k == nullptr || v == nullptr) return LA_ERR_NULL_POINTER;
  if (B <= 0 || N <= 0 || H <= 0 || D <= 0 || E <= 0) return LA_ERR_BAD_SHAPE;
  if (cu != nullptr && (B != 1 || M <= 0)) return LA_ERR_BAD_SHAPE;
  if (cu == nullptr && M != 0) return LA_ERR_BAD_SHAPE;  // M counts documents: meaningless without cu_seqlens
  if (!dtype_ok(dtype)) return LA_ERR_UNSUPPORTED;
  if (N > (int64_t)1 << 30 || B > 65535 || H > 65535 || M > 65535) return LA_ERR_TOO_LARGE;
  return LA_OK;
}

struct Seq {
  int B, N, H, D, E, M;
  const int64_t *cu;
  int nb() const { return cu ? M : B; }
};

// The four directional passes expressed on the scan primitive.
ScanParams base_params(const Seq &s, const float *ld, int64_t sb, int64_t sn, int64_t sh) {
  ScanParams p;
  p.B = s.B; p.N = s.N; p.H = s.H; p.M = s.M; p.cu = s.cu;
  p.ld = ld; p.ld_sb = sb; p.ld_sn = sn; p.ld_sh = sh;
  return p;
}

// rows = E (T = S^T): output pass and dv pass
void rows_e(ScanParams &p, const Seq &s, const float *ldk, const float *ldv) {
  p.R = s.E; p.C = s.D; p.st_rs = 1; p.st_cs = s.E; p.ldr = ldv; p.ldc = ldk;
}
// rows = D (T = S): dq pass and dk pass
void rows_d(ScanParams &p, const Seq &s, const float *ldk, const float *ldv) {
  p.R = s.D; p.C = s.E; p.st_rs = s.E; p.st_cs = 1; p.ldr = ldk; p.ldc = ldv;
}

int scan_forward(const Seq &s, const void *q, const void *k, const void *v, const float *ld,
                 int64_t sb, int64_t sn, int64_t sh, const float *ldk, const float *ldv,
                 const float *s0, void *o, float *sfin, int dtype, cudaStream_t st,
                 const int *enable = nullptr, int ld_act = 0, int ld16 = 0) {
  ScanParams p = base_params(s, ld, sb, sn, sh);
  p.enable = enable;
  p.ld_act = ld_act;
  p.ld16 = ld16;
  rows_e(p, s, ldk, ldv);
  p.a = v; p.b = k; p.w = q; p.out = o; p.t0 = s0; p.tfinal = sfin;
  return launch_scan(p, dtype, st);
}

}  // namespace
}  // namespace la

using namespace la;

extern "C" {

int la_abi_version(void) { return 1; }

const char *la_status_string(int status) {
  switch (status) {
    case LA_OK: return "ok";
    case LA_ERR_NULL_POINTER: return "a required pointer is NULL";
    case LA_ERR_BAD_SHAPE: return "bad shape";
    case LA_ERR_UNSUPPORTED: return "unsupported dtype or head dimension";
    case LA_ERR_CUDA: return "CUDA call failed";
    case LA_ERR_TOO_LARGE: return "size exceeds a fixed maximum";
    case LA_ERR_MISALIGNED: return "pointer not aligned as required";
    case LA_ERR_WORKSPACE: return "workspace missing or too small";
  }
  return "unknown status";
}

int la_lasd_path(int64_t N, int64_t D, int64_t E, int dtype, unsigned flags) {
  if (!dtype_ok(dtype)) return LA_ERR_UNSUPPORTED;
  const bool tensor = !(flags & LA_FLAG_FORCE_RECURRENCE) && chunk_supported(N, D, E, dtype);
  if (!tensor && (flags & LA_FLAG_REQUIRE_TENSOR)) return LA_ERR_UNSUPPORTED;
  return tensor ? 1 : 0;
}

int la_device_status(void *stream, int *status_out) {
  if (status_out == nullptr) return LA_ERR_NULL_POINTER;
  int *p = status_word_ptr();
  if (p == nullptr) return LA_ERR_CUDA;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cudaMemcpyAsync(status_out, p, sizeof(int), cudaMemcpyDeviceToHost, st) != cudaSuccess) return LA_ERR_CUDA;
  if (cudaStreamSynchronize(st) != cudaSuccess) return LA_ERR_CUDA;
  return LA_OK;
}

int la_device_status_clear(void *stream) {
  int *p = status_word_ptr();
  if (p == nullptr) return LA_ERR_CUDA;
  if (cudaMemsetAsync(p, 0, sizeof(int), static_cast<cudaStream_t>(stream)) != cudaSuccess) return LA_ERR_CUDA;
  return LA_OK;
}

int la_debug_lavd_unsafe(void *stream, int *flag_out) {
  if (flag_out == nullptr) return LA_ERR_NULL_POINTER;
  int *p = lavd_unsafe_ptr();
  if (p == nullptr) return LA_ERR_CUDA;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int w[2] = {0, 0};
  if (cudaMemcpyAsync(w, p, sizeof(w), cudaMemcpyDeviceToHost, st) != cudaSuccess) return LA_ERR_CUDA;
  if (cudaStreamSynchronize(st) != cudaSuccess) return LA_ERR_CUDA;
  *flag_out = w[1] != 0 ? 2 : (w[0] != 0 ? 1 : 0);
  return LA_OK;
}

const char *la_debug_last_cuda_error(void) { return last_cuda_error_buf(); }

int la_debug_wait_probe(int64_t limit_us, void *stream) {
  if (limit_us <= 0 || limit_us > 1000000) return LA_ERR_BAD_SHAPE;
  return wait_probe((uint32_t)limit_us, static_cast<cudaStream_t>(stream));
}

int la_debug_umma_probe(int variant, const void *a, const void *b, float *d, int dtype, void *stream) {
  return umma_probe(variant, a, b, d, dtype, static_cast<cudaStream_t>(stream));
}

// ------------------------------------------------------------------------------------------------
// scalar decay
// ------------------------------------------------------------------------------------------------
int la_lasd_fwd(const void *q, const void *k, const void *v, const float *ld, int64_t ld_sb,
                int64_t ld_sn, int64_t ld_sh, const float *initial_state,
                const int64_t *cu_seqlens, void *o, float *final_state, int64_t B, int64_t N,
                int64_t H, int64_t D, int64_t E, int64_t M, int dtype, unsigned flags,
                void *stream) {
  int rc = check_common(q, k, v, B, N, H, D, E, M, cu_seqlens, dtype);
  if (rc != LA_OK) return rc;
  if (o == nullptr || ld == nullptr) return LA_ERR_NULL_POINTER;
  if (flags & LA_FLAG_LD_16BIT) return LA_ERR_UNSUPPORTED;  // the scalar decay is always fp32
  const int path = la_lasd_path(N, D, E, dtype, flags);
  if (path < 0) return path;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Seq s{(int)B, (int)N, (int)H, (int)D, (int)E, (int)M, cu_seqlens};
  if (path == 1) {
    ChunkPass c;
    c.x = q; c.y = k; c.z = v; c.out = o;
    c.ld = ld; c.ld_sb = ld_sb; c.ld_sn = ld_sn; c.ld_sh = ld_sh;
    c.t0 = initial_state; c.tfinal = final_state; c.state_transposed = 0; c.reverse = 0;
    c.B = s.B; c.N = s.N; c.H = s.H; c.M = s.M; c.cu = cu_seqlens;
    c.fx = s.D; c.fz = s.E;
    c.ld_act = (flags & LA_FLAG_LD_LOGSIGMOID) ? 1 : 0;
    return launch_chunk_pass(c, dtype, st);
  }
  return scan_forward(s, q, k, v, ld, ld_sb, ld_sn, ld_sh, nullptr, nullptr, initial_state, o,
                      final_state, dtype, st, nullptr, (flags & LA_FLAG_LD_LOGSIGMOID) ? 1 : 0);
}

// Workspace layout: [recomputed final state, rounded up to 16 bytes][row dots of q.dq][row dots of
// k.dk].  The state comes first so that it is 16-byte aligned whatever B*N*H is (the chunk
// kernel writes it with 128-bit stores).
static int64_t lasd_ws_state_floats(int64_t nb, int64_t H, int64_t D, int64_t E) {
  return (nb * H * D * E + 3) / 4 * 4;
}

int64_t la_lasd_bwd_workspace_bytes(int64_t B, int64_t N, int64_t H, int64_t D, int64_t E,
                                    int64_t M, int want_dld) {
  if (!want_dld) return 0;
  const int64_t nb = M > 0 ? M : B;
  const int nt = scan_row_tiles((int)D, (int)E, (int)H, (int)nb);
  return (lasd_ws_state_floats(nb, H, D, E) + (int64_t)2 * nt * B * N * H) * (int64_t)sizeof(float);
}

// no_scratch: the chunk passes may not take hand-off scratch from the library's pool
static int lasd_bwd_impl(const void *q, const void *k, const void *v, const float *ld, int64_t ld_sb,
                         int64_t ld_sn, int64_t ld_sh, const float *initial_state, const void *d_o,
                         const float *dfinal_state, const int64_t *cu_seqlens, void *dq, void *dk,
                         void *dv, float *dld, float *dinitial_state, void *workspace,
                         int64_t workspace_bytes, int64_t B, int64_t N, int64_t H, int64_t D, int64_t E,
                         int64_t M, int dtype, unsigned flags, void *stream, int no_scratch) {
  int rc = check_common(q, k, v, B, N, H, D, E, M, cu_seqlens, dtype);
  if (rc != LA_OK) return rc;
  if (d_o == nullptr || dq == nullptr || dk == nullptr || dv == nullptr || ld == nullptr)
    return LA_ERR_NULL_POINTER;
  if (flags & LA_FLAG_LD_16BIT) return LA_ERR_UNSUPPORTED;  // the scalar decay is always fp32
  const int path = la_lasd_path(N, D, E, dtype, flags);
  if (path < 0) return path;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Seq s{(int)B, (int)N, (int)H, (int)D, (int)E, (int)M, cu_seqlens};
  const bool want_dld = dld != nullptr;
  const int64_t bnh = B * N * H;
  const int nt = path == 1 ? 1 : scan_row_tiles(s.D, s.E, s.H, s.nb());
  float *slots_q = nullptr, *slots_k = nullptr, *ws_state = nullptr;
  if (want_dld) {
    if (workspace == nullptr ||
        workspace_bytes < la_lasd_bwd_workspace_bytes(B, N, H, D, E, M, 1))
      return LA_ERR_WORKSPACE;
    if (reinterpret_cast<uintptr_t>(workspace) & 15u) return LA_ERR_MISALIGNED;
    ws_state = static_cast<float *>(workspace);
    slots_q = ws_state + lasd_ws_state_floats(s.nb(), H, D, E);
    slots_k = slots_q + (int64_t)nt * bnh;
  }
  const bool state_term = want_dld && dfinal_state != nullptr;
  const int ld_act = (flags & LA_FLAG_LD_LOGSIGMOID) ? 1 : 0;

  if (path == 1) {
    ChunkPass c;
    c.ld_act = ld_act;
    c.ld = ld; c.ld_sb = ld_sb; c.ld_sn = ld_sn; c.ld_sh = ld_sh;
    c.B = s.B; c.N = s.N; c.H = s.H; c.M = s.M; c.cu = cu_seqlens; c.no_scratch = no_scratch;
    // dq: (X,Y,Z) = (do, v, k), state S^T, forward direction
    c.x = d_o; c.y = v; c.z = k; c.out = dq; c.t0 = initial_state; c.state_transposed = 1;
    c.fx = s.E; c.fz = s.D;
    c.tfinal = state_term ? ws_state : nullptr; c.reverse = 0;
    c.xrow = want_dld ? q : nullptr; c.rowdot = slots_q;
    // With few (sequence, head) pairs the dq pass runs beside the merged dk/dv launch.
    SideStream *side = (!no_scratch && 3 * (int64_t)s.nb() * s.H <= sm_count() + sm_count() / 2) ? side_stream() : nullptr;
    std::unique_lock<std::mutex> side_lock;
    if (side != nullptr) {
      side_lock = std::unique_lock<std::mutex>(side->mu);
      if (!side_fork(side, st)) return LA_ERR_CUDA;
      rc = launch_chunk_pass(c, dtype, side->stream);
      if (rc != LA_OK) { side_join(side, st); return rc; }
    } else if ((rc = launch_chunk_pass(c, dtype, st)) != LA_OK) {
      return rc;
    }
    // dk: (v, do, q), state dS^T, reverse direction
    c.x = v; c.y = d_o; c.z = q; c.out = dk; c.t0 = dfinal_state; c.state_transposed = 1;
    c.tfinal = nullptr; c.reverse = 1;
    c.xrow = want_dld ? k : nullptr; c.rowdot = slots_k;
    // dv: (k, q, do), state dS, reverse direction; its end state is d initial_state.  Both walk
    // the tokens last to first and both read q and do: one launch, neighbouring CTAs.
    ChunkPass c2 = c;
    c2.x = k; c2.y = q; c2.z = d_o; c2.out = dv; c2.t0 = dfinal_state; c2.state_transposed = 0;
    c2.fx = s.D; c2.fz = s.E;
    c2.tfinal = dinitial_state; c2.reverse = 1; c2.xrow = nullptr; c2.rowdot = nullptr;
    rc = launch_chunk_pass_pair(c, c2, dtype, st);
    if (side != nullptr) {
      if (!side_join(side, st) && rc == LA_OK) rc = LA_ERR_CUDA;
      side_lock.unlock();
    }
    if (rc != LA_OK) return rc;
  } else {
    // dq: T = S (rows D): a = k, b = v, w = do
    ScanParams p = base_params(s, ld, ld_sb, ld_sn, ld_sh);
    p.ld_act = ld_act;
    rows_d(p, s, nullptr, nullptr);
    p.a = k; p.b = v; p.w = d_o; p.out = dq; p.t0 = initial_state;
    p.tfinal = state_term ? ws_state : nullptr;
    if (want_dld) { p.x = q; p.xout = slots_q; p.xmode = 1; }
    if ((rc = launch_scan(p, dtype, st)) != LA_OK) return rc;
    // dk: T = dS (rows D), reverse: a = q, b = do, w = v
    p = base_params(s, ld, ld_sb, ld_sn, ld_sh);
    p.ld_act = ld_act;
    rows_d(p, s, nullptr, nullptr);
    p.reverse = 1;
    p.a = q; p.b = d_o; p.w = v; p.out = dk; p.t0 = dfinal_state; p.tfinal = dinitial_state;
    if (want_dld) { p.x = k; p.xout = slots_k; p.xmode = 1; }
    if ((rc = launch_scan(p, dtype, st)) != LA_OK) return rc;
    // dv: T = dS^T (rows E), reverse: a = do, b = q, w = k
    p = base_params(s, ld, ld_sb, ld_sn, ld_sh);
    p.ld_act = ld_act;
    rows_e(p, s, nullptr, nullptr);
    p.reverse = 1;
    p.a = d_o; p.b = q; p.w = k; p.out = dv; p.t0 = dfinal_state;
    if ((rc = launch_scan(p, dtype, st)) != LA_OK) return rc;
  }
  if (want_dld) {
    rc = launch_dld_scalar(slots_q, nt, slots_k, nt, state_term ? ws_state : nullptr,
                           dfinal_state, cu_seqlens, dld, s.B, s.N, s.H, s.D * s.E, s.M, st,
                           ld_act ? ld : nullptr, ld_sb, ld_sn, ld_sh);
    if (rc != LA_OK) return rc;
  }
  return LA_OK;
}

int la_lasd_bwd(const void *q, const void *k, const void *v, const float *ld, int64_t ld_sb,
                int64_t ld_sn, int64_t ld_sh, const float *initial_state, const void *d_o,
                const float *dfinal_state, const int64_t *cu_seqlens, void *dq, void *dk,
                void *dv, float *dld, float *dinitial_state, void *workspace,
                int64_t workspace_bytes, int64_t B, int64_t N, int64_t H, int64_t D, int64_t E,
                int64_t M, int dtype, unsigned flags, void *stream) {
  return lasd_bwd_impl(q, k, v, ld, ld_sb, ld_sn, ld_sh, initial_state, d_o, dfinal_state, cu_seqlens, dq, dk,
                       dv, dld, dinitial_state, workspace, workspace_bytes, B, N, H, D, E, M, dtype, flags,
                       stream, 0);
}

// ------------------------------------------------------------------------------------------------
// la_lasd_bwd without caller scratch
// ------------------------------------------------------------------------------------------------
// Scratch that lives in the library image: one copy per GPU that loads the library, held until
// the process exits.  Host code may not use the array's name as a pointer (on the host the name
// is only a handle for the runtime); the device address is looked up once per device below.
static __device__ __align__(256) unsigned char g_noalloc_scratch[LA_NOALLOC_SCRATCH_BYTES];

static void *noalloc_scratch_ptr() {
  static void *ptrs[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (ptrs[dev] == nullptr) {
    void *p = nullptr;
    if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess) return nullptr;
    ptrs[dev] = p;
  }
  return ptrs[dev];
}

int la_lasd_bwd_noalloc(const void *q, const void *k, const void *v, const float *ld, int64_t ld_sb,
                        int64_t ld_sn, int64_t ld_sh, const float *initial_state, const void *d_o,
                        const float *dfinal_state, const int64_t *cu_seqlens, void *dq, void *dk,
                        void *dv, float *dld, float *dinitial_state, int64_t B, int64_t N, int64_t H,
                        int64_t D, int64_t E, int64_t M, int dtype, unsigned flags, void *stream) {
  const int rc = check_common(q, k, v, B, N, H, D, E, M, cu_seqlens, dtype);
  if (rc != LA_OK) return rc;
  const int64_t need = la_lasd_bwd_workspace_bytes(B, N, H, D, E, M, dld != nullptr);
  if (need > (int64_t)LA_NOALLOC_SCRATCH_BYTES) return LA_ERR_TOO_LARGE;
  void *scratch = noalloc_scratch_ptr();
  if (scratch == nullptr) return LA_ERR_CUDA;
  // Nothing in the scratch has to start at zero: the row-dot slots and the recomputed final state
  // are written in full by the dq / dk passes of this call before the reduction reads them.
  return lasd_bwd_impl(q, k, v, ld, ld_sb, ld_sn, ld_sh, initial_state, d_o, dfinal_state, cu_seqlens, dq,
                       dk, dv, dld, dinitial_state, scratch, (int64_t)LA_NOALLOC_SCRATCH_BYTES, B, N, H, D, E,
                       M, dtype, flags, stream, 1);
}

// ------------------------------------------------------------------------------------------------
// vector decay
// ------------------------------------------------------------------------------------------------
int la_lavd_path(int64_t N, int64_t D, int64_t E, int dtype, int has_ldk, int has_ldv, unsigned flags) {
  if (!dtype_ok(dtype)) return LA_ERR_UNSUPPORTED;
  const bool tensor = !(flags & LA_FLAG_FORCE_RECURRENCE) &&
                      lavd_chunk_supported(N, D, E, dtype, has_ldk != 0, has_ldv != 0);
  if (!tensor && (flags & LA_FLAG_REQUIRE_TENSOR)) return LA_ERR_UNSUPPORTED;
  return tensor ? 1 : 0;
}

int la_lavd_fwd(const void *q, const void *k, const void *v, const float *ldk, const float *ldv,
                const float *initial_state, const int64_t *cu_seqlens, void *o,
                float *final_state, int64_t B, int64_t N, int64_t H, int64_t D, int64_t E,
                int64_t M, int dtype, unsigned flags, void *stream) {
  int rc = check_common(q, k, v, B, N, H, D, E, M, cu_seqlens, dtype);
  if (rc != LA_OK) return rc;
  if (o == nullptr || (ldk == nullptr && ldv == nullptr)) return LA_ERR_NULL_POINTER;
  const int ld16 = (flags & LA_FLAG_LD_16BIT) ? 1 : 0;
  if (ld16 && dtype == LA_F32) return LA_ERR_UNSUPPORTED;  // the decays take the 16-bit type of q, k, v
  const int path = la_lavd_path(N, D, E, dtype, ldk != nullptr, ldv != nullptr, flags);
  if (path < 0) return path;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Seq s{(int)B, (int)N, (int)H, (int)D, (int)E, (int)M, cu_seqlens};
  const int *enable = nullptr;
  if (path == 1) {
    int *unsafe = lavd_unsafe_ptr();
    if (unsafe == nullptr) return LA_ERR_CUDA;
    if (cudaMemsetAsync(unsafe, 0, 2 * sizeof(int), st) != cudaSuccess) return LA_ERR_CUDA;
    LavdPass c;
    c.x = q; c.y = k; c.z = v; c.ldk = ldk; c.out = o; c.t0 = initial_state; c.tfinal = final_state;
    if (ldk == nullptr) {
      // decay on the value features: o_i[e] = sum_j (q_i . k_j) exp(cv_i[e] - cv_j[e]) v_j[e] has the
      // shape of the dq pass of the key-decay case (decay on the features of Z and of the output),
      // with the state in its natural layout
      c.ldk = ldv; c.tmode = 1; c.state_transposed = 0;
    }
    c.B = s.B; c.N = s.N; c.H = s.H; c.M = s.M; c.cu = cu_seqlens; c.unsafe = unsafe;
    c.ld_act = (flags & LA_FLAG_LD_LOGSIGMOID) ? 1 : 0;
    c.ld16 = ld16;
    if ((rc = launch_lavd_pass(c, dtype, st)) != LA_OK) return rc;
    // the two-reference kernels run only if a chunk left the one-reference range ...
    c.ref2 = 1; c.enable = unsafe; c.unsafe = unsafe + 1;
    if ((rc = launch_lavd_pass(c, dtype, st)) != LA_OK) return rc;
    enable = unsafe + 1;  // ... and the scan below only if one left theirs too
  }
  return scan_forward(s, q, k, v, nullptr, 0, 0, 0, ldk, ldv, initial_state, o, final_state, dtype, st,
                      enable, (flags & LA_FLAG_LD_LOGSIGMOID) ? 1 : 0, ld16);
}

int64_t la_lavd_bwd_workspace_bytes(int64_t B, int64_t N, int64_t H, int64_t D, int64_t E,
                                    int64_t M) {
  (void)N;
  const int64_t nb = M > 0 ? M : B;
  return nb * H * D * E * (int64_t)sizeof(float);
}

int la_lavd_bwd(const void *q, const void *k, const void *v, const float *ldk, const float *ldv,
                const float *initial_state, const void *d_o, const float *dfinal_state,
                const int64_t *cu_seqlens, void *dq, void *dk, void *dv, float *dldk, float *dldv,
                float *dinitial_state, void *workspace, int64_t workspace_bytes, int64_t B,
                int64_t N, int64_t H, int64_t D, int64_t E, int64_t M, int dtype, unsigned flags,
                void *stream) {
  int rc = check_common(q, k, v, B, N, H, D, E, M, cu_seqlens, dtype);
  if (rc != LA_OK) return rc;
  if (d_o == nullptr || dq == nullptr || dk == nullptr || dv == nullptr) return LA_ERR_NULL_POINTER;
  if (ldk == nullptr && ldv == nullptr) return LA_ERR_NULL_POINTER;
  if ((ldk != nullptr && dldk == nullptr) || (ldv != nullptr && dldv == nullptr)) return LA_ERR_NULL_POINTER;
  const int ld16 = (flags & LA_FLAG_LD_16BIT) ? 1 : 0;
  if (ld16 && dtype == LA_F32) return LA_ERR_UNSUPPORTED;  // the decays take the 16-bit type of q, k, v
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Seq s{(int)B, (int)N, (int)H, (int)D, (int)E, (int)M, cu_seqlens};
  float *ws_state = nullptr;
  if (dfinal_state != nullptr) {
    if (workspace == nullptr || workspace_bytes < la_lavd_bwd_workspace_bytes(B, N, H, D, E, M))
      return LA_ERR_WORKSPACE;
    ws_state = static_cast<float *>(workspace);
  }
  const int path = la_lavd_path(N, D, E, dtype, ldk != nullptr, ldv != nullptr, flags);
  if (path < 0) return path;
  const int *enable = nullptr;
  if (path == 1) {
    int *unsafe = lavd_unsafe_ptr();
    if (unsafe == nullptr) return LA_ERR_CUDA;
    if (cudaMemsetAsync(unsafe, 0, 2 * sizeof(int), st) != cudaSuccess) return LA_ERR_CUDA;
    LavdPass c;
    c.ld_act = (flags & LA_FLAG_LD_LOGSIGMOID) ? 1 : 0;
    c.ld16 = ld16;
    c.ldk = ldk; c.B = s.B; c.N = s.N; c.H = s.H; c.M = s.M; c.cu = cu_seqlens; c.unsafe = unsafe;
    if (ldk == nullptr) {
      // Decay on the value features (ldv only): the four passes exchange roles with the key-decay
      // case.  The decay now sits on the features of v, do, o and dv, so
      //   o  (recomputed for the term o * do of dldv) and dv are T-mode passes (decay on Z and on
      //      the output), the state in its natural layout;
      //   dq and dk are N-mode passes (decay on the contraction of X Y^T), the state transposed.
      // All on the caller's stream, in an order that lets the recomputed o use the dv buffer as its
      // scratch output before the dv pass overwrites it.
      c.ldk = ldv;
      LavdPass po = c;  // o again: (q, k, v), forward; dldv = o * do; its end state feeds the state term
      po.x = q; po.y = k; po.z = v; po.out = dv; po.tmode = 1; po.state_transposed = 0; po.reverse = 0;
      po.t0 = initial_state; po.tfinal = ws_state; po.xrow = d_o; po.dld = dldv; po.dld_sub = 0;
      LavdPass pv = po;  // dv: (k, q, do), reverse; dldv -= v * dv; its end state is d initial_state
      pv.x = k; pv.y = q; pv.z = d_o; pv.out = dv; pv.reverse = 1;
      pv.t0 = dfinal_state; pv.tfinal = dinitial_state; pv.xrow = v; pv.dld_sub = 1;
      LavdPass pq = c;   // dq: (do, v, k), forward, state S^T
      pq.x = d_o; pq.y = v; pq.z = k; pq.out = dq; pq.tmode = 0; pq.state_transposed = 1; pq.reverse = 0;
      pq.t0 = initial_state; pq.tfinal = nullptr; pq.xrow = nullptr; pq.dld = nullptr;
      LavdPass pk = pq;  // dk: (v, do, q), reverse, state dS^T
      pk.x = v; pk.y = d_o; pk.z = q; pk.out = dk; pk.reverse = 1; pk.t0 = dfinal_state;
      const LavdPass *order[4] = {&po, &pv, &pq, &pk};
      for (int level = 0; level < 2 && rc == LA_OK; ++level)
        for (int i = 0; i < 4 && rc == LA_OK; ++i) {
          LavdPass x = *order[i];
          if (level == 1) { x.ref2 = 1; x.enable = unsafe; x.unsafe = unsafe + 1; }
          rc = launch_lavd_pass(x, dtype, st);
        }
      if (rc != LA_OK) return rc;
      enable = unsafe + 1;
    } else {
    // dv: (k, q, do), state dS, reverse; its end state is d initial_state.  It shares nothing
    // with the other two passes, so while one CTA per (sequence, head) leaves SMs idle it runs
    // beside them on a side stream.
    LavdPass cv = c;
    cv.x = k; cv.y = q; cv.z = d_o; cv.out = dv; cv.tmode = 0; cv.state_transposed = 0; cv.reverse = 1;
    cv.t0 = dfinal_state; cv.tfinal = dinitial_state; cv.xrow = nullptr; cv.dld = nullptr;
    // dq: (do, v, k), state S^T, forward; dldk = q * dq
    LavdPass cq = c;
    cq.x = d_o; cq.y = v; cq.z = k; cq.out = dq; cq.tmode = 1; cq.state_transposed = 1; cq.reverse = 0;
    cq.t0 = initial_state; cq.tfinal = ws_state; cq.xrow = q; cq.dld = dldk; cq.dld_sub = 0;
    // dk: (v, do, q), state dS^T, reverse; dldk -= k * dk
    LavdPass ck = cq;
    ck.x = v; ck.y = d_o; ck.z = q; ck.out = dk; ck.reverse = 1;
    ck.t0 = dfinal_state; ck.tfinal = nullptr; ck.xrow = k; ck.dld_sub = 1;
    const int64_t pairs = (int64_t)s.nb() * s.H;
    SideStream *side = (2 * pairs <= sm_count() + sm_count() / 2) ? side_stream() : nullptr;
    // With room for the dq and dk passes at once (2 x pairs <= SMs) all three run side by side:
    // dq then adds to a zeroed gradient buffer instead of storing into it, so that it and dk may
    // touch a tile in either order.
    const bool all3 = side != nullptr && 2 * pairs <= sm_count();
    // The same three passes with two reference rows per chunk, enqueued behind the first set and
    // run only if that set raised its word: dv beside dq and dk when a side stream is in use, dq
    // before dk (dk subtracts from the terms dq stored).
    auto second_set = [&](cudaStream_t s_v) -> int {
      LavdPass v2 = cv, q2 = cq, k2 = ck;
      v2.ref2 = q2.ref2 = k2.ref2 = 1;
      v2.enable = q2.enable = k2.enable = unsafe;
      v2.unsafe = q2.unsafe = k2.unsafe = unsafe + 1;
      q2.dld_add = k2.dld_add = 0;
      int r2 = launch_lavd_pass(v2, dtype, s_v);
      if (r2 == LA_OK) r2 = launch_lavd_pass(q2, dtype, st);
      if (r2 == LA_OK) r2 = launch_lavd_pass(k2, dtype, st);
      return r2;
    };
    if (side == nullptr) {
      rc = launch_lavd_pass(cq, dtype, st);
      if (rc == LA_OK) rc = launch_lavd_pass(ck, dtype, st);
      if (rc == LA_OK) rc = launch_lavd_pass(cv, dtype, st);
      if (rc == LA_OK) rc = second_set(st);
    } else {
      std::unique_lock<std::mutex> side_lock(side->mu);
      if (all3) {
        cq.dld_add = ck.dld_add = 1;
        if (cudaMemsetAsync(dldk, 0, (size_t)B * N * H * D * sizeof(float), st) != cudaSuccess) return LA_ERR_CUDA;
      }
      if (!side_fork(side, st) || (all3 && !side_fork2(side))) return LA_ERR_CUDA;
      if (all3) {
        rc = launch_lavd_pass(cq, dtype, side->stream);
        if (rc == LA_OK) rc = launch_lavd_pass(ck, dtype, st);
        if (rc == LA_OK) rc = launch_lavd_pass(cv, dtype, side->stream2);
        if (!side_join2(side, st) && rc == LA_OK) rc = LA_ERR_CUDA;
      } else {
        rc = launch_lavd_pass(cv, dtype, side->stream);
        if (rc == LA_OK) rc = launch_lavd_pass(cq, dtype, st);
        if (rc == LA_OK) rc = launch_lavd_pass(ck, dtype, st);
      }
      if (!side_join(side, st) && rc == LA_OK) rc = LA_ERR_CUDA;
      if (rc == LA_OK) {  // second set: fork again, dv on the side stream
        if (!side_fork(side, st)) return LA_ERR_CUDA;
        rc = second_set(side->stream);
        if (!side_join(side, st) && rc == LA_OK) rc = LA_ERR_CUDA;
      }
    }
    if (rc != LA_OK) return rc;
    enable = unsafe + 1;
    }  // key decay
  }
  ScanParams p;
  const int ld_act = (flags & LA_FLAG_LD_LOGSIGMOID) ? 1 : 0;
  if (ldv != nullptr) {
    // recompute o only to form o*do for dldv (the reference's optional dldv_o pass,
    // vector_decay/lavd_parallel_triton.py:1104-1127)
    p = base_params(s, nullptr, 0, 0, 0);
    p.enable = enable;
    p.ld_act = ld_act;
    p.ld16 = ld16;
    rows_e(p, s, ldk, ldv);
    p.a = v; p.b = k; p.w = q; p.out = nullptr; p.t0 = initial_state;
    p.x = d_o; p.xout = dldv; p.xmode = 2;
    if ((rc = launch_scan(p, dtype, st)) != LA_OK) return rc;
  }
  // dq
  p = base_params(s, nullptr, 0, 0, 0);
  p.enable = enable;
  p.ld_act = ld_act;
  p.ld16 = ld16;
  rows_d(p, s, ldk, ldv);
  p.a = k; p.b = v; p.w = d_o; p.out = dq; p.t0 = initial_state; p.tfinal = ws_state;
  if (ldk != nullptr) { p.x = q; p.xout = dldk; p.xmode = 2; }
  if ((rc = launch_scan(p, dtype, st)) != LA_OK) return rc;
  // dk
  p = base_params(s, nullptr, 0, 0, 0);
  p.enable = enable;
  p.ld_act = ld_act;
  p.ld16 = ld16;
  rows_d(p, s, ldk, ldv);
  p.reverse = 1;
  p.a = q; p.b = d_o; p.w = v; p.out = dk; p.t0 = dfinal_state; p.tfinal = dinitial_state;
  if (ldk != nullptr) { p.x = k; p.xout = dldk; p.xmode = 3; }
  if ((rc = launch_scan(p, dtype, st)) != LA_OK) return rc;
  // dv
  p = base_params(s, nullptr, 0, 0, 0);
  p.enable = enable;
  p.ld_act = ld_act;
  p.ld16 = ld16;
  rows_e(p, s, ldk, ldv);
  p.reverse = 1;
  p.a = d_o; p.b = q; p.w = k; p.out = dv; p.t0 = dfinal_state;
  if (ldv != nullptr) { p.x = v; p.xout = dldv; p.xmode = 3; }
  if ((rc = launch_scan(p, dtype, st)) != LA_OK) return rc;
  if (ldk != nullptr) {
    rc = launch_revcumsum_vec(dldk, ws_state, dfinal_state, cu_seqlens, s.B, s.N, s.H, s.D, s.D,
                              s.E, 1, s.M, st, ld_act ? ldk : nullptr, ld16 ? dtype : LA_F32);
    if (rc != LA_OK) return rc;
  }
  if (ldv != nullptr) {
    rc = launch_revcumsum_vec(dldv, ws_state, dfinal_state, cu_seqlens, s.B, s.N, s.H, s.E, s.D,
                              s.E, 0, s.M, st, ld_act ? ldv : nullptr, ld16 ? dtype : LA_F32);
    if (rc != LA_OK) return rc;
  }
  return LA_OK;
}

// ------------------------------------------------------------------------------------------------
// sequence-parallel correction
// ------------------------------------------------------------------------------------------------
int la_seqpar_correct(const void *q, void *o, const float *cum, const float *s_in, int64_t T1,
                      int64_t N, int64_t H, int64_t D, int64_t E, int dtype, void *stream) {
  if (q == nullptr || o == nullptr || cum == nullptr || s_in == nullptr) return LA_ERR_NULL_POINTER;
  if (T1 < 0 || T1 > N || N <= 0 || H <= 0 || D <= 0 || E <= 0) return LA_ERR_BAD_SHAPE;
  if (!dtype_ok(dtype)) return LA_ERR_UNSUPPORTED;
  if (N > (int64_t)1 << 30 || H > 65535) return LA_ERR_TOO_LARGE;
  return launch_seqpar_correct(q, o, cum, s_in, (int)T1, (int)N, (int)H, (int)D, (int)E, dtype,
                               static_cast<cudaStream_t>(stream));
}

int la_seqpar_fold_segments(float *states, const float *seg_decay, const int32_t *seg_table, float *s_in,
                            int64_t nseg, int64_t H, int64_t D, int64_t E, void *stream) {
  if (states == nullptr || seg_decay == nullptr || seg_table == nullptr || s_in == nullptr) return LA_ERR_NULL_POINTER;
  if (nseg <= 0 || H <= 0 || D <= 0 || E <= 0) return LA_ERR_BAD_SHAPE;
  if (nseg > 65535 || H * D * E > 0x7fffffff) return LA_ERR_TOO_LARGE;
  return launch_seqpar_fold_segments(states, seg_decay, seg_table, s_in, (int)nseg, (int)H, (int)(D * E),
                                     static_cast<cudaStream_t>(stream));
}

int la_seqpar_correct_multi(const void *q, void *o, const float *cum, const float *s_in, const int32_t *seg_table,
                            int64_t nseg, int64_t total_tiles, int64_t N, int64_t H, int64_t D, int64_t E, int dtype,
                            void *stream) {
  if (q == nullptr || o == nullptr || cum == nullptr || s_in == nullptr || seg_table == nullptr)
    return LA_ERR_NULL_POINTER;
  if (nseg < 0 || total_tiles < 0 || N <= 0 || H <= 0) return LA_ERR_BAD_SHAPE;
  if (D != 128 || E != 128 || N < 128 || !(dtype == LA_BF16 || dtype == LA_F16)) return LA_ERR_UNSUPPORTED;
  if (N > (int64_t)1 << 30 || H > 65535 || total_tiles > 0x7fffffff || nseg > 65535) return LA_ERR_TOO_LARGE;
  return launch_seqpar_correct_multi(q, o, cum, s_in, seg_table, (int)nseg, (int)total_tiles, (int)N, (int)H, dtype,
                                     static_cast<cudaStream_t>(stream));
}

int la_lasd_state_pass(const void *y, const void *z, const float *ld, int64_t ld_sb, int64_t ld_sn, int64_t ld_sh,
                       const int64_t *cu_seqlens, float *states, float *gsum, int64_t B, int64_t N, int64_t H,
                       int64_t D, int64_t E, int64_t M, int dtype, int reverse, int ranges, unsigned flags,
                       void *stream) {
  int rc = check_common(y, z, y, B, N, H, D, E, M, cu_seqlens, dtype);
  if (rc == LA_OK && ranges != 0 && cu_seqlens == nullptr) rc = LA_ERR_NULL_POINTER;
  if (rc != LA_OK) return rc;
  if (ld == nullptr || states == nullptr) return LA_ERR_NULL_POINTER;
  if (D != 128 || E != 128 || !(dtype == LA_BF16 || dtype == LA_F16)) return LA_ERR_UNSUPPORTED;
  if (flags & LA_FLAG_LD_16BIT) return LA_ERR_UNSUPPORTED;  // the scalar decay is always fp32
  StatePass p;
  p.y = y; p.z = z; p.ld = ld; p.ld_sb = ld_sb; p.ld_sn = ld_sn; p.ld_sh = ld_sh; p.cu = cu_seqlens;
  p.states = states; p.gsum = gsum; p.B = (int)B; p.N = (int)N; p.H = (int)H; p.M = (int)M; p.reverse = reverse != 0;
  p.ranges = ranges != 0;
  p.ld_act = (flags & LA_FLAG_LD_LOGSIGMOID) ? 1 : 0;
  return launch_state_pass(p, dtype, static_cast<cudaStream_t>(stream));
}

int la_lasd_fold_states(const float *local, const float *gsum, const int32_t *seg_table, const int32_t *emit,
                        const float *ext, float *incoming, float *ends, int64_t nseg, int64_t H, int64_t D, int64_t E, int reverse,
                        void *stream) {
  if (local == nullptr || gsum == nullptr || seg_table == nullptr) return LA_ERR_NULL_POINTER;
  if (incoming == nullptr && ends == nullptr) return LA_ERR_NULL_POINTER;  // at least one output
  if (nseg <= 0 || H <= 0 || D <= 0 || E <= 0) return LA_ERR_BAD_SHAPE;
  if (nseg > 65535 || H * D * E > 0x7fffffff) return LA_ERR_TOO_LARGE;
  return launch_fold_states(local, gsum, seg_table, emit, ext, incoming, ends, (int)nseg, (int)H, (int)(D * E),
                            reverse != 0, static_cast<cudaStream_t>(stream));
}

int la_lavd_state_pass(const void *y, const void *z, const float *ldk, const int64_t *cu_seqlens, float *states,
                       float *gsum, int64_t B, int64_t N, int64_t H, int64_t D, int64_t E, int64_t M, int dtype,
                       int reverse, int ranges, unsigned flags, void *stream) {
  int rc = check_common(y, z, y, B, N, H, D, E, M, cu_seqlens, dtype);
  if (rc == LA_OK && ranges != 0 && cu_seqlens == nullptr) rc = LA_ERR_NULL_POINTER;
  if (rc != LA_OK) return rc;
  if (ldk == nullptr || states == nullptr) return LA_ERR_NULL_POINTER;
  if (D != 128 || E != 128 || !(dtype == LA_BF16 || dtype == LA_F16)) return LA_ERR_UNSUPPORTED;
  StatePass p;
  p.y = y; p.z = z; p.ldv = ldk; p.cu = cu_seqlens; p.states = states; p.gsum = gsum;
  p.B = (int)B; p.N = (int)N; p.H = (int)H; p.M = (int)M; p.reverse = reverse != 0; p.ranges = ranges != 0;
  p.ld_act = (flags & LA_FLAG_LD_LOGSIGMOID) ? 1 : 0;
  p.ld16 = (flags & LA_FLAG_LD_16BIT) ? 1 : 0;
  return launch_state_pass_vec(p, dtype, static_cast<cudaStream_t>(stream));
}

int la_lavd_fold_states(const float *local, const float *gsum, const int32_t *seg_table, const int32_t *emit,
                        const float *ext, float *incoming, int64_t nseg, int64_t H, int64_t D, int64_t E, int reverse,
                        void *stream) {
  if (local == nullptr || gsum == nullptr || seg_table == nullptr || incoming == nullptr) return LA_ERR_NULL_POINTER;
  if (nseg <= 0 || H <= 0 || D <= 0 || E <= 0) return LA_ERR_BAD_SHAPE;
  if (nseg > 65535 || H * D * E > 0x7fffffff) return LA_ERR_TOO_LARGE;
  return launch_fold_states_vec(local, gsum, seg_table, emit, ext, incoming, (int)nseg, (int)H, (int)D, (int)E,
                                reverse != 0, static_cast<cudaStream_t>(stream));
}

int la_seqpar_fold(const float *gathered, float *s_in, int64_t rank, int64_t H, int64_t D, int64_t E,
                   void *stream) {
  if (gathered == nullptr || s_in == nullptr) return LA_ERR_NULL_POINTER;
  if (rank < 0 || H <= 0 || D <= 0 || E <= 0) return LA_ERR_BAD_SHAPE;
  if (rank > 4096 || H * D * E > 0x7fffffff) return LA_ERR_TOO_LARGE;
  return launch_seqpar_fold(gathered, s_in, (int)rank, (int)H, (int)(D * E), static_cast<cudaStream_t>(stream));
}

// ------------------------------------------------------------------------------------------------
// decode
// ------------------------------------------------------------------------------------------------
static int decode_common(const void *q, const void *k, const void *v, const float *ld,
                         int64_t ld_sb, int64_t ld_sh, const float *ldk, const float *ldv,
                         const float *state_in, float *state_out, void *o, int64_t B, int64_t H,
                         int64_t D, int64_t E, int dtype, void *stream) {
  int rc = check_common(q, k, v, B, 1, H, D, E, 0, nullptr, dtype);
  if (rc != LA_OK) return rc;
  if (state_in == nullptr || state_out == nullptr || o == nullptr) return LA_ERR_NULL_POINTER;
  if (B * H > 0x7fffffff) return LA_ERR_TOO_LARGE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  rc = launch_decode(q, k, v, ld, ld_sb, ld_sh, ldk, ldv, state_in, state_out, o, (int)B, (int)H,
                     (int)D, (int)E, dtype, st);
  if (rc != LA_ERR_UNSUPPORTED && rc != LA_ERR_MISALIGNED) return rc;
  // shapes the vectorised kernel does not take: same update through the scan kernel (N = 1);
  // it cannot run in place because tiles of one (b,h) live in different CTAs.
  if (state_in == state_out) return rc;
  Seq s{(int)B, 1, (int)H, (int)D, (int)E, 0, nullptr};
  return scan_forward(s, q, k, v, ld, ld_sb, 0, ld_sh, ldk, ldv, state_in, o, state_out, dtype, st);
}

int la_decode_scalar(const void *q, const void *k, const void *v, const float *ld, int64_t ld_sb,
                     int64_t ld_sh, const float *state_in, float *state_out, void *o, int64_t B,
                     int64_t H, int64_t D, int64_t E, int dtype, void *stream) {
  if (ld == nullptr) return LA_ERR_NULL_POINTER;
  return decode_common(q, k, v, ld, ld_sb, ld_sh, nullptr, nullptr, state_in, state_out, o, B, H, D,
                       E, dtype, stream);
}

int la_decode_vector(const void *q, const void *k, const void *v, const float *ldk,
                     const float *ldv, const float *state_in, float *state_out, void *o,
                     int64_t B, int64_t H, int64_t D, int64_t E, int dtype, void *stream) {
  if (ldk == nullptr && ldv == nullptr) return LA_ERR_NULL_POINTER;
  return decode_common(q, k, v, nullptr, 0, 0, ldk, ldv, state_in, state_out, o, B, H, D, E, dtype,
                       stream);
}

}  // extern "C"
