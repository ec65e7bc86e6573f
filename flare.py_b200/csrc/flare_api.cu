// C ABI of flare_b200: argument checks, workspace carving and kernel selection.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include "common.cuh"
#include "launch.h"

using namespace flare;

namespace {

thread_local char g_err[512] = "";
std::atomic<int> g_path{FLARE_PATH_AUTO};
std::atomic<long long> g_tc_passes{0}, g_simt_passes{0};   // passes enqueued on each kernel family (flare_pass_counts)

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

inline size_t esize(int dtype) { return dtype == FLARE_F32 ? 4 : 2; }
inline size_t up256(size_t x) { return (x + 255) & ~size_t(255); }
inline bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

int check_problem(const FlareProblem* p) {
  if (!p) return fail(FLARE_EINVAL, "null problem");
  if (p->B < 1 || p->H < 1 || p->M < 1 || p->N < 0) return fail(FLARE_EINVAL, "bad sizes B=%d H=%d N=%d M=%d", p->B, p->H, p->N, p->M);
  if (p->dtype != FLARE_F32 && p->dtype != FLARE_F16 && p->dtype != FLARE_BF16) return fail(FLARE_EINVAL, "bad dtype %d", p->dtype);
  if (p->D != 8 && p->D != 16 && p->D != 32 && p->D != 64 && p->D != 128)
    return fail(FLARE_EUNSUPPORTED, "head dim %d not in {8,16,32,64,128}", p->D);
  if (!(p->scale > 0.f)) return fail(FLARE_EINVAL, "scale must be > 0");
  if (p->n_splits < 0) return fail(FLARE_EINVAL, "n_splits < 0");
  if (!(p->dropout_p >= 0.f) || p->dropout_p >= 1.f) return fail(FLARE_EINVAL, "dropout_p must be in [0, 1)");
  if ((long long)p->B * p->H > 65535) return fail(FLARE_EUNSUPPORTED, "B*H > 65535");
  return FLARE_OK;
}

int check_tok(const char* name, const void* ptr, const int64_t* st, int dtype) {
  if (!ptr) return fail(FLARE_EINVAL, "%s is null", name);
  if (!al16(ptr)) return fail(FLARE_EALIGN, "%s pointer not 16-byte aligned", name);
  const size_t e = esize(dtype);
  for (int i = 0; i < 3; ++i)
    if ((st[i] * (int64_t)e) % 16 != 0) return fail(FLARE_EALIGN, "%s stride[%d]=%lld elements is not a multiple of 16 bytes", name, i, (long long)st[i]);
  return FLARE_OK;
}

int auto_splits(const FlareProblem* p) {
  const int tpt = p->D <= 32 ? 1 : p->D / 32;
  const int lpb = 128 / tpt;
  const long long base = (long long)p->B * p->H * ((p->M + lpb - 1) / lpb);
  long long s = (4LL * 148 + base - 1) / base;
  const long long max_s = (p->N + 127) / 128;
  // short ranges (a context-parallel shard, a small N): one wave of CTAs instead of two, so that the
  // per-CTA set-up (resident operands, first tiles) is paid once
  if (max_s / s < 64) s = (2LL * 148) / base > 0 ? (2LL * 148) / base : 1;
  if (s > max_s) s = max_s;
  if (s > 1024) s = 1024;
  if (s < 1) s = 1;
  // ranges are whole multiples of 128 tokens: drop ranges that would be empty
  const long long chunk = (((p->N + s - 1) / s + 127) / 128) * 128;
  if (chunk > 0) s = (p->N + chunk - 1) / chunk;
  if (s < 1) s = 1;
  return (int)s;
}

Ctx make_ctx(const FlareProblem* p, int terms = FLARE_TERM_BOTH) {
  Ctx c;
  c.B = p->B; c.H = p->H; c.N = p->N; c.M = p->M; c.D = p->D;
  c.scale = p->scale;
  c.n_splits = p->n_splits > 0 ? p->n_splits : auto_splits(p);
  const long long per = (p->N + c.n_splits - 1) / c.n_splits;
  c.chunk = (int)(((per + 127) / 128) * 128);
  if (c.chunk < 128) c.chunk = 128;
  c.terms = terms;
  c.drop_p = p->dropout_p;
  c.drop_seed = p->dropout_seed;
  for (int i = 0; i < 3; ++i) {
    c.qs[i] = p->q_stride[i]; c.ks[i] = p->k_stride[i]; c.vs[i] = p->v_stride[i];
    c.ys[i] = p->y_stride[i]; c.dys[i] = p->dy_stride[i]; c.dks[i] = p->dk_stride[i];
    c.dvs[i] = p->dv_stride[i];
  }
  return c;
}

int after_launch(const char* what) {
  cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) return fail(FLARE_ECUDA, "%s: %s", what, cudaGetErrorString(e));
  return FLARE_OK;
}

#define TRY(x) do { int rc_ = (x); if (rc_ != FLARE_OK) return rc_; } while (0)

}  // namespace

namespace flare {
// Lets entry points defined in other files of the library report through flare_last_error().
void set_last_error(const char* msg) { snprintf(g_err, sizeof(g_err), "%s", msg ? msg : ""); }
}  // namespace flare

extern "C" {

int flare_version(void) { return 100; }

const char* flare_last_error(void) { return g_err; }

int flare_set_path(int path) { return g_path.exchange(path); }

int flare_pick_splits(const FlareProblem* p) {
  if (check_problem(p) != FLARE_OK) return 1;
  return p->n_splits > 0 ? p->n_splits : auto_splits(p);
}

size_t flare_fwd_workspace_bytes(const FlareProblem* p) {
  if (check_problem(p) != FLARE_OK) return 0;
  const size_t S = (size_t)flare_pick_splits(p);
  return up256(S * p->B * p->H * p->M * (p->D + 2) * sizeof(float)) + 256;
}

size_t flare_bwd_workspace_bytes(const FlareProblem* p) {
  if (check_problem(p) != FLARE_OK) return 0;
  const size_t S = (size_t)flare_pick_splits(p);
  const size_t part = up256(S * p->B * p->H * p->M * p->D * sizeof(float));
  const size_t dz = up256((size_t)p->B * p->H * p->M * p->D * sizeof(float));
  const size_t del = up256((size_t)p->B * p->H * (size_t)p->N * sizeof(float));
  return part + dz + del + 256;
}

int flare_gather_partial(const FlareProblem* p, const void* q, const void* k, const void* v,
                         const uint8_t* key_mask, float* rec, flare_stream_t stream) {
  TRY(check_problem(p));
  if (p->n_splits < 1) return fail(FLARE_EINVAL, "flare_gather_partial needs n_splits >= 1");
  TRY(check_tok("q", q, p->q_stride, p->dtype));
  TRY(check_tok("k", k, p->k_stride, p->dtype));
  TRY(check_tok("v", v, p->v_stride, p->dtype));
  if (!rec) return fail(FLARE_EINVAL, "rec is null");
  Ctx c = make_ctx(p);
  const bool drop = p->dropout_p > 0.f;
  if (drop && (g_path.load() == FLARE_PATH_SIMT || !tc_lat2_supported(c, p->dtype)))
    return fail(FLARE_EUNSUPPORTED, "attention dropout needs the tensor-core kernels (bf16/fp16, D in {16,32})");
  if (g_path.load() != FLARE_PATH_SIMT && (tc_lat2_supported(c, p->dtype) || (!key_mask && tc_lat_supported(c, p->dtype)))) {
    // head dims 16 and 32: the decoupled-schedule kernel; 64 (bf16, no mask): the first-generation one
    const int rc = tc_lat2_supported(c, p->dtype) ? tc_gather_partial2(c, p->dtype, q, k, v, key_mask, rec, (cudaStream_t)stream)
                                                  : tc_gather_partial(c, q, k, v, rec, (cudaStream_t)stream);
    if (rc == FLARE_OK) { ++g_tc_passes; return after_launch("gather_partial (tcgen05)"); }
    if (rc != FLARE_EUNSUPPORTED) return fail(rc, "gather_partial (tcgen05): launch setup failed");
  }
  ++g_simt_passes;
  TRY(simt_gather_partial(c, p->dtype, q, k, v, key_mask, rec, (cudaStream_t)stream));
  return after_launch("gather_partial");
}

int flare_combine(const FlareProblem* p, const float* rec, int n_parts, float* z32, void* z_out,
                  float* lse_m, float* rec_out, flare_stream_t stream) {
  TRY(check_problem(p));
  if (!rec || n_parts < 1) return fail(FLARE_EINVAL, "combine: rec null or n_parts < 1");
  const long long rows = (long long)p->B * p->H * p->M;
  TRY(launch_combine(rec, n_parts, rows, p->D, p->dtype, z32, z_out, lse_m, rec_out, (cudaStream_t)stream));
  return after_launch("combine");
}

int flare_combine_peers(const FlareProblem* p, const float* const* rec_ptrs, int n_parts, float* z32,
                        void* z_out, float* lse_m, float* rec_out, flare_stream_t stream) {
  TRY(check_problem(p));
  if (!rec_ptrs || n_parts < 1) return fail(FLARE_EINVAL, "combine_peers: rec_ptrs null or n_parts < 1");
  const long long rows = (long long)p->B * p->H * p->M;
  TRY(launch_combine_ptrs(rec_ptrs, n_parts, rows, p->D, p->dtype, z32, z_out, lse_m, rec_out, (cudaStream_t)stream));
  return after_launch("combine_peers");
}

int flare_reduce_sum_peers(const float* const* part_ptrs, int n_parts, int64_t rows, int width, float* out,
                           flare_stream_t stream) {
  if (!part_ptrs || !out || n_parts < 1 || rows < 0 || width < 1) return fail(FLARE_EINVAL, "reduce_sum_peers: bad arguments");
  if (rows == 0) return FLARE_OK;
  TRY(launch_reduce_sum_ptrs(part_ptrs, n_parts, (long long)rows * width, out, (cudaStream_t)stream));
  return after_launch("reduce_sum_peers");
}

int flare_scatter(const FlareProblem* p, const void* q, const void* k, const float* z32,
                  const uint8_t* key_mask, void* y, float* lse_n, flare_stream_t stream) {
  TRY(check_problem(p));
  TRY(check_tok("q", q, p->q_stride, p->dtype));
  TRY(check_tok("k", k, p->k_stride, p->dtype));
  TRY(check_tok("y", y, p->y_stride, p->dtype));
  if (!z32) return fail(FLARE_EINVAL, "z32 is null");
  if (p->N == 0) return FLARE_OK;
  Ctx c = make_ctx(p);
  if (p->dropout_p > 0.f && (g_path.load() == FLARE_PATH_SIMT || !tc_scatter2_supported(c, p->dtype)))
    return fail(FLARE_EUNSUPPORTED, "attention dropout needs the tensor-core kernels (bf16/fp16, D in {16,32}, M a multiple of 32)");
  if (g_path.load() != FLARE_PATH_SIMT && (tc_scatter_supported(c, p->dtype) || tc_scatter2_supported(c, p->dtype))) {
    const int rc = tc_scatter2_supported(c, p->dtype) ? tc_scatter2(c, p->dtype, q, k, z32, key_mask, y, lse_n, (cudaStream_t)stream)
                                                      : tc_scatter(c, q, k, z32, key_mask, y, lse_n, (cudaStream_t)stream);
    if (rc == FLARE_OK) { ++g_tc_passes; return after_launch("scatter (tcgen05)"); }
    if (rc != FLARE_EUNSUPPORTED) return fail(rc, "scatter (tcgen05): launch setup failed");
  }
  ++g_simt_passes;
  TRY(simt_scatter(c, p->dtype, q, k, z32, key_mask, y, lse_n, (cudaStream_t)stream));
  return after_launch("scatter");
}

int flare_bwd_dz_partial(const FlareProblem* p, const void* q, const void* k, const void* dy,
                         const uint8_t* key_mask, const float* lse_n, float* dz_part,
                         flare_stream_t stream) {
  TRY(check_problem(p));
  if (p->n_splits < 1) return fail(FLARE_EINVAL, "flare_bwd_dz_partial needs n_splits >= 1");
  TRY(check_tok("q", q, p->q_stride, p->dtype));
  TRY(check_tok("k", k, p->k_stride, p->dtype));
  TRY(check_tok("dy", dy, p->dy_stride, p->dtype));
  if (!lse_n || !dz_part) return fail(FLARE_EINVAL, "lse_n or dz_part is null");
  Ctx c = make_ctx(p);
  if (p->dropout_p > 0.f && (g_path.load() == FLARE_PATH_SIMT || !tc_lat2_supported(c, p->dtype)))
    return fail(FLARE_EUNSUPPORTED, "attention dropout needs the tensor-core kernels (bf16/fp16, D in {16,32})");
  if (g_path.load() != FLARE_PATH_SIMT && (tc_lat2_supported(c, p->dtype) || (!key_mask && tc_lat_supported(c, p->dtype)))) {
    const int rc = tc_lat2_supported(c, p->dtype)
                       ? tc_dz_partial2(c, p->dtype, q, k, dy, key_mask, lse_n, dz_part, (cudaStream_t)stream)
                       : tc_dz_partial(c, q, k, dy, lse_n, dz_part, (cudaStream_t)stream);
    if (rc == FLARE_OK) { ++g_tc_passes; return after_launch("bwd_dz_partial (tcgen05)"); }
    if (rc != FLARE_EUNSUPPORTED) return fail(rc, "bwd_dz_partial (tcgen05): launch setup failed");
  }
  ++g_simt_passes;
  TRY(simt_dz_partial(c, p->dtype, q, k, dy, key_mask, lse_n, dz_part, (cudaStream_t)stream));
  return after_launch("bwd_dz_partial");
}

int flare_reduce_sum(const float* parts, int n_parts, int64_t rows, int width, float* out,
                     flare_stream_t stream) {
  if (!parts || !out || n_parts < 1 || rows < 0 || width < 1) return fail(FLARE_EINVAL, "reduce_sum: bad arguments");
  if (rows == 0) return FLARE_OK;
  TRY(launch_reduce_sum(parts, n_parts, (long long)rows * width, out, (cudaStream_t)stream));
  return after_launch("reduce_sum");
}

int flare_bwd_tokens(const FlareProblem* p, int terms, const void* q, const void* k, const void* v,
                     const void* dy, const void* y, const uint8_t* key_mask, const float* z32,
                     const float* dz32, const float* lse_m, const float* lse_n, void* dk, void* dv,
                     float* delta_n, flare_stream_t stream) {
  TRY(check_problem(p));
  if (terms < 1 || terms > 3) return fail(FLARE_EINVAL, "terms must be 1, 2 or 3");
  TRY(check_tok("q", q, p->q_stride, p->dtype));
  TRY(check_tok("k", k, p->k_stride, p->dtype));
  TRY(check_tok("dk", dk, p->dk_stride, p->dtype));
  if (!z32) return fail(FLARE_EINVAL, "z32 is null");
  if (terms & FLARE_TERM_GATHER) {
    TRY(check_tok("v", v, p->v_stride, p->dtype));
    TRY(check_tok("dv", dv, p->dv_stride, p->dtype));
    if (!dz32 || !lse_m) return fail(FLARE_EINVAL, "gather term needs dz32 and lse_m");
  }
  if (terms & FLARE_TERM_SCATTER) {
    TRY(check_tok("dy", dy, p->dy_stride, p->dtype));
    TRY(check_tok("y", y, p->y_stride, p->dtype));
    if (!lse_n) return fail(FLARE_EINVAL, "scatter term needs lse_n");
  }
  if (p->N == 0) return FLARE_OK;
  Ctx c = make_ctx(p, terms);
  ++g_simt_passes;
  TRY(simt_bwd_tokens(c, p->dtype, q, k, v, dy, y, key_mask, z32, dz32, lse_m, lse_n, dk, dv, delta_n,
                      (cudaStream_t)stream));
  return after_launch("bwd_tokens");
}

int flare_bwd_dq_partial(const FlareProblem* p, int terms, const void* q, const void* k, const void* v,
                         const void* dy, const uint8_t* key_mask, const float* z32, const float* dz32,
                         const float* lse_m, const float* lse_n, const float* delta_n, float* dq_part,
                         flare_stream_t stream) {
  TRY(check_problem(p));
  if (terms < 1 || terms > 3) return fail(FLARE_EINVAL, "terms must be 1, 2 or 3");
  if (p->n_splits < 1) return fail(FLARE_EINVAL, "flare_bwd_dq_partial needs n_splits >= 1");
  TRY(check_tok("q", q, p->q_stride, p->dtype));
  TRY(check_tok("k", k, p->k_stride, p->dtype));
  if (!z32 || !dq_part) return fail(FLARE_EINVAL, "z32 or dq_part is null");
  if (terms & FLARE_TERM_GATHER) {
    TRY(check_tok("v", v, p->v_stride, p->dtype));
    if (!dz32 || !lse_m) return fail(FLARE_EINVAL, "gather term needs dz32 and lse_m");
  }
  if (terms & FLARE_TERM_SCATTER) {
    TRY(check_tok("dy", dy, p->dy_stride, p->dtype));
    if (!lse_n || !delta_n) return fail(FLARE_EINVAL, "scatter term needs lse_n and delta_n");
  }
  Ctx c = make_ctx(p, terms);
  ++g_simt_passes;
  TRY(simt_dq_partial(c, p->dtype, q, k, v, dy, key_mask, z32, dz32, lse_m, lse_n, delta_n, dq_part,
                      (cudaStream_t)stream));
  return after_launch("bwd_dq_partial");
}

int flare_device_status(int* out, int clear) {
  if (!out) return fail(FLARE_EINVAL, "device_status: out is null");
  const int rc = tc_read_status(out, clear != 0);
  if (rc != FLARE_OK) return fail(rc, "device_status: %s", cudaGetErrorString(cudaGetLastError()));
  return FLARE_OK;
}

int flare_pass_counts(long long* tensor_core, long long* simt) {
  if (tensor_core) *tensor_core = g_tc_passes.load();
  if (simt) *simt = g_simt_passes.load();
  return FLARE_OK;
}

int flare_probe_ex2(int blocks, int iters, float* out, flare_stream_t stream) {
  if (blocks < 1 || iters < 1 || !out) return fail(FLARE_EINVAL, "probe_ex2: bad arguments");
  TRY(launch_probe_ex2(blocks, iters, out, (cudaStream_t)stream));
  return after_launch("probe_ex2");
}

int flare_mixer_fwd(const FlareProblem* p, const void* q, const void* k, const void* v,
                    const uint8_t* key_mask, void* y, float* z32, float* lse_m, float* lse_n,
                    void* workspace, size_t workspace_bytes, flare_stream_t stream) {
  TRY(check_problem(p));
  if (!z32 || !lse_m) return fail(FLARE_EINVAL, "z32 and lse_m are required outputs");
  const size_t need = flare_fwd_workspace_bytes(p);
  if (!workspace || workspace_bytes < need) return fail(FLARE_EWORKSPACE, "forward workspace: have %zu bytes, need %zu", workspace_bytes, need);
  FlareProblem pp = *p;
  pp.n_splits = flare_pick_splits(p);
  float* rec = reinterpret_cast<float*>((reinterpret_cast<uintptr_t>(workspace) + 255) & ~uintptr_t(255));
  TRY(flare_gather_partial(&pp, q, k, v, key_mask, rec, stream));
  TRY(flare_combine(&pp, rec, pp.n_splits, z32, nullptr, lse_m, nullptr, stream));
  TRY(flare_scatter(&pp, q, k, z32, key_mask, y, lse_n, stream));
  return FLARE_OK;
}

int flare_bwd_main(const FlareProblem* p, int terms, const void* q, const void* k, const void* v,
                   const void* dy, const void* y, const uint8_t* key_mask, const float* z32,
                   const float* dz32, const float* lse_m, const float* lse_n, void* dk, void* dv,
                   float* delta_n, float* dq_part, flare_stream_t stream) {
  TRY(check_problem(p));
  if (terms < 1 || terms > 3) return fail(FLARE_EINVAL, "terms must be 1, 2 or 3");
  if (p->n_splits < 1) return fail(FLARE_EINVAL, "flare_bwd_main needs n_splits >= 1");
  if (!dq_part) return fail(FLARE_EINVAL, "dq_part is null");
  Ctx c = make_ctx(p, terms);
  const bool use_g = (terms & FLARE_TERM_GATHER) != 0, use_s = (terms & FLARE_TERM_SCATTER) != 0;
  if (g_path.load() != FLARE_PATH_SIMT && p->N > 0 && tc_bwd_supported(c, p->dtype)) {
    TRY(check_tok("q", q, p->q_stride, p->dtype));
    TRY(check_tok("k", k, p->k_stride, p->dtype));
    TRY(check_tok("dk", dk, p->dk_stride, p->dtype));
    if (!z32) return fail(FLARE_EINVAL, "bwd_main: z32 is null");
    if (use_g) {
      TRY(check_tok("v", v, p->v_stride, p->dtype));
      TRY(check_tok("dv", dv, p->dv_stride, p->dtype));
      if (!dz32 || !lse_m) return fail(FLARE_EINVAL, "bwd_main: the gather term needs dz32 and lse_m");
    }
    if (use_s) {
      TRY(check_tok("dy", dy, p->dy_stride, p->dtype));
      TRY(check_tok("y", y, p->y_stride, p->dtype));
      if (!lse_n) return fail(FLARE_EINVAL, "bwd_main: the scatter term needs lse_n");
    }
    // The one-exponential kernel covers the plain case (bf16, both terms, no mask, D = 32, 32 to 1024
    // latents).  An on-device range check picks, per (b, h), between it (flag 0) and the general
    // two-exponential kernel (flag 1); both are launched and each returns at once on the (b, h) it does
    // not own.  delta_n ([B,H,N] floats) is not needed by the fused kernels and doubles as
    // the scratch of that check.  Everything else goes to the general kernel directly.
    const int* flag = nullptr;
    int rc = FLARE_OK;
    const size_t have = (size_t)p->B * p->H * (size_t)p->N * sizeof(float);
    const bool fast = p->dtype == FLARE_BF16 && terms == FLARE_TERM_BOTH && !key_mask && !(p->dropout_p > 0.f) && g_path.load() != FLARE_PATH_TC_EXACT &&
                      tc_bwd_fast_supported(c, p->dtype) && delta_n && (reinterpret_cast<uintptr_t>(delta_n) & 255) == 0 &&
                      have >= tc_bwd_fast_scratch_bytes(c);
    if (fast)
      rc = tc_bwd_fast_main(c, q, k, v, dy, y, z32, dz32, lse_m, lse_n, dk, dv, dq_part, delta_n, &flag, (cudaStream_t)stream);
    if (rc == FLARE_OK)
      rc = tc_bwd_main(c, p->dtype, q, k, v, dy, y, key_mask, z32, dz32, lse_m, lse_n, dk, dv, dq_part, flag, (cudaStream_t)stream);
    if (rc == FLARE_OK) { ++g_tc_passes; return after_launch("bwd_main (tcgen05)"); }
    if (rc != FLARE_EUNSUPPORTED) return fail(rc, "bwd_main (tcgen05): launch setup failed");
  }
  if (p->dropout_p > 0.f)
    return fail(FLARE_EUNSUPPORTED, "attention dropout needs the tensor-core kernels (bf16/fp16, D in {16,32}, M <= 1024)");
  if (use_s && !delta_n) return fail(FLARE_EINVAL, "bwd_main: delta_n scratch is null");
  TRY(flare_bwd_tokens(p, terms, q, k, v, dy, y, key_mask, z32, dz32, lse_m, lse_n, dk, dv, delta_n, stream));
  TRY(flare_bwd_dq_partial(p, terms, q, k, v, dy, key_mask, z32, dz32, lse_m, lse_n, delta_n, dq_part, stream));
  return FLARE_OK;
}

int check_peers(const char* what, const FlarePeers* g) {
  if (!g || !g->bufs || !g->mine || !g->flags) return fail(FLARE_EINVAL, "%s: incomplete peer description", what);
  if (g->world < 1 || g->world > 32 || g->rank < 0 || g->rank >= g->world)
    return fail(FLARE_EINVAL, "%s: rank %d of %d", what, g->rank, g->world);
  return FLARE_OK;
}

int flare_peer_barrier(const FlarePeers* g, flare_stream_t stream) {
  TRY(check_peers("peer_barrier", g));
  TRY(launch_peer_barrier(g->flags, g->rank, g->world, g->epoch, (cudaStream_t)stream));
  return after_launch("peer_barrier");
}

int flare_cp_mixer_fwd(const FlareProblem* p, const void* q, const void* k, const void* v,
                       const uint8_t* key_mask, void* y, float* z32, float* lse_m, float* lse_n,
                       void* workspace, size_t workspace_bytes, const FlarePeers* rec, flare_stream_t stream) {
  TRY(check_problem(p));
  TRY(check_peers("cp_mixer_fwd", rec));
  if (!z32 || !lse_m) return fail(FLARE_EINVAL, "z32 and lse_m are required outputs");
  const size_t need = flare_fwd_workspace_bytes(p);
  if (!workspace || workspace_bytes < need) return fail(FLARE_EWORKSPACE, "forward workspace: have %zu bytes, need %zu", workspace_bytes, need);
  FlareProblem pp = *p;
  pp.n_splits = flare_pick_splits(p);
  float* part = reinterpret_cast<float*>((reinterpret_cast<uintptr_t>(workspace) + 255) & ~uintptr_t(255));
  TRY(flare_gather_partial(&pp, q, k, v, key_mask, part, stream));
  TRY(flare_combine(&pp, part, pp.n_splits, nullptr, nullptr, nullptr, rec->mine, stream));
  TRY(flare_peer_barrier(rec, stream));
  TRY(flare_combine_peers(&pp, rec->bufs, rec->world, z32, nullptr, lse_m, nullptr, stream));
  TRY(flare_scatter(&pp, q, k, z32, key_mask, y, lse_n, stream));
  return FLARE_OK;
}

int flare_cp_mixer_bwd(const FlareProblem* p, const void* q, const void* k, const void* v, const void* dy,
                       const void* y, const uint8_t* key_mask, const float* z32, const float* lse_m,
                       const float* lse_n, float* dq32, void* dk, void* dv, void* workspace,
                       size_t workspace_bytes, const FlarePeers* dz, const FlarePeers* dq, flare_stream_t stream) {
  TRY(check_problem(p));
  TRY(check_peers("cp_mixer_bwd", dz));
  if (dq) TRY(check_peers("cp_mixer_bwd", dq));
  if (!dq32) return fail(FLARE_EINVAL, "dq32 is null");
  const size_t need = flare_bwd_workspace_bytes(p);
  if (!workspace || workspace_bytes < need) return fail(FLARE_EWORKSPACE, "backward workspace: have %zu bytes, need %zu", workspace_bytes, need);
  FlareProblem pp = *p;
  pp.n_splits = flare_pick_splits(p);
  const size_t S = (size_t)pp.n_splits;
  const size_t rows = (size_t)p->B * p->H * p->M;
  char* w = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(workspace) + 255) & ~uintptr_t(255));
  float* part = reinterpret_cast<float*>(w);      w += up256(S * rows * p->D * sizeof(float));
  float* dz32 = reinterpret_cast<float*>(w);      w += up256(rows * p->D * sizeof(float));
  float* delta = reinterpret_cast<float*>(w);
  TRY(flare_bwd_dz_partial(&pp, q, k, dy, key_mask, lse_n, part, stream));
  TRY(flare_reduce_sum(part, pp.n_splits, (int64_t)rows, p->D, dz->mine, stream));
  TRY(flare_peer_barrier(dz, stream));
  TRY(flare_reduce_sum_peers(dz->bufs, dz->world, (int64_t)rows, p->D, dz32, stream));
  TRY(flare_bwd_main(&pp, FLARE_TERM_BOTH, q, k, v, dy, y, key_mask, z32, dz32, lse_m, lse_n, dk, dv, delta, part, stream));
  const bool shared = p->q_stride[0] == 0;
  const int n_parts = shared ? pp.n_splits * p->B : pp.n_splits;
  const int64_t qrows = shared ? (int64_t)p->H * p->M : (int64_t)rows;
  TRY(flare_reduce_sum(part, n_parts, qrows, p->D, dq ? dq->mine : dq32, stream));
  if (dq) {
    TRY(flare_peer_barrier(dq, stream));
    TRY(flare_reduce_sum_peers(dq->bufs, dq->world, qrows, p->D, dq32, stream));
  }
  return FLARE_OK;
}

int flare_mixer_bwd(const FlareProblem* p, const void* q, const void* k, const void* v, const void* dy,
                    const void* y, const uint8_t* key_mask, const float* z32, const float* lse_m,
                    const float* lse_n, float* dq32, void* dk, void* dv, void* workspace,
                    size_t workspace_bytes, flare_stream_t stream) {
  TRY(check_problem(p));
  if (!dq32) return fail(FLARE_EINVAL, "dq32 is null");
  const size_t need = flare_bwd_workspace_bytes(p);
  if (!workspace || workspace_bytes < need) return fail(FLARE_EWORKSPACE, "backward workspace: have %zu bytes, need %zu", workspace_bytes, need);
  FlareProblem pp = *p;
  pp.n_splits = flare_pick_splits(p);
  const size_t S = (size_t)pp.n_splits;
  const size_t rows = (size_t)p->B * p->H * p->M;
  char* w = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(workspace) + 255) & ~uintptr_t(255));
  float* part = reinterpret_cast<float*>(w);      w += up256(S * rows * p->D * sizeof(float));
  float* dz32 = reinterpret_cast<float*>(w);      w += up256(rows * p->D * sizeof(float));
  float* delta = reinterpret_cast<float*>(w);
  TRY(flare_bwd_dz_partial(&pp, q, k, dy, key_mask, lse_n, part, stream));
  TRY(flare_reduce_sum(part, pp.n_splits, (int64_t)rows, p->D, dz32, stream));
  TRY(flare_bwd_main(&pp, FLARE_TERM_BOTH, q, k, v, dy, y, key_mask, z32, dz32, lse_m, lse_n, dk, dv, delta, part, stream));
  if (p->q_stride[0] == 0) {
    TRY(flare_reduce_sum(part, pp.n_splits * p->B, (int64_t)p->H * p->M, p->D, dq32, stream));
  } else {
    TRY(flare_reduce_sum(part, pp.n_splits, (int64_t)rows, p->D, dq32, stream));
  }
  return FLARE_OK;
}

}  // extern "C"
