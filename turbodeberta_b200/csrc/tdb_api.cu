// extern "C" entry points: argument validation, error reporting, kernel selection.
#include "tdb_internal.h"
#include <cstdarg>
#include <cstdio>
#include <cstring>

namespace tdb {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap; va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int cuda_fail(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return TDB_OK;
  set_error("%s: %s", what, cudaGetErrorString(e));
  return TDB_ERR_CUDA;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static int check_tensor(const char* name, const void* ptr, int dtype, int64_t st, int64_t sh, int64_t sb) {
  if (!ptr) { set_error("%s is null", name); return TDB_ERR_ARG; }
  int64_t per16 = dtype == TDB_DTYPE_F32 ? 4 : 8;
  if (!aligned16(ptr)) { set_error("%s is not 16-byte aligned", name); return TDB_ERR_ALIGN; }
  if (st % per16 || sh % per16 || sb % per16) {
    set_error("%s strides (%lld, %lld, %lld) are not multiples of 16 bytes", name, (long long)sb, (long long)st, (long long)sh);
    return TDB_ERR_ALIGN;
  }
  if (st <= 0 || sh <= 0 || sb < 0) { set_error("%s has a non-positive stride", name); return TDB_ERR_ARG; }
  return TDB_OK;
}

static int check_common(const AttnParams& p, int dtype, int kernel) {
  if (dtype != TDB_DTYPE_F32 && dtype != TDB_DTYPE_BF16) { set_error("dtype %d is not f32 or bf16", dtype); return TDB_ERR_DTYPE; }
  if (p.D != 64) { set_error("head_dim %d: only 64 is supported", p.D); return TDB_ERR_SHAPE; }
  if (p.H <= 0 || p.n_seqs < 0 || p.L < 0) { set_error("negative or zero size (H=%d, n_seqs=%d, L=%d)", p.H, p.n_seqs, p.L); return TDB_ERR_ARG; }
  const bool gathered = p.c2p_scores || p.p2c_scores;
  if (p.flags & ~(TDB_FLAG_C2P | TDB_FLAG_P2C | (gathered ? TDB_FLAG_P2C_MIRRORED : 0))) { set_error("unknown flag bits 0x%x", p.flags); return TDB_ERR_ARG; }
  if (kernel < TDB_KERNEL_AUTO || kernel > TDB_KERNEL_UMMA) { set_error("unknown kernel selector %d", kernel); return TDB_ERR_ARG; }
  if (!(p.sm_scale > 0.f) || !(p.sm_scale < 1e6f)) { set_error("sm_scale must be a positive finite number"); return TDB_ERR_ARG; }
  if (!p.status) { set_error("status word pointer is null"); return TDB_ERR_ARG; }
  int rc;
  if ((rc = check_tensor("q", p.q, dtype, p.q_st, p.q_sh, p.q_sb))) return rc;
  if ((rc = check_tensor("k", p.k, dtype, p.k_st, p.k_sh, p.k_sb))) return rc;
  if ((rc = check_tensor("v", p.v, dtype, p.v_st, p.v_sh, p.v_sb))) return rc;
  if ((rc = check_tensor("o", p.o, dtype, p.o_st, p.o_sh, p.o_sb))) return rc;
  if (p.flags) {
    if (p.two_span <= 0 || p.two_span > 32767) { set_error("two_span %d out of range", p.two_span); return TDB_ERR_SHAPE; }
    if (!p.idx || p.idx_delta_max <= 0) { set_error("position terms requested without an index table"); return TDB_ERR_ARG; }
    if (gathered) {
      if ((p.flags & TDB_FLAG_C2P) && !p.c2p_scores) { set_error("c2p requested without c2p_scores"); return TDB_ERR_ARG; }
      if ((p.flags & TDB_FLAG_P2C) && !p.p2c_scores) { set_error("p2c requested without p2c_scores"); return TDB_ERR_ARG; }
      if (((p.flags & TDB_FLAG_C2P) && (p.c2p_st <= 0 || p.c2p_sh <= 0 || p.c2p_sb < 0)) ||
          ((p.flags & TDB_FLAG_P2C) && (p.p2c_st <= 0 || p.p2c_sh <= 0 || p.p2c_sb < 0))) {
        set_error("position score tensor has a non-positive stride"); return TDB_ERR_ARG;
      }
    } else {
      if ((p.flags & TDB_FLAG_C2P) && (!p.kr || !aligned16(p.kr))) { set_error("kr table missing or misaligned"); return p.kr ? TDB_ERR_ALIGN : TDB_ERR_ARG; }
      if ((p.flags & TDB_FLAG_P2C) && (!p.qr || !aligned16(p.qr))) { set_error("qr table missing or misaligned"); return p.qr ? TDB_ERR_ALIGN : TDB_ERR_ARG; }
    }
  }
  return TDB_OK;
}

static int pick_kernel(int dtype, int kernel) {
  if (kernel != TDB_KERNEL_AUTO) return kernel;
  return dtype == TDB_DTYPE_BF16 ? TDB_KERNEL_UMMA : TDB_KERNEL_SIMT;
}

static int check_umma(const AttnParams& p, int dtype) {
  if (dtype != TDB_DTYPE_BF16) { set_error("the tensor-core kernel takes bf16 only"); return TDB_ERR_DTYPE; }
  if (p.flags & TDB_FLAG_C2P) {
    if (!p.kr_exp || !aligned16(p.kr_exp)) { set_error("kr_exp (expanded table) missing or misaligned"); return p.kr_exp ? TDB_ERR_ALIGN : TDB_ERR_ARG; }
  }
  if (p.flags & TDB_FLAG_P2C) {
    if (!p.qr_exp || !aligned16(p.qr_exp)) { set_error("qr_exp (expanded table) missing or misaligned"); return p.qr_exp ? TDB_ERR_ALIGN : TDB_ERR_ARG; }
  }
  if (p.flags) {
    if (p.exp_delta_max < 256 || p.exp_rows < 2 * p.exp_delta_max + 1 || (p.exp_rows % 8)) {
      set_error("expanded table geometry (delta_max=%d, rows=%d) invalid: need delta_max>=256, rows>=2*delta_max+1, rows%%8==0",
                p.exp_delta_max, p.exp_rows);
      return TDB_ERR_SHAPE;
    }
  }
  return TDB_OK;
}

}  // namespace tdb

using namespace tdb;

extern "C" {

TDB_API int tdb_version(void) { return TDB_VERSION; }

TDB_API const char* tdb_strerror(int code) {
  switch (code) {
    case TDB_OK: return "ok";
    case TDB_ERR_ARG: return "invalid argument";
    case TDB_ERR_DTYPE: return "unsupported dtype";
    case TDB_ERR_ALIGN: return "pointer or stride not 16-byte aligned";
    case TDB_ERR_SHAPE: return "unsupported shape";
    case TDB_ERR_UNSUPPORTED: return "not implemented in this build";
    case TDB_ERR_CUDA: return "CUDA call failed";
    case TDB_ERR_TIMEOUT: return "device-side wait timed out";
    case TDB_ERR_WORKSPACE: return "workspace missing or too small";
    default: return "unknown error code";
  }
}

TDB_API const char* tdb_last_error(void) { return g_err; }

TDB_API int tdb_bucket_table(int position_buckets, int max_relative_positions, int delta_max, int16_t* idx_out, void* stream) {
  if (!idx_out) { set_error("idx_out is null"); return TDB_ERR_ARG; }
  if (delta_max <= 0 || delta_max > (1 << 24)) { set_error("delta_max %d out of range", delta_max); return TDB_ERR_ARG; }
  int span = position_buckets > 0 ? position_buckets : max_relative_positions;
  if (span <= 0 || 2 * span - 1 > 32767) { set_error("span %d out of range", span); return TDB_ERR_SHAPE; }
  if (position_buckets > 0 && max_relative_positions <= position_buckets / 2) {
    set_error("max_relative_positions %d must exceed position_buckets/2", max_relative_positions); return TDB_ERR_ARG;
  }
  return launch_bucket_table(position_buckets, max_relative_positions, delta_max, idx_out, (cudaStream_t)stream);
}

TDB_API int tdb_relpos_project(const void* rel, const void* W, const void* bias, int two_span, int hidden, int H, int D,
                       int dtype, void* out, int32_t* status, void* stream) {
  if (!rel || !W || !out) { set_error("rel, W or out is null"); return TDB_ERR_ARG; }
  if (dtype != TDB_DTYPE_F32 && dtype != TDB_DTYPE_BF16) { set_error("dtype %d is not f32 or bf16", dtype); return TDB_ERR_DTYPE; }
  if (two_span <= 0 || hidden <= 0 || H <= 0 || D <= 0) { set_error("non-positive size"); return TDB_ERR_ARG; }
  if (relpos_umma_applicable(rel, W, out, hidden, D, dtype) && (!bias || (reinterpret_cast<uintptr_t>(bias) & 1u) == 0)) {
    if (!status) { set_error("status word pointer is null (required for the bf16 tensor-core projection)"); return TDB_ERR_ARG; }
    if (H > 65535) { set_error("more than 65535 heads"); return TDB_ERR_SHAPE; }
    return launch_relpos_project_umma(rel, W, bias, two_span, hidden, H, out, status, (cudaStream_t)stream);
  }
  return launch_relpos_project(rel, W, bias, two_span, hidden, H, D, dtype, out, (cudaStream_t)stream);
}

TDB_API int tdb_relpos_expand(const void* table, const int16_t* idx, int idx_delta_max, int H, int two_span, int D, int dtype,
                      int exp_delta_max, int exp_rows, void* out, void* stream) {
  if (!table || !idx || !out) { set_error("table, idx or out is null"); return TDB_ERR_ARG; }
  if (dtype != TDB_DTYPE_F32 && dtype != TDB_DTYPE_BF16) { set_error("dtype %d is not f32 or bf16", dtype); return TDB_ERR_DTYPE; }
  if (H <= 0 || two_span <= 0 || D <= 0 || idx_delta_max <= 0 || exp_delta_max <= 0 || exp_rows < 2 * exp_delta_max + 1) {
    set_error("invalid sizes for relpos_expand"); return TDB_ERR_ARG;
  }
  return launch_relpos_expand(table, idx, idx_delta_max, H, two_span, D, dtype, exp_delta_max, exp_rows, out,
                              (cudaStream_t)stream);
}

TDB_API int tdb_selftest_bounded_wait(int32_t* status, int code, int limit_us, void* stream) {
  if (!status) { set_error("status word pointer is null"); return TDB_ERR_ARG; }
  if (code <= 0) { set_error("code must be positive"); return TDB_ERR_ARG; }
  if (limit_us <= 0 || limit_us > 100000) { set_error("limit of %d us outside (0, 100000]", limit_us); return TDB_ERR_ARG; }
  return launch_bounded_wait_selftest(status, code, (uint64_t)limit_us * 1000ull, (cudaStream_t)stream);
}

TDB_API size_t tdb_attn_workspace_bytes(int n_seqs, int64_t total_tokens) {
  if (n_seqs < 0 || total_tokens < 0) return 0;
  return umma_workspace_bytes(n_seqs, total_tokens);
}

TDB_API int tdb_attn_fwd_fixed(const void* q, const void* k, const void* v, void* o,
                       int64_t q_sb, int64_t q_st, int64_t q_sh, int64_t k_sb, int64_t k_st, int64_t k_sh,
                       int64_t v_sb, int64_t v_st, int64_t v_sh, int64_t o_sb, int64_t o_st, int64_t o_sh,
                       const void* kr, const void* qr, int two_span, const int16_t* idx, int idx_delta_max,
                       const void* kr_exp, const void* qr_exp, int exp_delta_max, int exp_rows,
                       const int32_t* seqlens, int B, int L, int H, int D, float sm_scale, int flags, int dtype,
                       int kernel, float* lse, int32_t* status, void* stream) {
  AttnParams p;
  memset(&p, 0, sizeof(p));
  p.q = q; p.k = k; p.v = v; p.o = o;
  p.q_sb = q_sb; p.q_st = q_st; p.q_sh = q_sh; p.k_sb = k_sb; p.k_st = k_st; p.k_sh = k_sh;
  p.v_sb = v_sb; p.v_st = v_st; p.v_sh = v_sh; p.o_sb = o_sb; p.o_st = o_st; p.o_sh = o_sh;
  p.kr = kr; p.qr = qr; p.two_span = two_span; p.idx = idx; p.idx_delta_max = idx_delta_max;
  p.kr_exp = kr_exp; p.qr_exp = qr_exp; p.exp_delta_max = exp_delta_max; p.exp_rows = exp_rows;
  p.seqlens = seqlens; p.cu_seqlens = nullptr; p.varlen = 0; p.n_seqs = B; p.L = L; p.total_tokens = (int64_t)B * L;
  p.H = H; p.D = D; p.sm_scale = sm_scale; p.flags = flags;
  p.lse = lse; p.lse_sb = (int64_t)H * L; p.lse_sh = L; p.status = status;
  if (B < 0 || L < 0) { set_error("negative size"); return TDB_ERR_ARG; }
  if (B == 0 || L == 0) return TDB_OK;     // nothing to compute: pointers of empty tensors may be null
  int rc = check_common(p, dtype, kernel);
  if (rc) return rc;
  if (B > 1 && (q_sb <= 0 || k_sb <= 0 || v_sb <= 0 || o_sb <= 0)) { set_error("batch stride must be positive when B > 1"); return TDB_ERR_ARG; }
  int kn = pick_kernel(dtype, kernel);
  if (kn == TDB_KERNEL_SIMT) return launch_attn_simt(p, dtype, (cudaStream_t)stream);
  if ((rc = check_umma(p, dtype))) return rc;
  return launch_attn_umma(p, (cudaStream_t)stream);
}

TDB_API int tdb_attn_fwd_varlen(const void* q, const void* k, const void* v, void* o,
                        int64_t q_st, int64_t q_sh, int64_t k_st, int64_t k_sh, int64_t v_st, int64_t v_sh,
                        int64_t o_st, int64_t o_sh, const void* kr, const void* qr, int two_span,
                        const int16_t* idx, int idx_delta_max, const void* kr_exp, const void* qr_exp,
                        int exp_delta_max, int exp_rows, const int32_t* cu_seqlens, int n_seqs, int64_t total_tokens,
                        int max_seqlen, int H, int D, float sm_scale, int flags, int dtype, int kernel,
                        void* workspace, size_t workspace_bytes, float* lse, int32_t* status, void* stream) {
  AttnParams p;
  memset(&p, 0, sizeof(p));
  p.q = q; p.k = k; p.v = v; p.o = o;
  p.q_st = q_st; p.q_sh = q_sh; p.k_st = k_st; p.k_sh = k_sh; p.v_st = v_st; p.v_sh = v_sh; p.o_st = o_st; p.o_sh = o_sh;
  p.kr = kr; p.qr = qr; p.two_span = two_span; p.idx = idx; p.idx_delta_max = idx_delta_max;
  p.kr_exp = kr_exp; p.qr_exp = qr_exp; p.exp_delta_max = exp_delta_max; p.exp_rows = exp_rows;
  p.seqlens = nullptr; p.cu_seqlens = cu_seqlens; p.varlen = 1; p.n_seqs = n_seqs; p.L = max_seqlen;
  p.total_tokens = total_tokens;
  p.H = H; p.D = D; p.sm_scale = sm_scale; p.flags = flags;
  p.lse = lse; p.lse_sb = 0; p.lse_sh = total_tokens; p.status = status;
  p.workspace = workspace; p.workspace_bytes = workspace_bytes;
  if (n_seqs == 0 || total_tokens == 0) {
    if (n_seqs < 0 || total_tokens < 0) { set_error("negative size"); return TDB_ERR_ARG; }
    return TDB_OK;
  }
  if (!cu_seqlens) { set_error("cu_seqlens is null"); return TDB_ERR_ARG; }
  if (max_seqlen <= 0 || max_seqlen > total_tokens) { set_error("max_seqlen %d outside [1, total_tokens]", max_seqlen); return TDB_ERR_ARG; }
  int rc = check_common(p, dtype, kernel);
  if (rc) return rc;
  int kn = pick_kernel(dtype, kernel);
  if (kn == TDB_KERNEL_SIMT) return launch_attn_simt(p, dtype, (cudaStream_t)stream);
  if ((rc = check_umma(p, dtype))) return rc;
  if (!workspace || workspace_bytes < umma_workspace_bytes(n_seqs, total_tokens)) {
    set_error("workspace of %zu bytes is smaller than the %zu required", workspace_bytes, umma_workspace_bytes(n_seqs, total_tokens));
    return TDB_ERR_WORKSPACE;
  }
  return launch_attn_umma(p, (cudaStream_t)stream);
}

TDB_API int tdb_attn_fwd_fixed_scores(const void* q, const void* k, const void* v, void* o,
                        int64_t q_sb, int64_t q_st, int64_t q_sh, int64_t k_sb, int64_t k_st, int64_t k_sh,
                        int64_t v_sb, int64_t v_st, int64_t v_sh, int64_t o_sb, int64_t o_st, int64_t o_sh,
                        const void* c2p_scores, int64_t c2p_sb, int64_t c2p_st, int64_t c2p_sh,
                        const void* p2c_scores, int64_t p2c_sb, int64_t p2c_st, int64_t p2c_sh,
                        int two_span, const int16_t* idx, int idx_delta_max,
                        const int32_t* seqlens, int B, int L, int H, int D, float sm_scale, int flags, int dtype,
                        float* lse, int32_t* status, void* stream) {
  AttnParams p;
  memset(&p, 0, sizeof(p));
  p.q = q; p.k = k; p.v = v; p.o = o;
  p.q_sb = q_sb; p.q_st = q_st; p.q_sh = q_sh; p.k_sb = k_sb; p.k_st = k_st; p.k_sh = k_sh;
  p.v_sb = v_sb; p.v_st = v_st; p.v_sh = v_sh; p.o_sb = o_sb; p.o_st = o_st; p.o_sh = o_sh;
  p.c2p_scores = c2p_scores; p.c2p_sb = c2p_sb; p.c2p_st = c2p_st; p.c2p_sh = c2p_sh;
  p.p2c_scores = p2c_scores; p.p2c_sb = p2c_sb; p.p2c_st = p2c_st; p.p2c_sh = p2c_sh;
  p.two_span = two_span; p.idx = idx; p.idx_delta_max = idx_delta_max;
  p.seqlens = seqlens; p.varlen = 0; p.n_seqs = B; p.L = L; p.total_tokens = (int64_t)B * L;
  p.H = H; p.D = D; p.sm_scale = sm_scale; p.flags = flags;
  p.lse = lse; p.lse_sb = (int64_t)H * L; p.lse_sh = L; p.status = status;
  if (B < 0 || L < 0) { set_error("negative size"); return TDB_ERR_ARG; }
  if (B == 0 || L == 0) return TDB_OK;
  if (!c2p_scores && !p2c_scores) { set_error("no position scores given: use tdb_attn_fwd_fixed"); return TDB_ERR_ARG; }
  int rc = check_common(p, dtype, TDB_KERNEL_SIMT);
  if (rc) return rc;
  if (B > 1 && (q_sb <= 0 || k_sb <= 0 || v_sb <= 0 || o_sb <= 0)) { set_error("batch stride must be positive when B > 1"); return TDB_ERR_ARG; }
  return launch_attn_simt(p, dtype, (cudaStream_t)stream);
}

TDB_API int tdb_attn_fwd_varlen_scores(const void* q, const void* k, const void* v, void* o,
                        int64_t q_st, int64_t q_sh, int64_t k_st, int64_t k_sh, int64_t v_st, int64_t v_sh,
                        int64_t o_st, int64_t o_sh,
                        const void* c2p_scores, int64_t c2p_st, int64_t c2p_sh,
                        const void* p2c_scores, int64_t p2c_st, int64_t p2c_sh,
                        int two_span, const int16_t* idx, int idx_delta_max,
                        const int32_t* cu_seqlens, int n_seqs, int64_t total_tokens, int max_seqlen,
                        int H, int D, float sm_scale, int flags, int dtype,
                        float* lse, int32_t* status, void* stream) {
  AttnParams p;
  memset(&p, 0, sizeof(p));
  p.q = q; p.k = k; p.v = v; p.o = o;
  p.q_st = q_st; p.q_sh = q_sh; p.k_st = k_st; p.k_sh = k_sh; p.v_st = v_st; p.v_sh = v_sh; p.o_st = o_st; p.o_sh = o_sh;
  p.c2p_scores = c2p_scores; p.c2p_st = c2p_st; p.c2p_sh = c2p_sh;
  p.p2c_scores = p2c_scores; p.p2c_st = p2c_st; p.p2c_sh = p2c_sh;
  p.two_span = two_span; p.idx = idx; p.idx_delta_max = idx_delta_max;
  p.cu_seqlens = cu_seqlens; p.varlen = 1; p.n_seqs = n_seqs; p.L = max_seqlen; p.total_tokens = total_tokens;
  p.H = H; p.D = D; p.sm_scale = sm_scale; p.flags = flags;
  p.lse = lse; p.lse_sb = 0; p.lse_sh = total_tokens; p.status = status;
  if (n_seqs == 0 || total_tokens == 0) {
    if (n_seqs < 0 || total_tokens < 0) { set_error("negative size"); return TDB_ERR_ARG; }
    return TDB_OK;
  }
  if (!cu_seqlens) { set_error("cu_seqlens is null"); return TDB_ERR_ARG; }
  if (max_seqlen <= 0 || max_seqlen > total_tokens) { set_error("max_seqlen %d outside [1, total_tokens]", max_seqlen); return TDB_ERR_ARG; }
  if (!c2p_scores && !p2c_scores) { set_error("no position scores given: use tdb_attn_fwd_varlen"); return TDB_ERR_ARG; }
  int rc = check_common(p, dtype, TDB_KERNEL_SIMT);
  if (rc) return rc;
  return launch_attn_simt(p, dtype, (cudaStream_t)stream);
}

// Same as tdb_attn_fwd_varlen, with the tile list kept in the library's fixed device array instead of a
// caller-provided workspace.  Allocates nothing; the first call on a device resolves the array's address.
TDB_API int tdb_attn_fwd_varlen_static(const void* q, const void* k, const void* v, void* o,
                        int64_t q_st, int64_t q_sh, int64_t k_st, int64_t k_sh, int64_t v_st, int64_t v_sh,
                        int64_t o_st, int64_t o_sh, const void* kr, const void* qr, int two_span,
                        const int16_t* idx, int idx_delta_max, const void* kr_exp, const void* qr_exp,
                        int exp_delta_max, int exp_rows, const int32_t* cu_seqlens, int n_seqs, int64_t total_tokens,
                        int max_seqlen, int H, int D, float sm_scale, int flags, int dtype, int kernel,
                        float* lse, int32_t* status, void* stream) {
  if (n_seqs < 0 || total_tokens < 0) { set_error("negative size"); return TDB_ERR_ARG; }
  const size_t need = umma_workspace_bytes(n_seqs, total_tokens);
  if (need > (size_t)TDB_STATIC_SCRATCH_BYTES) {
    set_error("problem needs %zu bytes of tile list but the built-in scratch holds %zu "
              "(limit: n_seqs + ceil(total_tokens/128) + 1 <= %d); use tdb_attn_fwd_varlen with a workspace",
              need, (size_t)TDB_STATIC_SCRATCH_BYTES, TDB_STATIC_MAX_TILES);
    return TDB_ERR_WORKSPACE;
  }
  void* scratch = nullptr;
  int rc = static_tile_scratch(&scratch);
  if (rc) return rc;
  return tdb_attn_fwd_varlen(q, k, v, o, q_st, q_sh, k_st, k_sh, v_st, v_sh, o_st, o_sh, kr, qr, two_span, idx,
                             idx_delta_max, kr_exp, qr_exp, exp_delta_max, exp_rows, cu_seqlens, n_seqs, total_tokens,
                             max_seqlen, H, D, sm_scale, flags, dtype, kernel, scratch, (size_t)TDB_STATIC_SCRATCH_BYTES,
                             lse, status, stream);
}

}  // extern "C"
