/*
 * tdb_b200.h -- C ABI of the B200 (sm_100a) disentangled-attention library.
 *
 * The reference package (Ingvarstep/TurboDeBERTa) is pure Python + Triton and has no FFI; each
 * entry point below names the Python interface of the reference that it stands behind
 * (paths are relative to src/turbodeberta/ of the reference).  All pointers are DEVICE pointers
 * unless stated otherwise; the library never allocates, frees or keeps device memory, launches on
 * the stream it is given and does not synchronise.  Every function returns TDB_OK (0) or a
 * negative TDB_ERR_* code; tdb_last_error() gives a thread-local detail string.  Entry points may be called
 * from several host threads and for several devices at once.
 *
 * Element strides are in ELEMENTS of the tensor's dtype.  dtype: TDB_DTYPE_F32 or TDB_DTYPE_BF16.
 */
#ifndef TDB_B200_H_
#define TDB_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TDB_VERSION 100

#if defined(__GNUC__)
#define TDB_API __attribute__((visibility("default")))
#else
#define TDB_API
#endif

enum {
  TDB_OK = 0,
  TDB_ERR_ARG = -1,         /* null pointer, negative size, inconsistent arguments        */
  TDB_ERR_DTYPE = -2,       /* dtype code not supported by this entry point                */
  TDB_ERR_ALIGN = -3,       /* pointer or stride breaks the 16-byte rule of the bulk copies */
  TDB_ERR_SHAPE = -4,       /* head_dim != 64, table too small, sizes out of range        */
  TDB_ERR_UNSUPPORTED = -5, /* valid request that this build does not implement            */
  TDB_ERR_CUDA = -6,        /* a CUDA runtime/driver call failed (see tdb_last_error)      */
  TDB_ERR_TIMEOUT = -7,     /* a device-side bounded wait gave up (reported via status word) */
  TDB_ERR_WORKSPACE = -8    /* workspace missing or smaller than tdb_attn_workspace_bytes  */
};

enum { TDB_DTYPE_F32 = 0, TDB_DTYPE_BF16 = 1 };

/* which position terms are added to the content score (pos_att_type, model.py:84-90) */
enum { TDB_FLAG_C2P = 1, TDB_FLAG_P2C = 2, TDB_FLAG_P2C_MIRRORED = 4 /* only with materialised scores */ };

/* kernel selection: AUTO = tensor-core (tcgen05) kernel for bf16, CUDA-core kernel for f32. */
enum { TDB_KERNEL_AUTO = 0, TDB_KERNEL_SIMT = 1, TDB_KERNEL_UMMA = 2 };

/* Width, in rows, of the distance-expanded tables for a given max_relative_positions (or
 * position_buckets <= 0: the span): rows cover delta in [-(P+256), P+256], padded to a multiple of 8. */
#define TDB_EXPAND_MARGIN 256

TDB_API int tdb_version(void);
TDB_API const char* tdb_strerror(int code);
TDB_API const char* tdb_last_error(void);

/* Relative-position row index for every distance delta = q - k in [-delta_max, delta_max]:
 *   idx_out[delta + delta_max] = clamp(bucket(delta) + span, 0, 2*span - 1)   (int16, 2*delta_max+1 entries)
 * bucket() is the log bucket when position_buckets > 0 (span = position_buckets), else the identity
 * (span = max_relative_positions).  Replaces the per-score-element evaluation in
 * ops/flash_attention.py:100-122 and ops/flash_attention_varlen.py:118-140; bit-exact with the eager
 * module's make_log_bucket_position + clamp. */
TDB_API int tdb_bucket_table(int position_buckets, int max_relative_positions, int delta_max,
                     int16_t* idx_out, void* stream);

/* out[h, r, :] = rel[r, :] . W[h*D:(h+1)*D, :]^T + bias[h*D:(h+1)*D]      (r < two_span)
 * rel [two_span, hidden] (already LayerNorm'd by the encoder), W [H*D, hidden] row-major, bias [H*D] or NULL,
 * out [H, two_span, D]; all of `dtype`.  Replaces model.py:92-110 (key_proj/query_proj or
 * pos_key_proj/pos_query_proj applied to rel_embeddings followed by the head split at :70-73).
 * bf16 with D == 64 runs as a tcgen05 GEMM (TMA-staged operands, accumulator in tensor memory); f32 runs on
 * the CUDA cores with fp32 accumulation.  status: int32[4] zeroed device words as for the attention calls
 * (word 0 reports a bounded wait that gave up); required for bf16, may be NULL for f32. */
TDB_API int tdb_relpos_project(const void* rel, const void* W, const void* bias, int two_span, int hidden,
                       int H, int D, int dtype, void* out, int32_t* status, void* stream);

/* Distance-expanded copy of a projected table, always bf16:
 *   out[h, x, :] = table[h, idx[clamp(x - exp_delta_max, -idx_delta_max, idx_delta_max) + idx_delta_max], :]
 * for x in [0, exp_rows), exp_rows >= 2*exp_delta_max+1.  table [H, two_span, D] of `dtype`.  With it the
 * rows a 128x128 score tile needs are one contiguous window, which the tensor-core kernel loads with a
 * single bulk copy.  exp_delta_max must be (saturation distance + TDB_EXPAND_MARGIN), where the saturation distance
 * is the smallest |delta| from which idx[] no longer changes on either side (max_relative_positions for an even
 * position_buckets, the span without buckets): the attention kernel derives the saturation distance from
 * exp_delta_max to recognise tiles whose scores all use one table row.  No counterpart in the reference, which
 * instead materialises Q.Kr^T and K.Qr^T for every token (model.py:122-125, 143-148). */
TDB_API int tdb_relpos_expand(const void* table, const int16_t* idx, int idx_delta_max, int H, int two_span,
                      int D, int dtype, int exp_delta_max, int exp_rows, void* out, void* stream);

/* Bytes of scratch the packed (varlen) tensor-core path needs for its device-built tile list. */
TDB_API size_t tdb_attn_workspace_bytes(int n_seqs, int64_t total_tokens);

/* Fused disentangled attention, padded form.  Stands behind flash_attention_with_disentangled
 * (ops/flash_attention.py:345-369) as called from model.py:127-137, with two differences: the two
 * [B,H,L,2*span] score tensors of that call are replaced by the projected tables kr/qr [H, two_span, D]
 * (the products are formed on chip), and `seqlens` adds the right-padding mask that the reference
 * kernel lacks.  q, k, v, o: logical shape [B, L, H, D], D contiguous, strides given per tensor.
 * seqlens: int32 [B] valid lengths or NULL (all L).  Query rows at or beyond the length are written as zeros;
 * rows of q, k, v at or beyond the length may hold anything (NaN included) and never reach the result.
 * idx: table from tdb_bucket_table; kr_exp/qr_exp: tables from tdb_relpos_expand (needed by the
 * tensor-core kernel; may be NULL for the CUDA-core kernel).  lse: float [B, H, L] or NULL.
 * status: int32[4] device words, zero on entry; word 0 becomes non-zero if a bounded wait gave up, word 1 if
 * cu_seqlens was malformed (packed form: decreasing offsets, a sequence longer than max_seqlen, a last offset that
 * differs from total_tokens); word 2 is used by the tensor-core kernel as its work counter (the launch
 * resets it), word 3 is reserved.  Do not share one status block between launches that can overlap. */
TDB_API int tdb_attn_fwd_fixed(const void* q, const void* k, const void* v, void* o,
                       int64_t q_sb, int64_t q_st, int64_t q_sh,
                       int64_t k_sb, int64_t k_st, int64_t k_sh,
                       int64_t v_sb, int64_t v_st, int64_t v_sh,
                       int64_t o_sb, int64_t o_st, int64_t o_sh,
                       const void* kr, const void* qr, int two_span,
                       const int16_t* idx, int idx_delta_max,
                       const void* kr_exp, const void* qr_exp, int exp_delta_max, int exp_rows,
                       const int32_t* seqlens, int B, int L, int H, int D,
                       float sm_scale, int flags, int dtype, int kernel,
                       float* lse, int32_t* status, void* stream);

/* Fused disentangled attention, packed form.  Stands behind flash_attention_with_disentangled_varlen
 * (ops/flash_attention_varlen.py:348-374) as called from model.py:170-182; same table arguments as above.
 * q, k, v, o: [T, H, D]; cu_seqlens int32 [n_seqs+1]; relative positions restart at each sequence.
 * workspace: at least tdb_attn_workspace_bytes(n_seqs, T) bytes (tensor-core kernel only).  lse: float [H, T] or NULL. */
TDB_API int tdb_attn_fwd_varlen(const void* q, const void* k, const void* v, void* o,
                        int64_t q_st, int64_t q_sh, int64_t k_st, int64_t k_sh,
                        int64_t v_st, int64_t v_sh, int64_t o_st, int64_t o_sh,
                        const void* kr, const void* qr, int two_span,
                        const int16_t* idx, int idx_delta_max,
                        const void* kr_exp, const void* qr_exp, int exp_delta_max, int exp_rows,
                        const int32_t* cu_seqlens, int n_seqs, int64_t total_tokens, int max_seqlen,
                        int H, int D, float sm_scale, int flags, int dtype, int kernel,
                        void* workspace, size_t workspace_bytes,
                        float* lse, int32_t* status, void* stream);

/* Packed-form attention for callers that cannot provide scratch memory.  No counterpart in the reference.
 *
 * Some hosts of this library cannot allocate device memory at the point where they call it: an inference
 * server's execute callback that is handed only its bound input and output buffers, or a C/C++ program that has
 * given all device memory to a framework's pool and holds no handle to that pool.  tdb_attn_fwd_varlen needs a
 * caller-provided workspace for its device-built tile list; this variant keeps that list in a fixed array that
 * lives inside the library image on the device (TDB_STATIC_SCRATCH_BYTES, held by every GPU that loads the
 * library until the process exits) and therefore takes no workspace arguments.  It calls no allocator.
 *
 * Limit: tdb_attn_workspace_bytes(n_seqs, total_tokens) must not exceed TDB_STATIC_SCRATCH_BYTES, i.e.
 * n_seqs + ceil(total_tokens / 128) + 1 <= TDB_STATIC_MAX_TILES; larger problems return TDB_ERR_WORKSPACE.
 * The first call on each device looks up the array's device address (cudaGetSymbolAddress); make that first
 * call outside any stream capture.  All calls on a device share the one array and it keeps the previous call's
 * contents (each call rewrites the part it reads, nothing has to start at zero), so two calls whose kernels can
 * overlap on the GPU -- different streams, or different host threads -- race on it: serialise them.
 * All other arguments are those of tdb_attn_fwd_varlen. */
#define TDB_STATIC_MAX_TILES 65535
#define TDB_STATIC_SCRATCH_BYTES (16 + 8 * TDB_STATIC_MAX_TILES)
TDB_API int tdb_attn_fwd_varlen_static(const void* q, const void* k, const void* v, void* o,
                        int64_t q_st, int64_t q_sh, int64_t k_st, int64_t k_sh,
                        int64_t v_st, int64_t v_sh, int64_t o_st, int64_t o_sh,
                        const void* kr, const void* qr, int two_span,
                        const int16_t* idx, int idx_delta_max,
                        const void* kr_exp, const void* qr_exp, int exp_delta_max, int exp_rows,
                        const int32_t* cu_seqlens, int n_seqs, int64_t total_tokens, int max_seqlen,
                        int H, int D, float sm_scale, int flags, int dtype, int kernel,
                        float* lse, int32_t* status, void* stream);

/* Diagnostic (no counterpart in the reference): launches one warp that waits, with the same bounded wait every hand-off
 * of the tensor-core kernels uses, on a barrier that nothing completes.  After at most limit_us microseconds (1..100000)
 * the wait gives up and writes `code` (> 0) into status[0]; the kernel then returns normally and the context stays
 * usable.  Lets a caller check, without any fault, that a stuck hand-off would be reported rather than hang. */
TDB_API int tdb_selftest_bounded_wait(int32_t* status, int code, int limit_us, void* stream);

/* Legacy operator form (reference ops/flash_attention.py:345-369 and ops/flash_attention_varlen.py:348-374 called with
 * the MATERIALISED position scores of model.py:122-125 / 143-148): c2p_scores[b, h, t, r] = Q[t].Kr[r] and
 * p2c_scores[b, h, t, r] = K[t].Qr[r] (rows of two_span contiguous elements of the I/O dtype; either may be null with
 * its flag clear).  The kernel only gathers them: score[q,k] = (Q[q].K[k] + c2p_scores[q, idx(q-k)] + p2c_scores[k,
 * idx(q-k)]) * sm_scale, the eager module's convention (HF modeling_deberta_v2.py:315-343); with
 * TDB_FLAG_P2C_MIRRORED the p2c term is read at idx(k-q) instead, which is what the reference's own kernel does
 * (ops/flash_attention.py:126-132).  CUDA-core kernel, f32 or bf16; a compatibility path, not a throughput path --
 * the fused entry points above exist to avoid these tensors.  Strides in elements; other arguments as above. */
TDB_API int tdb_attn_fwd_fixed_scores(const void* q, const void* k, const void* v, void* o,
                        int64_t q_sb, int64_t q_st, int64_t q_sh, int64_t k_sb, int64_t k_st, int64_t k_sh,
                        int64_t v_sb, int64_t v_st, int64_t v_sh, int64_t o_sb, int64_t o_st, int64_t o_sh,
                        const void* c2p_scores, int64_t c2p_sb, int64_t c2p_st, int64_t c2p_sh,
                        const void* p2c_scores, int64_t p2c_sb, int64_t p2c_st, int64_t p2c_sh,
                        int two_span, const int16_t* idx, int idx_delta_max,
                        const int32_t* seqlens, int B, int L, int H, int D, float sm_scale, int flags, int dtype,
                        float* lse, int32_t* status, void* stream);
TDB_API int tdb_attn_fwd_varlen_scores(const void* q, const void* k, const void* v, void* o,
                        int64_t q_st, int64_t q_sh, int64_t k_st, int64_t k_sh, int64_t v_st, int64_t v_sh,
                        int64_t o_st, int64_t o_sh,
                        const void* c2p_scores, int64_t c2p_st, int64_t c2p_sh,
                        const void* p2c_scores, int64_t p2c_st, int64_t p2c_sh,
                        int two_span, const int16_t* idx, int idx_delta_max,
                        const int32_t* cu_seqlens, int n_seqs, int64_t total_tokens, int max_seqlen,
                        int H, int D, float sm_scale, int flags, int dtype,
                        float* lse, int32_t* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TDB_B200_H_ */
