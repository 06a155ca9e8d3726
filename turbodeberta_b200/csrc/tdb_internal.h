// Internal declarations shared by the translation units of libtdb_b200.so.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stddef.h>
#include "../../include/tdb_b200.h"

namespace tdb {

// One attention problem in either form.  Padded form: sequence s is batch row s, tokens 0..L-1,
// valid length seqlens[s] (or L).  Packed form: sequence s is tokens cu_seqlens[s]..cu_seqlens[s+1]-1
// of batch row 0.
struct AttnParams {
  const void* q; const void* k; const void* v; void* o;
  int64_t q_sb, q_st, q_sh;
  int64_t k_sb, k_st, k_sh;
  int64_t v_sb, v_st, v_sh;
  int64_t o_sb, o_st, o_sh;
  const void* kr; const void* qr; int two_span;          // [H, two_span, D] of the I/O dtype
  const int16_t* idx; int idx_delta_max;                  // delta -> table row
  const void* kr_exp; const void* qr_exp;                 // [H, exp_rows, D] bf16, row x <-> delta = x - exp_delta_max
  // Materialised position scores (legacy op interface): c2p_scores[b, h, t, r] = Q[t].Kr[r], p2c_scores[b, h, t, r]
  // = K[t].Qr[r], rows of two_span contiguous elements of the I/O dtype.  When set they replace kr / qr.
  const void* c2p_scores; const void* p2c_scores;
  int64_t c2p_sb, c2p_st, c2p_sh, p2c_sb, p2c_st, p2c_sh;
  int exp_delta_max, exp_rows;
  const int32_t* seqlens;                                 // padded form, may be null
  const int32_t* cu_seqlens;                              // packed form
  int varlen;
  int n_seqs;                                             // B, or number of packed sequences
  int L;                                                  // padded length, or max_seqlen
  int64_t total_tokens;                                   // packed form: T
  int H, D;
  float sm_scale;
  int flags;
  float* lse; int64_t lse_sb, lse_sh;                     // lse[b*lse_sb + h*lse_sh + t] or null
  int32_t* status;
  void* workspace; size_t workspace_bytes;
};

void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);

int launch_bucket_table(int buckets, int max_pos, int delta_max, int16_t* out, cudaStream_t s);
int launch_relpos_project(const void* rel, const void* W, const void* bias, int two_span, int hidden,
                          int H, int D, int dtype, void* out, cudaStream_t s);
bool relpos_umma_applicable(const void* rel, const void* W, const void* out, int hidden, int D, int dtype);
int launch_relpos_project_umma(const void* rel, const void* W, const void* bias, int two_span, int hidden, int H,
                               void* out, int32_t* status, cudaStream_t s);
int launch_relpos_expand(const void* table, const int16_t* idx, int idx_delta_max, int H, int two_span, int D,
                         int dtype, int exp_delta_max, int exp_rows, void* out, cudaStream_t s);
int launch_bounded_wait_selftest(int32_t* status, int code, uint64_t limit_ns, cudaStream_t s);
int launch_attn_simt(const AttnParams& p, int dtype, cudaStream_t s);
int launch_attn_umma(const AttnParams& p, cudaStream_t s);
size_t umma_workspace_bytes(int n_seqs, int64_t total_tokens);
int static_tile_scratch(void** ptr);   // device address of the library's fixed tile-list array on the current device

}  // namespace tdb
