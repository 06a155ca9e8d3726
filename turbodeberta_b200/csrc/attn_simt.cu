// CUDA-core disentangled attention: exact fp32 arithmetic, any I/O dtype.
//
// This is the full-precision path (fp32 inputs must land within 1e-4 of the eager module, which the
// bf16 tensor-core pipeline cannot do) and the cross-check for the tensor-core kernel.  One warp owns
// one query row; lane l scores keys l, l+32, ... with its own online softmax state (max, sum, 64
// output partials) and the 32 states are merged once at the end.  All operands are read through the
// read-only cache; nothing is staged, so it is latency/L1-bound and is not the throughput path.
//
//   score[q,k] = (Q[q].K[k] + Q[q].Kr[r] + K[k].Qr[r]) * sm_scale,  r = idx[clamp(q-k)]
//
// Legacy form: the two position products arrive materialised (c2p_scores[q, r], p2c_scores[k, r]) and are only
// gathered; with TDB_FLAG_P2C_MIRRORED the p2c term is read at idx[clamp(k-q)], the reference kernel's convention.
#include "tdb_internal.h"
#include <math_constants.h>

namespace tdb {

template <typename T> __device__ __forceinline__ void load64(const T* p, float* dst);
template <> __device__ __forceinline__ void load64<float>(const float* p, float* dst) {
  const float4* p4 = reinterpret_cast<const float4*>(p);
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    float4 t = __ldg(p4 + i);
    dst[4 * i] = t.x; dst[4 * i + 1] = t.y; dst[4 * i + 2] = t.z; dst[4 * i + 3] = t.w;
  }
}
template <> __device__ __forceinline__ void load64<__nv_bfloat16>(const __nv_bfloat16* p, float* dst) {
  const uint4* p4 = reinterpret_cast<const uint4*>(p);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    uint4 t = __ldg(p4 + i);
    uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      dst[8 * i + 2 * j] = __uint_as_float(w[j] << 16);
      dst[8 * i + 2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
    }
  }
}
template <typename T> __device__ __forceinline__ T cast_out(float x);
template <> __device__ __forceinline__ float cast_out<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 cast_out<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

__device__ __forceinline__ float to_float(float x) { return x; }
__device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }

constexpr int SIMT_WARPS = 4;

template <typename T>
__global__ void __launch_bounds__(SIMT_WARPS * 32) attn_simt_kernel(const AttnParams p) {
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int s = blockIdx.z, h = blockIdx.y;
  const int qi = blockIdx.x * SIMT_WARPS + warp;
  int len, rows;                 // valid length; rows that exist in the output
  int64_t tok0; int b;
  if (p.varlen) {
    int c0 = p.cu_seqlens[s];
    len = p.cu_seqlens[s + 1] - c0; rows = len; tok0 = c0; b = 0;
    if (c0 < 0 || len < 0 || (int64_t)c0 + len > p.total_tokens) {   // malformed offsets: report, touch nothing
      if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0) atomicExch(p.status + 1, 1);
      return;
    }
    // The grid covers max_seqlen rows per sequence: a longer sequence would leave rows unwritten, and offsets that
    // do not end at the token count leave tokens outside every sequence.  Both are reported, not guessed around.
    if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 &&
        (len > p.L || (s == p.n_seqs - 1 && (int64_t)c0 + len != p.total_tokens)))
      atomicExch(p.status + 1, 1);
  } else {
    len = p.seqlens ? p.seqlens[s] : p.L; rows = p.L; tok0 = 0; b = s;
    len = len < 0 ? 0 : (len > p.L ? p.L : len);
  }
  if (qi >= rows) return;
  T* orow = reinterpret_cast<T*>(p.o) + b * p.o_sb + (tok0 + qi) * p.o_st + h * p.o_sh;
  if (qi >= len) {               // padded query row of the padded form: zeros
    orow[lane] = cast_out<T>(0.f); orow[lane + 32] = cast_out<T>(0.f);
    if (p.lse) p.lse[b * p.lse_sb + h * p.lse_sh + tok0 + qi] = 0.f;
    return;
  }
  const T* qb = reinterpret_cast<const T*>(p.q) + b * p.q_sb + (tok0 + qi) * p.q_st + h * p.q_sh;
  const T* kb = reinterpret_cast<const T*>(p.k) + b * p.k_sb + tok0 * p.k_st + h * p.k_sh;
  const T* vb = reinterpret_cast<const T*>(p.v) + b * p.v_sb + tok0 * p.v_st + h * p.v_sh;
  const bool gathered = p.c2p_scores || p.p2c_scores;
  const T* krh = (!gathered && (p.flags & TDB_FLAG_C2P)) ? reinterpret_cast<const T*>(p.kr) + (int64_t)h * p.two_span * 64 : nullptr;
  const T* qrh = (!gathered && (p.flags & TDB_FLAG_P2C)) ? reinterpret_cast<const T*>(p.qr) + (int64_t)h * p.two_span * 64 : nullptr;
  // materialised scores: this query's row of c2p, and the base of this head's p2c rows (one per key)
  const T* c2p_row = ((p.flags & TDB_FLAG_C2P) && p.c2p_scores)
      ? reinterpret_cast<const T*>(p.c2p_scores) + b * p.c2p_sb + (tok0 + qi) * p.c2p_st + h * p.c2p_sh : nullptr;
  const T* p2c_base = ((p.flags & TDB_FLAG_P2C) && p.p2c_scores)
      ? reinterpret_cast<const T*>(p.p2c_scores) + b * p.p2c_sb + tok0 * p.p2c_st + h * p.p2c_sh : nullptr;

  float qv[64], acc[64], kv[64], tv[64];
  load64<T>(qb, qv);
#pragma unroll
  for (int d = 0; d < 64; ++d) acc[d] = 0.f;
  float m = -CUDART_INF_F, l = 0.f;

  for (int kj = lane; kj < len; kj += 32) {
    load64<T>(kb + (int64_t)kj * p.k_st, kv);
    float sc = 0.f;
#pragma unroll
    for (int d = 0; d < 64; ++d) sc = fmaf(qv[d], kv[d], sc);
    if (c2p_row || p2c_base) {
      int delta = qi - kj;
      delta = delta < -p.idx_delta_max ? -p.idx_delta_max : (delta > p.idx_delta_max ? p.idx_delta_max : delta);
      if (c2p_row) sc += to_float(c2p_row[p.idx[delta + p.idx_delta_max]]);
      if (p2c_base) {
        const int r = (p.flags & TDB_FLAG_P2C_MIRRORED) ? p.idx[p.idx_delta_max - delta] : p.idx[delta + p.idx_delta_max];
        sc += to_float(p2c_base[(int64_t)kj * p.p2c_st + r]);
      }
    }
    if (krh || qrh) {
      int delta = qi - kj;
      delta = delta < -p.idx_delta_max ? -p.idx_delta_max : (delta > p.idx_delta_max ? p.idx_delta_max : delta);
      int r = p.idx[delta + p.idx_delta_max];
      if (krh) {
        load64<T>(krh + (int64_t)r * 64, tv);
        float c = 0.f;
#pragma unroll
        for (int d = 0; d < 64; ++d) c = fmaf(qv[d], tv[d], c);
        sc += c;
      }
      if (qrh) {
        load64<T>(qrh + (int64_t)r * 64, tv);
        float c = 0.f;
#pragma unroll
        for (int d = 0; d < 64; ++d) c = fmaf(kv[d], tv[d], c);
        sc += c;
      }
    }
    sc *= p.sm_scale;
    float mn = fmaxf(m, sc);
    float corr = expf(m - mn);                            // first key: m = -inf -> 0
    float pe = expf(sc - mn);
    l = l * corr + pe;
    load64<T>(vb + (int64_t)kj * p.v_st, tv);
#pragma unroll
    for (int d = 0; d < 64; ++d) acc[d] = fmaf(pe, tv[d], acc[d] * corr);
    m = mn;
  }
  // merge the 32 lane-local softmax states
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) {
    float mo = __shfl_xor_sync(0xffffffffu, m, off);
    float lo = __shfl_xor_sync(0xffffffffu, l, off);
    float mn = fmaxf(m, mo);
    float a = (m == -CUDART_INF_F) ? 0.f : expf(m - mn);
    float bb = (mo == -CUDART_INF_F) ? 0.f : expf(mo - mn);
    l = l * a + lo * bb;
#pragma unroll
    for (int d = 0; d < 64; ++d) {
      float oo = __shfl_xor_sync(0xffffffffu, acc[d], off);
      acc[d] = acc[d] * a + oo * bb;
    }
    m = mn;
  }
  float inv = 1.f / l;
  // every lane now holds the whole row; lane l writes elements l and l+32
  float o0 = 0.f, o1 = 0.f;
#pragma unroll
  for (int d = 0; d < 32; ++d) {
    if (d == lane) { o0 = acc[d]; o1 = acc[d + 32]; }
  }
  orow[lane] = cast_out<T>(o0 * inv);
  orow[lane + 32] = cast_out<T>(o1 * inv);
  if (p.lse && lane == 0) p.lse[b * p.lse_sb + h * p.lse_sh + tok0 + qi] = m + logf(l);
}

int launch_attn_simt(const AttnParams& p, int dtype, cudaStream_t s) {
  if (p.n_seqs == 0 || p.L == 0) return TDB_OK;
  dim3 grid((p.L + SIMT_WARPS - 1) / SIMT_WARPS, p.H, p.n_seqs);
  if (grid.z > 65535 || grid.y > 65535) { set_error("attn_simt: more than 65535 sequences or heads"); return TDB_ERR_SHAPE; }
  if (dtype == TDB_DTYPE_F32) attn_simt_kernel<float><<<grid, SIMT_WARPS * 32, 0, s>>>(p);
  else attn_simt_kernel<__nv_bfloat16><<<grid, SIMT_WARPS * 32, 0, s>>>(p);
  return cuda_fail(cudaGetLastError(), "attn_simt launch");
}

}  // namespace tdb
