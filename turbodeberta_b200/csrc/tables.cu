// Small once-per-layer kernels: the distance -> table-row index, the projection of the relative
// embeddings, and the distance-expanded copies of the projected tables.
#include "tdb_internal.h"

namespace tdb {

// ---------------------------------------------------------------------------------------------
// idx[delta + delta_max] = clamp(bucket(delta) + span, 0, 2*span-1).
// The eager module (transformers modeling_deberta_v2.py:56-69) evaluates
//   ceil( log(a/mid) / log((max_pos-1)/mid) * (mid-1) ) + mid
// in float32.  The same float32 sequence is followed here (IEEE divide and multiply with
// round-to-nearest); each logarithm is taken in double and rounded once to float, which is the
// correctly rounded float32 logarithm.  HBM-bound and tiny: 2 bytes written per distance.
__global__ void bucket_table_kernel(int buckets, int max_pos, int delta_max, int16_t* __restrict__ out) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  int n = 2 * delta_max + 1;
  if (i >= n) return;
  int delta = i - delta_max;
  int span, bucket;
  if (buckets > 0 && max_pos > 0) {
    span = buckets;
    int mid = buckets / 2;
    int a = (delta < mid && delta > -mid) ? (mid - 1) : (delta < 0 ? -delta : delta);
    if (a <= mid) {
      bucket = delta;
    } else {
      float ratio = __fdiv_rn((float)a, (float)mid);
      float denom_arg = (float)((double)(max_pos - 1) / (double)mid);
      float ln = (float)log((double)ratio);
      float ld = (float)log((double)denom_arg);
      float v = __fmul_rn(__fdiv_rn(ln, ld), (float)(mid - 1));
      float lp = __fadd_rn(ceilf(v), (float)mid);
      bucket = (int)(delta < 0 ? -lp : lp);
    }
  } else {
    span = max_pos;
    bucket = delta;
  }
  int r = bucket + span;
  r = r < 0 ? 0 : (r > 2 * span - 1 ? 2 * span - 1 : r);
  out[i] = (int16_t)r;
}

int launch_bucket_table(int buckets, int max_pos, int delta_max, int16_t* out, cudaStream_t s) {
  int n = 2 * delta_max + 1;
  bucket_table_kernel<<<(n + 255) / 256, 256, 0, s>>>(buckets, max_pos, delta_max, out);
  return cuda_fail(cudaGetLastError(), "bucket_table launch");
}

// ---------------------------------------------------------------------------------------------
// out[h, r, j] = sum_c rel[r, c] * W[h*D + j, c] + bias[h*D + j], fp32 accumulation.
// A 64x64 output tile per block, 16-wide k slices staged in shared memory.  Runs once per layer
// and is cached by the host; bounded by reading W (hidden^2 elements) from HBM.
template <typename T> __device__ __forceinline__ float to_f(T x);
template <> __device__ __forceinline__ float to_f<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T from_f(float x);
template <> __device__ __forceinline__ float from_f<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

template <typename T>
__global__ void __launch_bounds__(256) relpos_project_kernel(const T* __restrict__ rel, const T* __restrict__ W,
                                                             const T* __restrict__ bias, int two_span, int hidden,
                                                             int H, int D, T* __restrict__ out) {
  constexpr int TM = 64, TN = 64, TK = 16;
  __shared__ float sa[TK][TM + 1];
  __shared__ float sb[TK][TN + 1];
  int r0 = blockIdx.x * TM;      // rows of rel
  int n0 = blockIdx.y * TN;      // output features (h*D + j)
  int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  int N = H * D;
  for (int c0 = 0; c0 < hidden; c0 += TK) {
    for (int e = threadIdx.x; e < TM * TK; e += 256) {
      int rr = e / TK, cc = e % TK;
      int r = r0 + rr, c = c0 + cc;
      sa[cc][rr] = (r < two_span && c < hidden) ? to_f<T>(rel[(int64_t)r * hidden + c]) : 0.f;
      int n = n0 + rr;
      sb[cc][rr] = (n < N && c < hidden) ? to_f<T>(W[(int64_t)n * hidden + c]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int cc = 0; cc < TK; ++cc) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = sa[cc][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = sb[cc][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int r = r0 + ty * 4 + i;
    if (r >= two_span) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      float v = acc[i][j] + (bias ? to_f<T>(bias[n]) : 0.f);
      int h = n / D, jj = n % D;
      out[((int64_t)h * two_span + r) * D + jj] = from_f<T>(v);
    }
  }
}

int launch_relpos_project(const void* rel, const void* W, const void* bias, int two_span, int hidden, int H, int D,
                          int dtype, void* out, cudaStream_t s) {
  dim3 grid((two_span + 63) / 64, (H * D + 63) / 64);
  if (dtype == TDB_DTYPE_F32)
    relpos_project_kernel<float><<<grid, 256, 0, s>>>((const float*)rel, (const float*)W, (const float*)bias,
                                                      two_span, hidden, H, D, (float*)out);
  else
    relpos_project_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)rel, (const __nv_bfloat16*)W,
                                                              (const __nv_bfloat16*)bias, two_span, hidden, H, D,
                                                              (__nv_bfloat16*)out);
  return cuda_fail(cudaGetLastError(), "relpos_project launch");
}

// ---------------------------------------------------------------------------------------------
// out[h, x, :] = bf16(table[h, idx(delta = x - exp_delta_max), :]).  One warp per output row,
// 64 elements = 2 per lane.  HBM-bound: writes H*exp_rows*D*2 bytes, reads hit L2 (compact table).
template <typename T>
__global__ void relpos_expand_kernel(const T* __restrict__ table, const int16_t* __restrict__ idx, int idx_delta_max,
                                     int H, int two_span, int D, int exp_delta_max, int exp_rows,
                                     __nv_bfloat16* __restrict__ out) {
  int warp = (blockIdx.x * blockDim.x + threadIdx.x) / 32, lane = threadIdx.x % 32;
  if (warp >= H * exp_rows) return;
  int h = warp / exp_rows, x = warp % exp_rows;
  int delta = x - exp_delta_max;
  delta = delta < -idx_delta_max ? -idx_delta_max : (delta > idx_delta_max ? idx_delta_max : delta);
  int r = idx[delta + idx_delta_max];
  const T* src = table + ((int64_t)h * two_span + r) * D;
  __nv_bfloat16* dst = out + ((int64_t)h * exp_rows + x) * D;
  for (int j = lane; j < D; j += 32) dst[j] = __float2bfloat16_rn(to_f<T>(src[j]));
}

int launch_relpos_expand(const void* table, const int16_t* idx, int idx_delta_max, int H, int two_span, int D,
                         int dtype, int exp_delta_max, int exp_rows, void* out, cudaStream_t s) {
  int64_t warps = (int64_t)H * exp_rows;
  int blocks = (int)((warps * 32 + 255) / 256);
  if (dtype == TDB_DTYPE_F32)
    relpos_expand_kernel<float><<<blocks, 256, 0, s>>>((const float*)table, idx, idx_delta_max, H, two_span, D,
                                                       exp_delta_max, exp_rows, (__nv_bfloat16*)out);
  else
    relpos_expand_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>((const __nv_bfloat16*)table, idx, idx_delta_max, H,
                                                               two_span, D, exp_delta_max, exp_rows,
                                                               (__nv_bfloat16*)out);
  return cuda_fail(cudaGetLastError(), "relpos_expand launch");
}

}  // namespace tdb
