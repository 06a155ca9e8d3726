// Stand-alone timing kernel (not part of the library): does a running stream of tcgen05 products slow the CUDA-core
// loops beside it, and vice versa?  One CTA on one SM.  Sixteen warps repeat the attention kernel's exponential loop
// (skewed two-byte shared loads, mixed-precision adds, exponentials, bf16 packing, one block-wide barrier per "tile")
// while one lane of another warp issues tcgen05.mma products back to back, with the attention kernel's operand layouts,
// and never waits for them; the loop runs a fixed number of tiles, then tells the issuing lane to stop.
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o contend shared_port_contention.cu && ./contend
#include <cstdio>
#include <cstdint>
#include <cuda_runtime.h>
#include "../ptx_sm100.cuh"
using namespace tdb::ptx;
constexpr int STG_STRIDE = 336, KPT = 32;
__device__ __forceinline__ float add_bf16(float x, uint16_t h) { float y; asm("add.rn.f32.bf16 %0, %1, %2;" : "=f"(y) : "h"(h), "f"(x)); return y; }
__device__ __forceinline__ uint16_t lds_u16(uint32_t a) { uint16_t v; asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a)); return v; }

// LOOP: 0 = exponential loop with shared loads, 1 = the same without loads, 2 = loads + adds only
// MMA: 0 none, 1 = band-like SS products (N 256), 2 = score-like SS (N 128), 3 = P.V-like TS (A in tensor memory)
template <int LOOP, int MMA>
__global__ void __launch_bounds__(576, 1) k(long long* out, float* sink, int tiles, float sl2) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) unsigned long long bars[2];
  __shared__ uint32_t slot;
  __shared__ volatile int stop;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* g = smem_raw + (sbase - smem_u32(smem_raw));
  for (int i = tid; i < (160 * 1024) / 4; i += 576) reinterpret_cast<uint32_t*>(g)[i] = 0x3c003c00u + (i & 1023);
  if (tid == 0) { stop = 0; mbar_init(smem_u32(&bars[0]), 1u << 20); fence_mbar_init(); }
  if (warp == 16) { tmem_alloc(smem_u32(&slot), 512); tmem_relinquish(); }
  tc_fence_before(); __syncthreads(); tc_fence_after();
  const uint32_t tmem = slot;
  if (warp == 17) {
    if (lane == 0 && MMA > 0) {
      const uint64_t dA = smem_desc_sw128(sbase), dB = smem_desc_sw128(sbase + 16384), dV = smem_desc_sw128(sbase + 65536);
      const uint32_t i128 = make_idesc_bf16(128, 128, 0), i256 = make_idesc_bf16(128, 256, 0), ipv = make_idesc_bf16(128, 64, 1);
      long long n = 0, t0 = clock64();
      while (!stop) {
        if (MMA == 1) { for (int kk = 0; kk < 4; ++kk) mma_ss(tmem + 192, dA + 2 * kk, dB + 2 * kk, i256, kk > 0); }
        if (MMA == 2) { for (int kk = 0; kk < 4; ++kk) mma_ss(tmem, dA + 2 * kk, dB + 2 * kk, i128, kk > 0); }
        if (MMA == 3) { for (int kk = 0; kk < 8; ++kk) mma_ts(tmem + 128, tmem + 448 + 8 * kk, dV + (uint64_t)(128 * kk), ipv, 1u); }
        ++n;
      }
      out[2] = clock64() - t0; out[3] = n;
      tc_commit(smem_u32(&bars[0]));
      long long t = clock64(); while (clock64() - t < 200000) {}      // let everything retire
    }
  } else if (warp < 16) {
    const int qd = warp & 3, grp = warp >> 2, row_t = qd * 32 + lane;
    const uint32_t stP = sbase + 98304;
    const uint32_t p_read = stP + (uint32_t)(KPT * grp) * STG_STRIDE + 2u * (uint32_t)(row_t + 31);
    float s[KPT];
#pragma unroll
    for (int e = 0; e < KPT; ++e) s[e] = 0.01f * (e + lane);
    float lacc = 0.f; uint32_t pacc = 0;
    long long t0 = clock64();
    for (int t = 0; t < tiles; ++t) {
      float lsum = 0.f; uint32_t pk[KPT / 2];
#pragma unroll
      for (int e = 0; e < KPT; e += 2) {
        float x0 = s[e], x1 = s[e + 1];
        if (LOOP != 1) {
          x0 = add_bf16(x0, lds_u16(p_read + (uint32_t)(e * STG_STRIDE - 2 * (e & 31))));
          x1 = add_bf16(x1, lds_u16(p_read + (uint32_t)((e + 1) * STG_STRIDE - 2 * ((e + 1) & 31))));
        }
        s[e] = x0 * 0.999f; s[e + 1] = x1 * 0.999f;
        if (LOOP == 2) { lsum += x0 + x1; pk[e / 2] = pack_bf16x2(x0, x1); }
        else { const float a = ex2(fmaf(x0, sl2, -0.25f)), b = ex2(fmaf(x1, sl2, -0.25f)); lsum += a + b; pk[e / 2] = pack_bf16x2(a, b); }
      }
#pragma unroll
      for (int e = 0; e < KPT / 2; ++e) pacc ^= pk[e];
      lacc += lsum;
      asm volatile("bar.sync 1, 512;" ::: "memory");
    }
    if (tid == 0) { out[0] = clock64() - t0; stop = 1; }
    if (lacc == 1.2345f || pacc == 77u) sink[tid] = lacc;
  }
  tc_fence_before(); __syncthreads(); tc_fence_after();
  if (warp == 16) tmem_dealloc(tmem, 512);
}
template <int LOOP, int MMA> void run(const char* name, long long* out, float* sink) {
  cudaMemset(out, 0, 64);
  cudaFuncSetAttribute(k<LOOP, MMA>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  const int tiles = 2000;
  k<LOOP, MMA><<<1, 576, 200 * 1024>>>(out, sink, tiles, 0.1f);
  cudaError_t e = cudaDeviceSynchronize();
  long long h[4]; cudaMemcpy(h, out, 32, cudaMemcpyDeviceToHost);
  printf("%-58s %s  loop %6.0f cycles/tile", name, cudaGetErrorString(e), (double)h[0] / tiles);
  if (MMA) printf("   MMA batch every %6.0f cycles", (double)h[2] / (double)(h[3] ? h[3] : 1));
  printf("\n");
}
int main() {
  long long* out; float* sink; cudaMalloc(&out, 64); cudaMalloc(&sink, 4096);
  run<0, 0>("exp loop with shared loads, no MMA", out, sink);
  run<0, 1>("exp loop with shared loads + band products (4 x N256)", out, sink);
  run<0, 2>("exp loop with shared loads + score products (4 x N128)", out, sink);
  run<0, 3>("exp loop with shared loads + P.V products (8 x N64, TS)", out, sink);
  run<1, 0>("exp loop without loads, no MMA", out, sink);
  run<1, 1>("exp loop without loads + band products", out, sink);
  run<2, 0>("loads + adds only, no MMA", out, sink);
  run<2, 1>("loads + adds only + band products", out, sink);
  run<2, 2>("loads + adds only + score products", out, sink);
  return 0;
}
