// Relative-position projection on the tensor cores (bf16):  out[h, r, :] = rel[r, :] . W[h*64:(h+1)*64, :]^T + bias.
//
// A small tcgen05 GEMM that runs once per layer (its result is cached by the host): one CTA per (128 rows of the
// relative-embedding table, head).  A = rel tile [128 x 64k] and B = W tile [64 x 64k] are both K-major in HBM, so
// they arrive by TMA as 128-byte-swizzled tiles, four stages deep; one elected lane issues
// tcgen05.mma (M 128, N 64, K 16) into a 64-column fp32 accumulator in tensor memory; four warps read it back,
// add the bias and store bf16 rows.  Bound by HBM traffic: e * (hidden^2 + 2 * two_span * hidden) bytes per call,
// which at these sizes (a few MB) is a launch-latency-sized kernel.
#include "tdb_internal.h"
#include "ptx_sm100.cuh"
#include <cudaTypedefs.h>
#include <mutex>

namespace tdb {
using namespace ptx;

namespace {

constexpr int PM = 128, PN = 64, PK = 64, STAGES = 4;
constexpr int P_THREADS = 192;
constexpr uint32_t A_BYTES = PM * PK * 2, B_BYTES = PN * PK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr uint32_t P_OFF_BAR = STAGES * STAGE_BYTES;
constexpr uint32_t P_SMEM = P_OFF_BAR + 128 + 1024;
constexpr uint64_t P_WAIT_NS = 1000ull * 1000ull * 1000ull;

__global__ void __launch_bounds__(P_THREADS, 1)
relpos_project_umma_kernel(const __grid_constant__ CUtensorMap tm_rel, const __grid_constant__ CUtensorMap tm_w,
                           const __nv_bfloat16* __restrict__ bias, int two_span, int hidden, int H,
                           __nv_bfloat16* __restrict__ out, int32_t* status) {
  extern __shared__ uint8_t smem_raw[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int r0 = blockIdx.x * PM, h = blockIdx.y;
  const int n_k = (hidden + PK - 1) / PK;
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (sbase - smem_u32(smem_raw));
  const uint32_t bars = sbase + P_OFF_BAR;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gbase + P_OFF_BAR + 96);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbase + P_OFF_BAR + 104);
  // barriers: full[s] = 0..3, empty[s] = 4..7, accumulator ready = 8
  auto bar = [&](int i) { return bars + 8u * (uint32_t)i; };
  auto wait = [&](int i, uint32_t parity) { return mbar_wait(bar(i), parity, abort_flag, status, 100 + i, P_WAIT_NS); };

  if (tid == 0) {
    *abort_flag = 0;
    for (int i = 0; i < 2 * STAGES + 1; ++i) mbar_init(bar(i), 1u);
    fence_mbar_init();
    prefetch_tmap(&tm_rel);
    prefetch_tmap(&tm_w);
  }
  if (warp == 5) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), 64);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 4) {
    if (lane == 0) {                       // TMA producer
      for (int kc = 0; kc < n_k; ++kc) {
        const int s = kc % STAGES;
        if (kc >= STAGES) wait(STAGES + s, (uint32_t)(((kc / STAGES) - 1) & 1));
        if (*abort_flag) break;
        const uint32_t a_dst = sbase + s * STAGE_BYTES, b_dst = a_dst + A_BYTES;
        mbar_expect_tx(bar(s), STAGE_BYTES);
        asm volatile(
            "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
            ::"r"(a_dst), "l"(reinterpret_cast<uint64_t>(&tm_rel)), "r"(bar(s)), "r"(kc * PK), "r"(r0) : "memory");
        asm volatile(
            "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
            ::"r"(b_dst), "l"(reinterpret_cast<uint64_t>(&tm_w)), "r"(bar(s)), "r"(kc * PK), "r"(h * PN) : "memory");
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {                       // MMA issuer
      constexpr uint32_t IDESC = make_idesc_bf16(PM, PN, 0);
      for (int kc = 0; kc < n_k; ++kc) {
        const int s = kc % STAGES;
        wait(s, (uint32_t)((kc / STAGES) & 1));
        tc_fence_after();
        const uint64_t dA = smem_desc_sw128(sbase + s * STAGE_BYTES), dB = smem_desc_sw128(sbase + s * STAGE_BYTES + A_BYTES);
#pragma unroll
        for (int k = 0; k < PK / 16; ++k) mma_ss(tmem, dA + 2 * k, dB + 2 * k, IDESC, (kc > 0 || k > 0) ? 1u : 0u);
        tc_commit(bar(STAGES + s));        // the stage may be refilled once these products have read it
      }
      tc_commit(bar(2 * STAGES));          // accumulator complete
    }
  } else {
    // epilogue: warp w owns tensor-memory lanes 32w..32w+31 = rows r0 + 32w + lane
    wait(2 * STAGES, 0);
    tc_fence_after();
    const int r = r0 + warp * 32 + lane;
    const uint32_t taddr = tmem + (((uint32_t)(warp * 32)) << 16);
    uint32_t acc[64];
    tmem_ld32(taddr, acc);
    tmem_ld32(taddr + 32, acc + 32);
    tmem_ld_wait32(acc);
    tmem_ld_wait32(acc + 32);
    tc_fence_before();
    if (r < two_span && !*abort_flag) {
      uint4* dst = reinterpret_cast<uint4*>(out + ((int64_t)h * two_span + r) * PN);
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        uint32_t w[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = c * 8 + 2 * e;
          float b0 = 0.f, b1 = 0.f;
          if (bias) { b0 = __bfloat162float(bias[h * PN + j]); b1 = __bfloat162float(bias[h * PN + j + 1]); }
          w[e] = pack_bf16x2(__uint_as_float(acc[j]) + b0, __uint_as_float(acc[j + 1]) + b1);
        }
        dst[c] = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
  }
  if (*abort_flag) {                      // give copies that may still be in flight time to land
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 5) tmem_dealloc(tmem, 64);
}

// Self-test of the bounded wait that every hand-off of the tensor-core kernels goes through: one warp waits on an
// mbarrier that nothing will ever complete.  The wait must give up after `limit_ns`, set the abort flag, record
// `code` in the status word and return, leaving the context usable.
__global__ void __launch_bounds__(32, 1) bounded_wait_selftest_kernel(int32_t* status, int code, uint64_t limit_ns) {
  __shared__ __align__(8) uint64_t barrier_word;
  __shared__ int abort_word;
  const uint32_t b = smem_u32(&barrier_word);
  if (threadIdx.x == 0) {
    abort_word = 0;
    mbar_init(b, 1u);
    fence_mbar_init();
  }
  __syncwarp();
  const bool done = mbar_wait(b, 0u, &abort_word, status, code, limit_ns);
  if (done && threadIdx.x == 0) atomicExch(status + 3, 1);     // cannot happen: nobody arrives
}

PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  // looked up once; a function-local static's initialisation is safe against concurrent first calls
  static const PFN_cuTensorMapEncodeTiled_v12000 fn = []() -> PFN_cuTensorMapEncodeTiled_v12000 {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      return reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
    return nullptr;
  }();
  return fn;
}

int map_2d(CUtensorMap* m, const void* ptr, uint64_t cols, uint64_t rows, uint32_t box_rows, const char* what) {
  auto fn = encode_fn();
  if (!fn) { set_error("cuTensorMapEncodeTiled entry point not found"); return TDB_ERR_CUDA; }
  uint64_t dims[2] = {cols, rows};
  uint64_t strides[1] = {cols * 2};
  uint32_t box[2] = {PK, box_rows};
  uint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled(%s) failed with CUresult %d", what, (int)r); return TDB_ERR_CUDA; }
  return TDB_OK;
}

}  // namespace

// True when the tensor-core kernel applies: bf16, head_dim 64, rows of 16-byte multiples, 16-byte aligned bases.
bool relpos_umma_applicable(const void* rel, const void* W, const void* out, int hidden, int D, int dtype) {
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  return dtype == TDB_DTYPE_BF16 && D == PN && hidden % 8 == 0 && al(rel) && al(W) && al(out);
}

int launch_relpos_project_umma(const void* rel, const void* W, const void* bias, int two_span, int hidden, int H,
                               void* out, int32_t* status, cudaStream_t s) {
  CUtensorMap tm_rel, tm_w;
  int rc;
  if ((rc = map_2d(&tm_rel, rel, (uint64_t)hidden, (uint64_t)two_span, PM, "rel"))) return rc;
  if ((rc = map_2d(&tm_w, W, (uint64_t)hidden, (uint64_t)H * PN, PN, "W"))) return rc;
  {                                   // the shared-memory opt-in is a per-device attribute: set once per device
    static std::mutex mu;
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lock(mu);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
      cudaError_t e = cudaFuncSetAttribute(relpos_project_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)P_SMEM);
      if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(relpos projection)");
      if (dev >= 0 && dev < 64) configured[dev] = true;
    }
  }
  dim3 grid((two_span + PM - 1) / PM, H);
  relpos_project_umma_kernel<<<grid, P_THREADS, P_SMEM, s>>>(tm_rel, tm_w, (const __nv_bfloat16*)bias, two_span, hidden, H,
                                                             (__nv_bfloat16*)out, status);
  return cuda_fail(cudaGetLastError(), "relpos_project_umma launch");
}

int launch_bounded_wait_selftest(int32_t* status, int code, uint64_t limit_ns, cudaStream_t s) {
  bounded_wait_selftest_kernel<<<1, 32, 0, s>>>(status, code, limit_ns);
  return cuda_fail(cudaGetLastError(), "bounded-wait self-test launch");
}

}  // namespace tdb
