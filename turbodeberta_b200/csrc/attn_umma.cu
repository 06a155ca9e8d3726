// Fused disentangled attention on the sm_100a tensor cores (tcgen05 UMMA, accumulators in tensor memory).
//
// One CTA = one (sequence, head, 128-query tile); it walks the sequence's keys in tiles of 128:
//
//   S  = Q . K^T                         128x128   UMMA  (A = Q tile, B = K tile, both K-major in smem)
//   C  = Q . KrX[win]^T                  128x256   UMMA  content->position band
//   P2 = K . QrX[win]^T                  128x256   UMMA  position->content band (rows = keys)
//   s[i][j] = (S[i][j] + C[i][i-j+127] + P2[j][i-j+127]) * scale ;  mask ;  online softmax
//   O += P . V                           128x64    UMMA  (A = P as bf16 in tensor memory, B = V tile, MN-major)
//
// KrX / QrX are the distance-expanded tables (row x <-> distance x - exp_delta_max), so the rows a tile
// needs are the contiguous window win = [q0 - k0 - 127 + exp_delta_max, +256), one TMA box.  The diagonal
// read C[i][i-j+127] cannot be done from registers (the column depends on the lane), so both bands are
// drained from tensor memory to shared memory as bf16 rows and read back skewed: the c2p row belongs to
// the reading thread; the p2c rows are written by the thread that owns the key and read by every query.
//
// Warp roles (192 threads): warps 0-3 = drain + softmax + epilogue (thread t owns query row t and
// tensor-memory lane t), warp 4 = TMA producer (one lane), warp 5 = tensor-memory allocation + MMA issue
// (one lane).  All hand-offs are mbarriers with bounded waits; a wait that gives up sets a CTA-wide abort
// flag and the status word, after which every role keeps walking its loop without waiting so that the
// CTA-wide barriers still match, tensor memory is freed, and the host reports TDB_ERR_TIMEOUT.
//
// Tensor-memory columns: [0,128) S (P overlays [0,64) once S is in registers), [128,192) O, [256,512) band.
#include "tdb_internal.h"
#include "ptx_sm100.cuh"
#include <cudaTypedefs.h>
#include <math_constants.h>
#include <mutex>

namespace tdb {
using namespace ptx;

namespace {

constexpr int BQ = 128, BK = 128, HD = 64, BAND = 256;
constexpr int NTHREADS = 192;
constexpr int STG_STRIDE = 336;                 // bytes per staging row: 160 bf16 + 16 pad (odd multiple of 16)
constexpr int STG_COLS = 160;
constexpr uint32_t OFF_Q = 0, OFF_K = 16384, OFF_V = 32768, OFF_KR = 49152, OFF_QR = 81920;
constexpr uint32_t OFF_STC = 114688, OFF_STP = OFF_STC + BQ * STG_STRIDE, OFF_BAR = OFF_STP + BK * STG_STRIDE;
constexpr uint32_t SMEM_BYTES = OFF_BAR + 256 + 1024;   // + slack for the 1024-byte alignment of the base
static_assert(OFF_STP % 16 == 0 && OFF_BAR % 16 == 0, "staging offsets must stay 16-byte aligned");
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");

constexpr uint32_t TM_S = 0, TM_O = 128, TM_BAND = 256, TM_COLS = 512;
constexpr uint64_t WAIT_LIMIT_NS = 1000ull * 1000ull * 1000ull;   // 1 s per wait, then give up

enum Bar { Q_FULL = 0, K_FULL, K_EMPTY, V_FULL, V_EMPTY, KR_FULL, KR_EMPTY, QR_FULL, QR_EMPTY,
           SC_FULL, BAND_FREE, P2_FULL, P_READY, O_FULL, DONE, NBARS };

struct TileListHeader { int32_t n_tiles; int32_t pad[3]; };

// ---------------------------------------------------------------------------------------------
// Packed form: list of (sequence, first query row) per 128-row tile, built on the device from
// cu_seqlens so that the host never reads lengths back.  Also validates cu_seqlens: a negative
// length or an offset outside [0, T] sets status[1] and the sequence is dropped.
__global__ void __launch_bounds__(1024) build_tile_list_kernel(const int32_t* __restrict__ cu, int n_seqs,
                                                                int64_t total_tokens, int32_t* ws, int cap,
                                                                int32_t* status) {
  __shared__ int scan[1024];
  __shared__ int running;
  if (threadIdx.x == 0) running = 0;
  __syncthreads();
  int2* entries = reinterpret_cast<int2*>(ws + 4);
  for (int base = 0; base < n_seqs; base += 1024) {
    int s = base + threadIdx.x;
    int len = 0, nt = 0;
    if (s < n_seqs) {
      int a = cu[s], b = cu[s + 1];
      if (a < 0 || b < a || (int64_t)b > total_tokens) { atomicExch(status + 1, 1); }
      else { len = b - a; nt = (len + BQ - 1) / BQ; }
    }
    scan[threadIdx.x] = nt;
    __syncthreads();
    for (int off = 1; off < 1024; off <<= 1) {
      int v = threadIdx.x >= off ? scan[threadIdx.x - off] : 0;
      __syncthreads();
      scan[threadIdx.x] += v;
      __syncthreads();
    }
    int start = running + scan[threadIdx.x] - nt;
    for (int t = 0; t < nt; ++t)
      if (start + t < cap) entries[start + t] = make_int2(s, t * BQ);
    __syncthreads();
    if (threadIdx.x == 1023) running += scan[1023];
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    if (cu[n_seqs] != (int32_t)total_tokens) atomicExch(status + 1, 1);
    ws[0] = running < cap ? running : cap;
  }
}

__device__ __forceinline__ float bf16_bits_to_float(uint32_t u16) { return __uint_as_float(u16 << 16); }

__device__ __forceinline__ float lds_bf16(uint32_t addr) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
  return bf16_bits_to_float((uint32_t)v);
}
__device__ __forceinline__ void sts_128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void named_bar_sync_128() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Move STG_COLS fp32 columns of this thread's tensor-memory lane, starting at `taddr`, to one bf16 staging row.
__device__ __forceinline__ void drain_band_row(uint32_t taddr, uint32_t row_saddr) {
#pragma unroll
  for (int c = 0; c < STG_COLS / 32; ++c) {
    uint32_t r[32];
    tmem_ld32(taddr + c * 32, r);
    tmem_ld_wait32(r);
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      uint32_t w[4];
#pragma unroll
      for (int e = 0; e < 4; ++e)
        w[e] = pack_bf16x2(__uint_as_float(r[g * 8 + 2 * e]), __uint_as_float(r[g * 8 + 2 * e + 1]));
      sts_128(row_saddr + c * 64 + g * 16, w[0], w[1], w[2], w[3]);
    }
  }
}

template <bool C2P, bool P2C>
__global__ void __launch_bounds__(NTHREADS, 1)
attn_umma_kernel(const AttnParams p, const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_kr,
                 const __grid_constant__ CUtensorMap tm_qr) {
  extern __shared__ uint8_t smem_raw[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h = blockIdx.y;

  // ---- which tile --------------------------------------------------------------------------
  int seq, q0, len, rows, bcoord; int64_t tok0;
  if (p.varlen) {
    const int32_t* ws = reinterpret_cast<const int32_t*>(p.workspace);
    if ((int)blockIdx.x >= ws[0]) return;
    int2 e = reinterpret_cast<const int2*>(ws + 4)[blockIdx.x];
    seq = e.x; q0 = e.y;
    int c0 = p.cu_seqlens[seq];
    len = p.cu_seqlens[seq + 1] - c0; rows = len; tok0 = c0; bcoord = 0;
  } else {
    int qtiles = (p.L + BQ - 1) / BQ;
    seq = blockIdx.x / qtiles; q0 = (blockIdx.x % qtiles) * BQ;
    len = p.seqlens ? p.seqlens[seq] : p.L;
    len = len < 0 ? 0 : (len > p.L ? p.L : len);
    rows = p.L; tok0 = 0; bcoord = seq;
  }
  __nv_bfloat16* obase = reinterpret_cast<__nv_bfloat16*>(p.o) + (int64_t)bcoord * p.o_sb + (tok0 + q0) * p.o_st + (int64_t)h * p.o_sh;
  if (q0 >= len) {                       // tile of padded query rows only: zeros, no tensor work
    if (tid < BQ && q0 + tid < rows) {
      uint4 z = make_uint4(0, 0, 0, 0);
      uint4* dst = reinterpret_cast<uint4*>(obase + (int64_t)tid * p.o_st);
#pragma unroll
      for (int i = 0; i < 8; ++i) dst[i] = z;
      if (p.lse) p.lse[(int64_t)bcoord * p.lse_sb + (int64_t)h * p.lse_sh + tok0 + q0 + tid] = 0.f;
    }
    return;
  }
  {                                      // an earlier CTA gave up: do not start (decided once per CTA)
    __shared__ int s_skip;
    if (tid == 0) s_skip = (*reinterpret_cast<volatile int32_t*>(p.status) != 0) ? 1 : 0;
    __syncthreads();
    if (s_skip) return;
  }
  const int n_kv = (len + BK - 1) / BK;

  // ---- shared memory carve-up ----------------------------------------------------------------
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (sbase - smem_u32(smem_raw));
  const uint32_t sQ = sbase + OFF_Q, sK = sbase + OFF_K, sV = sbase + OFF_V, sKr = sbase + OFF_KR, sQr = sbase + OFF_QR;
  const uint32_t stC = sbase + OFF_STC, stP = sbase + OFF_STP;
  const uint32_t bars = sbase + OFF_BAR;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gbase + OFF_BAR + 128);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbase + OFF_BAR + 136);
  auto bar = [&](int i) { return bars + 8u * (uint32_t)i; };
  auto wait = [&](int i, uint32_t parity) { return mbar_wait(bar(i), parity, abort_flag, p.status, 1 + i, WAIT_LIMIT_NS); };

  if (tid == 0) {
    *abort_flag = 0;
    for (int i = 0; i < NBARS; ++i) mbar_init(bar(i), (i == BAND_FREE || i == P_READY) ? 128u : 1u);
    fence_mbar_init();
  }
  if (warp == 4 && lane == 0) {
    prefetch_tmap(&tm_q); prefetch_tmap(&tm_k); prefetch_tmap(&tm_v);
    if (C2P) prefetch_tmap(&tm_kr);
    if (P2C) prefetch_tmap(&tm_qr);
  }
  if (warp == 5) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), TM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 4) {
    // ================================ TMA producer ==========================================
    if (lane == 0) {
      mbar_expect_tx(bar(Q_FULL), BQ * HD * 2);
      tma_load_4d(sQ, &tm_q, bar(Q_FULL), 0, (int)(tok0 + q0), h, bcoord);
      for (int it = 0; it < n_kv; ++it) {
        const int k0 = it * BK;
        const uint32_t pe = (uint32_t)((it - 1) & 1);
        int x0 = q0 - k0 - (BK - 1) + p.exp_delta_max;
        x0 = x0 < 0 ? 0 : (x0 > p.exp_rows - BAND ? p.exp_rows - BAND : x0);
        if (C2P) {
          if (it > 0) wait(KR_EMPTY, pe);
          if (!*abort_flag) {
            mbar_expect_tx(bar(KR_FULL), BAND * HD * 2);
            tma_load_3d(sKr, &tm_kr, bar(KR_FULL), 0, x0, h);
          }
        }
        if (it > 0) wait(K_EMPTY, pe);
        if (!*abort_flag) {
          mbar_expect_tx(bar(K_FULL), BK * HD * 2);
          tma_load_4d(sK, &tm_k, bar(K_FULL), 0, (int)(tok0 + k0), h, bcoord);
        }
        if (P2C) {
          if (it > 0) wait(QR_EMPTY, pe);
          if (!*abort_flag) {
            mbar_expect_tx(bar(QR_FULL), BAND * HD * 2);
            tma_load_3d(sQr, &tm_qr, bar(QR_FULL), 0, x0, h);
          }
        }
        if (it > 0) wait(V_EMPTY, pe);
        if (!*abort_flag) {
          mbar_expect_tx(bar(V_FULL), BK * HD * 2);
          tma_load_4d(sV, &tm_v, bar(V_FULL), 0, (int)(tok0 + k0), h, bcoord);
        }
      }
    }
  } else if (warp == 5) {
    // ================================ MMA issuer ============================================
    if (lane == 0) {
      constexpr uint32_t ID_S = make_idesc_bf16(128, BK, 0);
      constexpr uint32_t ID_BAND = make_idesc_bf16(128, BAND, 0);
      constexpr uint32_t ID_PV = make_idesc_bf16(128, HD, 1);
      const uint64_t dQ = smem_desc_sw128(sQ), dK = smem_desc_sw128(sK), dV = smem_desc_sw128(sV);
      const uint64_t dKr = smem_desc_sw128(sKr), dQr = smem_desc_sw128(sQr);
      const uint32_t tS = tmem + TM_S, tO = tmem + TM_O, tB = tmem + TM_BAND;
      int band_n = 0;
      wait(Q_FULL, 0);
      for (int it = 0; it < n_kv; ++it) {
        const uint32_t ph = (uint32_t)(it & 1);
        wait(K_FULL, ph);
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) mma_ss(tS, dQ + 2 * k, dK + 2 * k, ID_S, k > 0);
        if (C2P) {
          wait(KR_FULL, ph);
          if (band_n > 0) wait(BAND_FREE, (uint32_t)((band_n - 1) & 1));
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < HD / 16; ++k) mma_ss(tB, dQ + 2 * k, dKr + 2 * k, ID_BAND, k > 0);
          ++band_n;
        }
        tc_commit(bar(SC_FULL));
        if (C2P) tc_commit(bar(KR_EMPTY));
        if (P2C) {
          wait(QR_FULL, ph);
          if (band_n > 0) wait(BAND_FREE, (uint32_t)((band_n - 1) & 1));
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < HD / 16; ++k) mma_ss(tB, dK + 2 * k, dQr + 2 * k, ID_BAND, k > 0);
          ++band_n;
          tc_commit(bar(P2_FULL));
          tc_commit(bar(QR_EMPTY));
        }
        tc_commit(bar(K_EMPTY));
        wait(V_FULL, ph);
        wait(P_READY, ph);
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < BK / 16; ++k)
          mma_ts(tO, tS + 8 * k, dV + (uint64_t)(128 * k), ID_PV, (it > 0 || k > 0) ? 1u : 0u);
        tc_commit(bar(O_FULL));
        tc_commit(bar(V_EMPTY));
      }
      // Everything issued above must have retired before tensor memory is released.
      tc_commit(bar(DONE));
      int never = 0;                       // this wait runs even after an abort, with its own limit
      mbar_wait(bar(DONE), 0, &never, p.status, 1 + DONE, WAIT_LIMIT_NS);
    }
  } else {
    // ================================ drain + softmax + epilogue ============================
    const uint32_t lane_base = ((uint32_t)(warp * 32)) << 16;
    const uint32_t tS = tmem + lane_base + TM_S, tO = tmem + lane_base + TM_O, tB = tmem + lane_base + TM_BAND;
    const float sl2 = p.sm_scale * 1.4426950408889634f;
    const uint32_t c_row = stC + (uint32_t)tid * STG_STRIDE;          // this thread's c2p staging row
    const uint32_t p_row = stP + (uint32_t)tid * STG_STRIDE;          // the p2c staging row of key `tid`
    const uint32_t c_read = c_row + 2u * (uint32_t)lane + 2u * (BK - 1);   // element for j is at c_read - 2*j
    const uint32_t p_read = stP + 2u * (uint32_t)tid + 62u;           // element for j is at p_read + j*STRIDE - 2*(j%32)
    float m_run = -CUDART_INF_F, l_run = 0.f;

    for (int it = 0; it < n_kv; ++it) {
      const uint32_t ph = (uint32_t)(it & 1);
      const int nvalid = len - it * BK;                               // >= 1; keys j >= nvalid are masked
      wait(SC_FULL, ph);
      tc_fence_after();
      if (C2P) {
        drain_band_row(tB + (uint32_t)(warp * 32), c_row);             // columns [32w, 32w+160)
        tc_fence_before();
        mbar_arrive(bar(BAND_FREE));
      }
      if (P2C) {
        wait(P2_FULL, ph);
        tc_fence_after();
        named_bar_sync_128();                                          // readers of the previous tile are done
        drain_band_row(tB + (uint32_t)(96 - warp * 32), p_row);        // columns [96-32w, 256-32w)
        tc_fence_before();
        mbar_arrive(bar(BAND_FREE));
        named_bar_sync_128();                                          // all key rows are visible
      }
      float s[BK];
      {
        uint32_t* sr = reinterpret_cast<uint32_t*>(s);
        tmem_ld32(tS + 0, sr + 0); tmem_ld32(tS + 32, sr + 32); tmem_ld32(tS + 64, sr + 64); tmem_ld32(tS + 96, sr + 96);
        tmem_ld_wait32(sr + 0); tmem_ld_wait32(sr + 32); tmem_ld_wait32(sr + 64); tmem_ld_wait32(sr + 96);
      }
      float mx = -CUDART_INF_F;
      if (nvalid >= BK) {
#pragma unroll
        for (int j = 0; j < BK; ++j) {
          float x = s[j];
          if (C2P) x += lds_bf16(c_read - 2u * j);
          if (P2C) x += lds_bf16(p_read + (uint32_t)(j * STG_STRIDE - 2 * (j & 31)));
          x *= sl2;
          s[j] = x;
          mx = fmaxf(mx, x);
        }
      } else {
#pragma unroll
        for (int j = 0; j < BK; ++j) {
          float x = s[j];
          if (C2P) x += lds_bf16(c_read - 2u * j);
          if (P2C) x += lds_bf16(p_read + (uint32_t)(j * STG_STRIDE - 2 * (j & 31)));
          x = (j < nvalid) ? x * sl2 : -CUDART_INF_F;
          s[j] = x;
          mx = fmaxf(mx, x);
        }
      }
      const float m_new = fmaxf(m_run, mx);
      const float alpha = ex2(m_run - m_new);
      if (it > 0) {
        wait(O_FULL, (uint32_t)((it - 1) & 1));
        tc_fence_after();
        if (__any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            uint32_t r[32];
            tmem_ld32(tO + c * 32, r);
            tmem_ld_wait32(r);
#pragma unroll
            for (int e = 0; e < 32; ++e) r[e] = __float_as_uint(__uint_as_float(r[e]) * alpha);
            tmem_st32(tO + c * 32, r);
          }
        }
      }
      float lsum = 0.f;
      uint32_t pk[BK / 2];
#pragma unroll
      for (int j = 0; j < BK; j += 2) {
        float a = ex2(s[j] - m_new), b = ex2(s[j + 1] - m_new);
        lsum += a + b;
        pk[j / 2] = pack_bf16x2(a, b);
      }
      l_run = l_run * alpha + lsum;
      m_run = m_new;
      tmem_st32(tS + 0, pk);
      tmem_st32(tS + 32, pk + 32);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(bar(P_READY));
    }
    // ---- epilogue: O / l -> global ----
    wait(O_FULL, (uint32_t)((n_kv - 1) & 1));
    tc_fence_after();
    const int row = q0 + tid;
    const float inv = 1.f / l_run;
    uint32_t outw[HD / 2];
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      uint32_t r[32];
      tmem_ld32(tO + c * 32, r);
      tmem_ld_wait32(r);
#pragma unroll
      for (int e = 0; e < 32; e += 2)
        outw[c * 16 + e / 2] = pack_bf16x2(__uint_as_float(r[e]) * inv, __uint_as_float(r[e + 1]) * inv);
    }
    tc_fence_before();
    if (row < rows) {
      const bool valid = row < len;
      uint4* dst = reinterpret_cast<uint4*>(obase + (int64_t)tid * p.o_st);
#pragma unroll
      for (int i = 0; i < 8; ++i)
        dst[i] = valid ? make_uint4(outw[4 * i], outw[4 * i + 1], outw[4 * i + 2], outw[4 * i + 3]) : make_uint4(0, 0, 0, 0);
      if (p.lse)
        p.lse[(int64_t)bcoord * p.lse_sb + (int64_t)h * p.lse_sh + tok0 + row] =
            valid ? (m_run * 0.6931471805599453f + logf(l_run)) : 0.f;
    }
  }

  // ---- teardown ------------------------------------------------------------------------------
  if (*abort_flag) {                      // give copies that may still be in flight time to land
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 5) tmem_dealloc(tmem, TM_COLS);
}

// ---------------------------------------------------------------------------------------------
PFN_cuTensorMapEncodeTiled_v12000 get_encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
  }
  return fn;
}

int encode_map(CUtensorMap* m, const void* ptr, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
               const uint32_t* box, const char* what) {
  auto fn = get_encode_fn();
  if (!fn) { set_error("cuTensorMapEncodeTiled entry point not found"); return TDB_ERR_CUDA; }
  uint32_t estr[5] = {1, 1, 1, 1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(ptr), dims, strides_bytes, box,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled(%s) failed with CUresult %d", what, (int)r); return TDB_ERR_CUDA; }
  return TDB_OK;
}

int token_map(CUtensorMap* m, const void* ptr, int64_t tokens, int H, int B, int64_t sb, int64_t st, int64_t sh,
              const char* what) {
  uint64_t dims[4] = {(uint64_t)HD, (uint64_t)tokens, (uint64_t)H, (uint64_t)(B > 0 ? B : 1)};
  uint64_t sbb = (B > 1 && sb > 0) ? (uint64_t)sb * 2 : (uint64_t)tokens * (uint64_t)st * 2;
  uint64_t strides[3] = {(uint64_t)st * 2, (uint64_t)sh * 2, sbb};
  uint32_t box[4] = {HD, BQ, 1, 1};
  return encode_map(m, ptr, 4, dims, strides, box, what);
}

int table_map(CUtensorMap* m, const void* ptr, int rows, int H, const char* what) {
  uint64_t dims[3] = {(uint64_t)HD, (uint64_t)rows, (uint64_t)H};
  uint64_t strides[2] = {(uint64_t)HD * 2, (uint64_t)rows * HD * 2};
  uint32_t box[3] = {HD, BAND, 1};
  return encode_map(m, ptr, 3, dims, strides, box, what);
}

template <bool C2P, bool P2C>
int launch_variant(const AttnParams& p, dim3 grid, const CUtensorMap* maps, cudaStream_t s) {
  auto kern = attn_umma_kernel<C2P, P2C>;
  static bool configured = false;           // per instantiation; attribute is per device, set on every device change
  static int configured_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured || configured_dev != dev) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
    if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(max dynamic shared memory)");
    configured = true; configured_dev = dev;
  }
  kern<<<grid, NTHREADS, SMEM_BYTES, s>>>(p, maps[0], maps[1], maps[2], maps[3], maps[4]);
  return cuda_fail(cudaGetLastError(), "attn_umma launch");
}

}  // namespace

// Fixed tile-list storage for tdb_attn_fwd_varlen_static: lives in the library image on every device that loads
// it.  In host code the name below is only a stand-in for the symbol, not a device address; the address comes
// from cudaGetSymbolAddress, looked up once per device with that device current.
static __device__ __align__(256) unsigned char g_static_tile_scratch[TDB_STATIC_SCRATCH_BYTES];

int static_tile_scratch(void** ptr) {
  constexpr int MAX_DEV = 64;
  static void* addr[MAX_DEV] = {nullptr};
  static std::mutex mu;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  if (dev < 0 || dev >= MAX_DEV) { set_error("device ordinal %d out of range", dev); return TDB_ERR_UNSUPPORTED; }
  std::lock_guard<std::mutex> lock(mu);
  if (!addr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_tile_scratch);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(static tile scratch)");
    if (!p) { set_error("cudaGetSymbolAddress returned a null address"); return TDB_ERR_CUDA; }
    addr[dev] = p;
  }
  *ptr = addr[dev];
  return TDB_OK;
}

size_t umma_workspace_bytes(int n_seqs, int64_t total_tokens) {
  int64_t cap = (total_tokens + BQ - 1) / BQ + n_seqs + 1;
  return sizeof(TileListHeader) + (size_t)cap * sizeof(int2);
}

int launch_attn_umma(const AttnParams& p, cudaStream_t s) {
  if (p.H > 65535) { set_error("more than 65535 heads"); return TDB_ERR_SHAPE; }
  CUtensorMap maps[5];
  memset(maps, 0, sizeof(maps));
  const int64_t tokens = p.varlen ? p.total_tokens : p.L;
  const int B = p.varlen ? 1 : p.n_seqs;
  int rc;
  if ((rc = token_map(&maps[0], p.q, tokens, p.H, B, p.q_sb, p.q_st, p.q_sh, "q"))) return rc;
  if ((rc = token_map(&maps[1], p.k, tokens, p.H, B, p.k_sb, p.k_st, p.k_sh, "k"))) return rc;
  if ((rc = token_map(&maps[2], p.v, tokens, p.H, B, p.v_sb, p.v_st, p.v_sh, "v"))) return rc;
  if (p.flags & TDB_FLAG_C2P) { if ((rc = table_map(&maps[3], p.kr_exp, p.exp_rows, p.H, "kr_exp"))) return rc; }
  else maps[3] = maps[0];
  if (p.flags & TDB_FLAG_P2C) { if ((rc = table_map(&maps[4], p.qr_exp, p.exp_rows, p.H, "qr_exp"))) return rc; }
  else maps[4] = maps[0];

  dim3 grid;
  if (p.varlen) {
    int64_t cap = (p.total_tokens + BQ - 1) / BQ + p.n_seqs + 1;
    if (cap > 0x7fffffff) { set_error("too many tiles"); return TDB_ERR_SHAPE; }
    build_tile_list_kernel<<<1, 1024, 0, s>>>(p.cu_seqlens, p.n_seqs, p.total_tokens,
                                              reinterpret_cast<int32_t*>(p.workspace), (int)cap, p.status);
    if ((rc = cuda_fail(cudaGetLastError(), "build_tile_list launch"))) return rc;
    grid = dim3((unsigned)cap, (unsigned)p.H, 1);
  } else {
    int64_t tiles = (int64_t)p.n_seqs * ((p.L + BQ - 1) / BQ);
    if (tiles > 0x7fffffff) { set_error("too many tiles"); return TDB_ERR_SHAPE; }
    grid = dim3((unsigned)tiles, (unsigned)p.H, 1);
  }
  const bool c2p = p.flags & TDB_FLAG_C2P, p2c = p.flags & TDB_FLAG_P2C;
  if (c2p && p2c) return launch_variant<true, true>(p, grid, maps, s);
  if (c2p) return launch_variant<true, false>(p, grid, maps, s);
  if (p2c) return launch_variant<false, true>(p, grid, maps, s);
  return launch_variant<false, false>(p, grid, maps, s);
}

}  // namespace tdb
