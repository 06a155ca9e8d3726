// Fused disentangled attention on the sm_100a tensor cores (tcgen05 UMMA, accumulators in tensor memory).
//
// Persistent kernel, one CTA per SM.  A work item is one (sequence, head, 128-query tile); the CTA walks the
// sequence's keys in tiles of 128:
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
// drained from tensor memory to shared memory as bf16 rows and read back skewed.  Tiles whose distances are all
// saturated (long-sequence variant of the kernel) use one table row for every score, and the tables repeat that row
// over their saturated ends, so both position terms become two more products into the score accumulator itself
// (operands = 128-row boxes of identical rows): such tiles have no band, no drain and no gather.
//
// Warp roles (608 threads): warps 0-15 do the CUDA-core work; warp w owns tensor-memory lanes 32*(w%4)..+31
// (query rows, or key rows of P2) and column group w/4, i.e. four threads share a query row and each handles 32
// of the 128 keys, which puts four warps on every scheduler to hide latency.  Warp 16 = TMA producers (lane 0:
// tables and K, lane 1: V, lane 2: Q), warp 17 = tensor-memory allocation + MMA issue (one lane), warp 18 =
// scheduler (draws work items from a device-wide counter, publishes them in a shared-memory ring of three, zeroes tiles
// that consist of padded rows only; in the padded form it hands the sequences out longest first, so that the items
// with the most key tiles are not the ones that finish last).
//
// Pipeline: the MMA lane issues C(0) | S(0) P2(0) C(1) | S(1) P2(1) PV(0) C(2) | ..., so the bands and scores of the
// next key tile are produced while the CUDA warps work on tile g; C and P2 pass through the one band buffer in tensor
// memory (one full/free barrier pair), each drained to its staging rows - 40 columns per warp - before the other is
// issued.  The CUDA warps walk one flat stream of key tiles across work items with two CTA-wide barriers per tile:
//   phase 1  add the c2p term (skewed 32-bit reads of the thread's own staging row); between the steps of that loop the
//            warp drains its share of THIS tile's p2c band, eight columns at a time (which frees the band buffer for
//            the next tile's c2p band)                                                        -> barrier
//   phase 2  add the p2c term and take the exponentials against the reference exponent of the tiles before; P goes to
//            tensor memory eight keys at a time as it is formed; in the second half of the loop the warp drains its
//            share of the NEXT tile's c2p band the same way                                   -> voting barrier
//   then     only if some row has to move its exponent: exchange maxima, form P again, rescale O; announce P.
// Fusing the drains into the two loops hides the tensor-memory load latency behind arithmetic that has issue slots to
// spare, and leaves each band product a whole phase of the CUDA warps to complete in.
// The epilogue of an item (O / l, staged in shared memory so that whole 128-byte rows are stored) runs inside the first
// tile of the next item, where the wait for its last P.V product costs nothing.
// All hand-offs are mbarriers with bounded waits; a wait that gives up sets a CTA-wide abort flag and the status
// word, after which every role runs out its loops without waiting (the CUDA warps take their trip counts from
// one copy of the work items kept by thread 0, so their named barriers still match), tensor memory is freed, and
// the host reports TDB_ERR_TIMEOUT.
//
// Rows of K and V beyond a sequence's length are padding and may hold anything: their scores are replaced (not
// multiplied) by -inf, and the softmax threads zero those rows of the V tile in shared memory before the P.V product
// (an exact-zero probability times a NaN would otherwise reach every query row of the tile).
//
// Tensor-memory columns: [0,128) S, [128,192) O, [192,448) band buffer, [448,512) P (bf16).
#include "tdb_internal.h"
#include "ptx_sm100.cuh"
#include <cudaTypedefs.h>
#include <math_constants.h>
#include <mutex>

namespace tdb {
using namespace ptx;

namespace {

constexpr int BQ = 128, BK = 128, HD = 64, BAND = 256;
#ifndef TDB_GROUPS
#define TDB_GROUPS 4
#endif
constexpr int GROUPS = TDB_GROUPS;              // threads per query row (2 or 4)
static_assert(GROUPS == 4, "four threads per query row (the drain split and the staging windows assume it)");
constexpr int KPT = BK / GROUPS;                // keys per thread in the softmax
constexpr int OPT = HD / GROUPS;                // output columns per thread
constexpr int NCW = 4 * GROUPS;                 // CUDA-core warps
constexpr int NCT = NCW * 32;                   // CUDA-core threads
constexpr int NTHREADS = (NCW + 3) * 32;       // + TMA producer warp, MMA warp, scheduler warp
constexpr int STG_STRIDE = 336;                 // bytes per staging row: 160 bf16 + 16 pad (odd multiple of 16)
constexpr int STG_COLS = 160;
constexpr uint32_t OFF_Q = 0 /* two buffers */, OFF_K = 32768, OFF_V = 49152, OFF_KR = 65536, OFF_QR = 98304;
constexpr uint32_t OFF_STC = 131072, OFF_STP = OFF_STC + BQ * STG_STRIDE, OFF_XCH = OFF_STP + BK * STG_STRIDE;
constexpr uint32_t OFF_BAR = OFF_XCH + GROUPS * BQ * 4;
constexpr uint32_t OFF_WORK = OFF_BAR + 256;        // ring of work items published by the scheduler lane
constexpr uint32_t OFF_CUR = OFF_WORK + 256;        // abort flag, tensor-memory base, the CUDA-core warps' copies of their items
constexpr uint32_t OFF_LX = OFF_CUR + 160;          // row-sum partials of a finished item, [item parity][group][row]
constexpr uint32_t OFF_MX = OFF_LX + 2 * GROUPS * BQ * 4;   // its reference exponents, [item parity][row]
constexpr uint32_t OFF_PERM = OFF_MX + 2 * BQ * 4;          // padded form: sequences by decreasing length
constexpr int PERM_MAX = 256;
#ifndef TDB_FCB
#define TDB_FCB 9
#endif
constexpr int FCB = TDB_FCB;                    // step of the exponential loop at which the fused c2p drain starts
static_assert(FCB >= 0 && FCB + STG_COLS / GROUPS / 8 <= KPT / 2 - 1, "the fused drain's last step must lie inside the loop");
constexpr uint32_t SMEM_BYTES = OFF_PERM + PERM_MAX * 2 + 1024;   // + slack for the 1024-byte alignment of the base
static_assert(OFF_STP % 16 == 0 && OFF_XCH % 16 == 0 && OFF_BAR % 16 == 0 && OFF_LX % 16 == 0, "offsets must stay 16-byte aligned");
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");

constexpr uint32_t TM_S = 0, TM_O = 128, TM_RING = 192, TM_P = 448, TM_COLS = 512;
constexpr uint64_t WAIT_LIMIT_NS = 1000ull * 1000ull * 1000ull;   // 1 s per wait, then give up

enum Bar { Q_FULL = 0 /* Q_FULL + buffer */, Q_FULL1, Q_EMPTY /* Q_EMPTY + buffer */, Q_EMPTY1, K_FULL, K_EMPTY, V_FULL, V_EMPTY, KR_FULL, KR_EMPTY, QR_FULL, QR_EMPTY,
           S_FULL, S_TAKEN, BAND_FULL, BAND_FREE, P_READY, O_FULL,
           DONE, WORK_FULL0, WORK_FULL1, WORK_FULL2, WORK_FULL3,
           WORK_EMPTY0, WORK_EMPTY1, WORK_EMPTY2, WORK_EMPTY3, NBARS };
constexpr int WORK_RING = 3;                     // the item in progress and the two after it: what the roles look ahead, and
                                                // no more (every item claimed early is taken from a CTA that may be free sooner)
constexpr int WORK_READERS = 3 + 1 + 1;         // three producer lanes, the MMA lane, the CUDA-core warps' leader
static_assert(NBARS * 8 <= 256, "barrier block");

struct TileListHeader { int32_t n_tiles; int32_t pad[3]; };

// ---------------------------------------------------------------------------------------------
// Packed form: list of (sequence, first query row) per 128-row tile, built on the device from cu_seqlens so that
// the host never reads lengths back.  Tiles are ordered by decreasing sequence length (a counting sort on the
// number of key tiles), so the device-wide work counter hands out the expensive tiles first and the short ones
// fill the tail.  Also validates cu_seqlens: a negative length or an offset outside [0, T] sets status[1] and
// the sequence is dropped.
constexpr int LIST_BUCKETS = 1024;
__global__ void __launch_bounds__(1024) build_tile_list_kernel(const int32_t* __restrict__ cu, int n_seqs,
                                                                int64_t total_tokens, int32_t* ws, int cap,
                                                                int32_t* status) {
  __shared__ int hist[LIST_BUCKETS];       // tiles per bucket, then the write cursor of the bucket
  int2* entries = reinterpret_cast<int2*>(ws + 4);
  for (int i = threadIdx.x; i < LIST_BUCKETS; i += blockDim.x) hist[i] = 0;
  __syncthreads();
  auto tiles_of = [&](int s) {
    const int a = cu[s], b = cu[s + 1];
    if (a < 0 || b < a || (int64_t)b > total_tokens) { atomicExch(status + 1, 1); return 0; }
    return (b - a + BQ - 1) / BQ;
  };
  for (int s = threadIdx.x; s < n_seqs; s += blockDim.x) {
    const int nt = tiles_of(s);
    if (nt > 0) atomicAdd(&hist[nt < LIST_BUCKETS ? nt : LIST_BUCKETS - 1], nt);
  }
  __syncthreads();
  if (threadIdx.x == 0) {                  // exclusive scan from the largest bucket down
    int run = 0;
    for (int bkt = LIST_BUCKETS - 1; bkt >= 0; --bkt) { const int c = hist[bkt]; hist[bkt] = run; run += c; }
    ws[0] = run < cap ? run : cap;
    if (cu[n_seqs] != (int32_t)total_tokens) atomicExch(status + 1, 1);
  }
  __syncthreads();
  for (int s = threadIdx.x; s < n_seqs; s += blockDim.x) {
    const int nt = tiles_of(s);
    if (nt <= 0) continue;
    const int start = atomicAdd(&hist[nt < LIST_BUCKETS ? nt : LIST_BUCKETS - 1], nt);
    for (int t = 0; t < nt; ++t)
      if (start + t < cap) entries[start + t] = make_int2(s, t * BQ);
  }
}

// x + (a bf16 value in a 16-bit register): the conversion rides on the add.
__device__ __forceinline__ float add_bf16(float x, uint16_t h) {
  float y;
  asm("add.rn.f32.bf16 %0, %1, %2;" : "=f"(y) : "h"(h), "f"(x));
  return y;
}
__device__ __forceinline__ uint16_t lds_u16(uint32_t addr) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ float lds_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts_f32(uint32_t addr, float v) {
  asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ uint4 lds_128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts_128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
// Makes this thread's earlier shared-memory writes visible to the asynchronous proxy (the tensor cores' operand fetch).
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void bar_all_cuda_warps() { asm volatile("bar.sync 1, %0;" ::"n"(NCT) : "memory"); }
// The same barrier with an OR-reduction of one predicate per thread.
__device__ __forceinline__ bool bar_all_cuda_warps_or(bool flag) {
  uint32_t r;
  asm volatile(
      "{\n"
      ".reg .pred p, q;\n"
      "setp.ne.u32 q, %1, 0;\n"
      "bar.red.or.pred p, 1, %2, q;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}"
      : "=r"(r) : "r"((uint32_t)flag), "n"(NCT) : "memory");
  return r != 0;
}
__device__ __forceinline__ void bar_quadrant(int qd) { asm volatile("bar.sync %0, %1;" ::"r"(2 + qd), "n"(GROUPS * 32) : "memory"); }

// N consecutive 32-bit columns of this thread's tensor-memory lane (N = 16, 32 or 64).
template <int N> __device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t* r) {
  if constexpr (N == 16) { tmem_ld16(taddr, r); tmem_ld_wait16(r); }
  else {
#pragma unroll
    for (int c = 0; c < N / 32; ++c) tmem_ld32(taddr + 32 * c, r + 32 * c);
#pragma unroll
    for (int c = 0; c < N / 32; ++c) tmem_ld_wait32(r + 32 * c);
  }
}
template <int N> __device__ __forceinline__ void tmem_st_cols(uint32_t taddr, const uint32_t* r) {
  if constexpr (N == 16) { tmem_st16(taddr, r); }
  else {
#pragma unroll
    for (int c = 0; c < N / 32; ++c) tmem_st32(taddr + 32 * c, r + 32 * c);
  }
}

// Four 32-bit columns of this thread's tensor-memory lane (asynchronous: tmem_st_wait() before anybody is told).
__device__ __forceinline__ void tmem_st4(uint32_t taddr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// Move 32 fp32 columns of this thread's tensor-memory lane to 32 bf16 of a staging row.
__device__ __forceinline__ void drain_chunk(uint32_t taddr, uint32_t dst_saddr) {
  uint32_t r[32];
  tmem_ld32(taddr, r);
  tmem_ld_wait32(r);
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    uint32_t w[4];
#pragma unroll
    for (int e = 0; e < 4; ++e)
      w[e] = pack_bf16x2(__uint_as_float(r[g * 8 + 2 * e]), __uint_as_float(r[g * 8 + 2 * e + 1]));
    sts_128(dst_saddr + g * 16, w[0], w[1], w[2], w[3]);
  }
}

// One unit of work: a 128-query tile of one sequence for one head.
// A 128x128 score tile whose distances q - k all lie at or beyond the saturation distance (on one side): every
// score of the tile uses the same table row r, so c2p is Q[i].Kr[r] and p2c is K[j].Qr[r].  The expanded tables repeat
// that row over their whole saturated end, so a 128-row box from there is a tile of identical rows, and both terms are
// folded into the score product itself:  S = Q.K^T + Q.KrRep^T + QrRep.K^T  (three accumulating products into the
// same accumulator).  Such a tile has no band products, no drains and no gathers at all.
__device__ __forceinline__ bool tile_saturated(const AttnParams& p, int q0, int k0) {
  const int sat = p.exp_delta_max - TDB_EXPAND_MARGIN;
  const int d = q0 - k0;
  return (d - (BK - 1) >= sat) || (d + (BQ - 1) <= -sat);
}
constexpr int SATN = 128;                       // rows of the repeated-row boxes

struct Work {
  int q0, len, rows, bcoord, h, n_kv;      // n_kv == 0: tile of padded query rows only (zeros, no tensor work)
  int64_t tok0;
};

// perm: padded form only, sequences by decreasing length (null: natural order).
__device__ __forceinline__ bool get_work(const AttnParams& p, int total_tiles, int w, const uint16_t* perm, Work& k) {
  const int tile = w / p.H;
  if (tile >= total_tiles) return false;
  k.h = w - tile * p.H;
  if (p.varlen) {
    const int32_t* ws = reinterpret_cast<const int32_t*>(p.workspace);
    const int2 e = reinterpret_cast<const int2*>(ws + 4)[tile];
    const int c0 = p.cu_seqlens[e.x];
    k.len = p.cu_seqlens[e.x + 1] - c0; k.rows = k.len; k.tok0 = c0; k.bcoord = 0; k.q0 = e.y;
  } else {
    const int qtiles = (p.L + BQ - 1) / BQ;
    int seq = tile / qtiles;
    k.q0 = (tile - seq * qtiles) * BQ;
    if (perm) seq = perm[seq];
    int len = p.seqlens ? p.seqlens[seq] : p.L;
    k.len = len < 0 ? 0 : (len > p.L ? p.L : len);
    k.rows = p.L; k.tok0 = 0; k.bcoord = seq;
  }
  k.n_kv = k.q0 < k.len ? (k.len + BK - 1) / BK : 0;
  return true;
}

// LONG: sequences can be long enough for saturated tiles (compiled out otherwise, which keeps the common kernel lean).
template <bool C2P, bool P2C, bool LONG>
__global__ void __launch_bounds__(NTHREADS, 1)
attn_umma_kernel(const AttnParams p, const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_kr,
                 const __grid_constant__ CUtensorMap tm_qr, const __grid_constant__ CUtensorMap tm_kr16,
                 const __grid_constant__ CUtensorMap tm_qr16) {
  extern __shared__ uint8_t smem_raw[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // Persistent CTA.  Work items (query tile x head) are handed out by a device-wide counter (status word 2), so a
  // CTA that drew short sequences simply draws more of them; a scheduler lane publishes each item in a small
  // shared-memory ring that every role reads in the same order.
  const int total_tiles = p.varlen ? reinterpret_cast<const int32_t*>(p.workspace)[0]
                                   : p.n_seqs * ((p.L + BQ - 1) / BQ);
  // An earlier CTA gave up: the scheduler lane (which reads the word while the CTA sets itself up) hands out no work.
  int32_t status_at_start = 0;
  if (warp == NCW + 2 && lane == 0) status_at_start = *reinterpret_cast<volatile int32_t*>(p.status);

  // ---- shared memory carve-up ----------------------------------------------------------------
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (sbase - smem_u32(smem_raw));
  const uint32_t sQ = sbase + OFF_Q, sK = sbase + OFF_K, sV = sbase + OFF_V, sKr = sbase + OFF_KR, sQr = sbase + OFF_QR;
  const uint32_t stC = sbase + OFF_STC, stP = sbase + OFF_STP, sX = sbase + OFF_XCH;
  const uint32_t bars = sbase + OFF_BAR;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gbase + OFF_CUR);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbase + OFF_CUR + 8);
  Work* work_ring = reinterpret_cast<Work*>(gbase + OFF_WORK);
  auto bar = [&](int i) { return bars + 8u * (uint32_t)i; };
  auto wait = [&](int i, uint32_t parity) { return mbar_wait(bar(i), parity, abort_flag, p.status, 1 + i, WAIT_LIMIT_NS); };

  if (tid == 0) {
    *abort_flag = 0;
    for (int i = 0; i < NBARS; ++i) {
      const bool by_warps = (i == S_TAKEN || i == BAND_FREE || i == P_READY);
      const bool by_readers = (i >= WORK_EMPTY0 && i <= WORK_EMPTY3);
      mbar_init(bar(i), by_readers ? (uint32_t)WORK_READERS : (by_warps ? (uint32_t)NCW : 1u));
    }
    fence_mbar_init();
  }
  if (warp == NCW && lane == 0) {
    prefetch_tmap(&tm_q); prefetch_tmap(&tm_k); prefetch_tmap(&tm_v);
    if (C2P) { prefetch_tmap(&tm_kr); prefetch_tmap(&tm_kr16); }
    if (P2C) { prefetch_tmap(&tm_qr); prefetch_tmap(&tm_qr16); }
  }
  if (warp == NCW + 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), TM_COLS);
    tmem_relinquish();
  }
  // Padded form with lengths: the items of long sequences cost more (one key tile per 128 valid keys), so the
  // sequences are handed out by decreasing number of key tiles - a counting sort that every CTA's scheduler warp
  // repeats for itself (a few hundred warp instructions; skipped for batches where it would cost more).  It runs
  // while the other warps set the CTA up: it needs nothing but the lengths in global memory and its own corner of
  // shared memory.
  const uint16_t* perm = nullptr;
  if (warp == NCW + 2) {
    const int qtiles = (p.L + BQ - 1) / BQ;
    if (!p.varlen && p.seqlens && p.n_seqs > 1 && p.n_seqs <= PERM_MAX && p.n_seqs * (qtiles + 1) <= 2048) {
      uint16_t* pw = reinterpret_cast<uint16_t*>(gbase + OFF_PERM);
      int base = 0;
      for (int b = qtiles; b >= 0; --b) {
        for (int s0 = 0; s0 < p.n_seqs; s0 += 32) {
          const int sq = s0 + lane;
          int key = -1;
          if (sq < p.n_seqs) {
            int len = p.seqlens[sq];
            len = len < 0 ? 0 : (len > p.L ? p.L : len);
            key = (len + BK - 1) / BK;
          }
          const uint32_t m = __ballot_sync(0xffffffffu, key == b);
          if (key == b) pw[base + __popc(m & ((1u << lane) - 1u))] = (uint16_t)sq;
          base += __popc(m);
        }
      }
      __syncwarp();
      perm = pw;
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  // Item n of this CTA's stream; n_kv < 0 marks the end of the stream.  (Tiles that consist of padded query rows
  // only never enter the ring: the scheduler warp zeroes them itself.)
  auto fetch = [&](int n, Work& k) {
    wait(WORK_FULL0 + (n % WORK_RING), (uint32_t)((n / WORK_RING) & 1));
    k = work_ring[n % WORK_RING];
    if (*abort_flag) k.n_kv = -1;
    return k.n_kv > 0;
  };
  auto release = [&](int n) { mbar_arrive(bar(WORK_EMPTY0 + (n % WORK_RING))); };
  auto next_tensor_item = [&](int& n, Work& k) { return fetch(n, k); };

  if (warp == NCW) {
    // ================================ TMA producers ==========================================
    if (lane == 0) {                       // relative tables and K, once per key tile
      Work k;
      int g = 0, n = 0;
      while (next_tensor_item(n, k)) {
        for (int it = 0; it < k.n_kv; ++it, ++g) {
          const int k0 = it * BK;
          const uint32_t pe = (uint32_t)((g - 1) & 1);
          int x0 = k.q0 - k0 - (BK - 1) + p.exp_delta_max;
          x0 = x0 < 0 ? 0 : (x0 > p.exp_rows - BAND ? p.exp_rows - BAND : x0);
          const bool sat = LONG && tile_saturated(p, k.q0, k0);
          if (C2P) {
            if (g > 0) wait(KR_EMPTY, pe);
            if (!*abort_flag) {
              mbar_expect_tx(bar(KR_FULL), (sat ? SATN : BAND) * HD * 2);
              tma_load_3d(sKr, sat ? &tm_kr16 : &tm_kr, bar(KR_FULL), 0, x0, k.h);
            }
          }
          if (g > 0) wait(K_EMPTY, pe);
          if (!*abort_flag) {
            mbar_expect_tx(bar(K_FULL), BK * HD * 2);
            tma_load_4d(sK, &tm_k, bar(K_FULL), 0, (int)(k.tok0 + k0), k.h, k.bcoord);
          }
          if (P2C) {
            if (g > 0) wait(QR_EMPTY, pe);
            if (!*abort_flag) {
              mbar_expect_tx(bar(QR_FULL), (sat ? SATN : BAND) * HD * 2);
              tma_load_3d(sQr, sat ? &tm_qr16 : &tm_qr, bar(QR_FULL), 0, x0, k.h);
            }
          }
        }
        release(n);
        ++n;
      }
      release(n);
    } else if (lane == 1) {                // V, once per key tile
      Work k;
      int g = 0, n = 0;
      while (next_tensor_item(n, k)) {
        for (int it = 0; it < k.n_kv; ++it, ++g) {
          if (g > 0) wait(V_EMPTY, (uint32_t)((g - 1) & 1));
          if (!*abort_flag) {
            mbar_expect_tx(bar(V_FULL), BK * HD * 2);
            tma_load_4d(sV, &tm_v, bar(V_FULL), 0, (int)(k.tok0 + it * BK), k.h, k.bcoord);
          }
        }
        release(n);
        ++n;
      }
      release(n);
    } else if (lane == 2) {                // Q, once per work item, into alternating buffers
      Work k;
      int n = 0;
      while (next_tensor_item(n, k)) {
        const int b = n & 1;
        if (n >= 2) wait(Q_EMPTY + b, (uint32_t)(((n >> 1) - 1) & 1));
        if (!*abort_flag) {
          mbar_expect_tx(bar(Q_FULL + b), BQ * HD * 2);
          tma_load_4d(sQ + (uint32_t)b * (BQ * HD * 2), &tm_q, bar(Q_FULL + b), 0, (int)(k.tok0 + k.q0), k.h, k.bcoord);
        }
        release(n);
        ++n;
      }
      release(n);
    }
  } else if (warp == NCW + 2) {
    // ================================ scheduler ==============================================
    // Draws work items from the device-wide counter and publishes those with tensor work in the ring; tiles made of
    // padded query rows only (padded form) are zeroed here by the whole warp and never reach the other roles.
    // The first item of a CTA is its own index (no round trip to the counter before the pipeline can start); the
    // counter hands out the items after those.
    // Padded form with lengths: the sequences are handed out in the order sorted above.
    int n = 0;
    bool first = true;
    while (true) {
      int w = 0;
      if (lane == 0)
        w = (*abort_flag || status_at_start != 0) ? 0x7fffffff
                                                  : (first ? (int)blockIdx.x : (int)gridDim.x + atomicAdd(p.status + 2, 1));
      first = false;
      w = __shfl_sync(0xffffffffu, w, 0);
      Work k;
      if (!get_work(p, total_tiles, w, perm, k)) k.n_kv = -1;
      if (k.n_kv == 0) {
        for (int r = lane; r < BQ; r += 32) {
          if (k.q0 + r >= k.rows) break;
          __nv_bfloat16* ob = reinterpret_cast<__nv_bfloat16*>(p.o) + (int64_t)k.bcoord * p.o_sb +
                              (k.tok0 + k.q0 + r) * p.o_st + (int64_t)k.h * p.o_sh;
          uint4* dst = reinterpret_cast<uint4*>(ob);
#pragma unroll
          for (int i = 0; i < 8; ++i) dst[i] = make_uint4(0, 0, 0, 0);
          if (p.lse) p.lse[(int64_t)k.bcoord * p.lse_sb + (int64_t)k.h * p.lse_sh + k.tok0 + k.q0 + r] = 0.f;
        }
        continue;
      }
      const int slot = n % WORK_RING;
      if (lane == 0) {
        if (n >= WORK_RING) wait(WORK_EMPTY0 + slot, (uint32_t)(((n / WORK_RING) - 1) & 1));
        work_ring[slot] = k;
        mbar_arrive(bar(WORK_FULL0 + slot));         // release: the item is visible to whoever observes the phase
      }
      __syncwarp();
      ++n;
      if (k.n_kv < 0) break;
    }
  } else if (warp == NCW + 1) {
    // ================================ MMA issuer ============================================
    if (lane == 0) {
      constexpr uint32_t ID_S = make_idesc_bf16(128, BK, 0);
      constexpr uint32_t ID_BAND = make_idesc_bf16(128, BAND, 0);
      constexpr uint32_t ID_PV = make_idesc_bf16(128, HD, 1);
      const uint64_t dQ = smem_desc_sw128(sQ), dK = smem_desc_sw128(sK), dV = smem_desc_sw128(sV);
      const uint64_t dKr = smem_desc_sw128(sKr), dQr = smem_desc_sw128(sQr);
      const uint32_t tS = tmem + TM_S, tO = tmem + TM_O, tP = tmem + TM_P;
      const uint32_t tBand = tmem + TM_RING;
      int fills = 0;                       // how often the band buffer has been filled so far

      // A position in this CTA's stream of key tiles: ring index of the work item, key tile inside it.
      struct TileCur { int n, it, n_kv, q0; bool ok; };
      auto cur_fetch = [&](TileCur& c) {
        Work k;
        c.ok = fetch(c.n, k);
        c.n_kv = k.n_kv; c.q0 = k.q0;
      };
      auto cur_next = [&](TileCur& c) {
        if (c.it + 1 < c.n_kv) { ++c.it; return; }
        ++c.n; c.it = 0;
        cur_fetch(c);
      };
      auto wait_q = [&](const TileCur& c) {                 // the item's Q tile has landed (once per item)
        if (c.it == 0) wait(Q_FULL + (c.n & 1), (uint32_t)((c.n >> 1) & 1));
      };
      auto wait_ring_free = [&]() {
        if (fills > 0) wait(BAND_FREE, (uint32_t)((fills - 1) & 1));
      };
      auto ring_filled = [&]() {
        tc_commit(bar(BAND_FULL));
        ++fills;
      };
      // content->position band of key tile g (global count): one 256-column product into the band buffer
      auto issue_c = [&](const TileCur& c, int g) {
        if (LONG && tile_saturated(p, c.q0, c.it * BK)) return;          // folded into the score product
        wait(KR_FULL, (uint32_t)(g & 1));
        wait_q(c);
        wait_ring_free();
        tc_fence_after();
        const uint64_t dQc = dQ + (uint64_t)((c.n & 1) * ((BQ * HD * 2) >> 4));
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) mma_ss(tBand, dQc + 2 * k, dKr + 2 * k, ID_BAND, k > 0);
        ring_filled();
        tc_commit(bar(KR_EMPTY));
      };
      // content score of key tile g; the last one of an item releases the item's Q buffer
      auto issue_s = [&](const TileCur& c, int g) {
        const bool sat = LONG && tile_saturated(p, c.q0, c.it * BK);
        wait(K_FULL, (uint32_t)(g & 1));
        wait_q(c);
        if (sat && C2P) wait(KR_FULL, (uint32_t)(g & 1));
        if (sat && P2C) wait(QR_FULL, (uint32_t)(g & 1));
        if (g > 0) wait(S_TAKEN, (uint32_t)((g - 1) & 1));
        tc_fence_after();
        const uint64_t dQc = dQ + (uint64_t)((c.n & 1) * ((BQ * HD * 2) >> 4));
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) mma_ss(tS, dQc + 2 * k, dK + 2 * k, ID_S, k > 0);
        if (sat) {                           // the two position terms of a saturated tile: repeated-row operands
          if (C2P) {
#pragma unroll
            for (int k = 0; k < HD / 16; ++k) mma_ss(tS, dQc + 2 * k, dKr + 2 * k, ID_S, 1u);
            tc_commit(bar(KR_EMPTY));
          }
          if (P2C) {
#pragma unroll
            for (int k = 0; k < HD / 16; ++k) mma_ss(tS, dQr + 2 * k, dK + 2 * k, ID_S, 1u);
            tc_commit(bar(QR_EMPTY));
          }
        }
        tc_commit(bar(S_FULL));
        if (c.it + 1 == c.n_kv) tc_commit(bar(Q_EMPTY + (c.n & 1)));
      };
      // position->content band of key tile g (rows = keys), once the c2p band has been drained; releases K
      auto issue_p2 = [&](const TileCur& c, int g) {
        if (P2C && !(LONG && tile_saturated(p, c.q0, c.it * BK))) {
          wait(QR_FULL, (uint32_t)(g & 1));
          wait_ring_free();
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < HD / 16; ++k) mma_ss(tBand, dK + 2 * k, dQr + 2 * k, ID_BAND, k > 0);
          ring_filled();
          tc_commit(bar(QR_EMPTY));
        }
        tc_commit(bar(K_EMPTY));
      };
      // O += P . V of key tile g.  The first one of an item overwrites O: the CUDA warps read the previous item's O
      // before they announce the P of this tile, so P_READY covers that as well.
      auto issue_pv = [&](const TileCur& c, int g) {
        wait(V_FULL, (uint32_t)(g & 1));
        wait(P_READY, (uint32_t)(g & 1));
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < BK / 16; ++k)
          mma_ts(tO, tP + 8 * k, dV + (uint64_t)(128 * k), ID_PV, (c.it > 0 || k > 0) ? 1u : 0u);
        tc_commit(bar(O_FULL));
        tc_commit(bar(V_EMPTY));
      };

      // Issue order, by rounds r = -1, 0, 1, ...:  S(r) P2(r) PV(r-1) C(r+1), i.e.
      //   C(0) | S(0) P2(0) C(1) | S(1) P2(1) PV(0) C(2) | S(2) P2(2) PV(1) C(3) | ...
      // While the CUDA warps work on tile g they enable, in this order: C(g+1) (the p2c band of tile g leaves the band
      // buffer during the c2p phase), P2(g+1) (the c2p band of tile g+1 leaves it during the exponentials) and
      // P.V(g); the lane waits idle at the two band products, which are the tile's critical chain, and fits S(g+1) -
      // enabled long before - between them.  One loop with every product issued from a single place keeps the lane's
      // code small (it runs once per tile and should not fall out of the instruction cache in between).
      TileCur cc, cs, cv;                  // c2p stream (two tiles ahead), score/p2c stream (one ahead), P.V stream
      cc.n = 0; cc.it = 0; cur_fetch(cc);
      cs = cc; cv = cc;
      int gc = 0, gs = 0, gv = 0;
      if (cv.ok) {
#pragma unroll 1
        for (int r = -1; ; ++r) {
          if (r >= 0 && cs.ok) {
            issue_s(cs, gs); issue_p2(cs, gs); ++gs;
            cur_next(cs);
          }
          if (r > 0) {
            issue_pv(cv, gv++);
            if (cv.it + 1 == cv.n_kv) release(cv.n);
            cur_next(cv);
            if (!cv.ok) break;
          }
          if (C2P && cc.ok) { issue_c(cc, gc++); cur_next(cc); }
        }
      }
      release(cv.n);                       // the end-of-stream marker
      // Everything issued above must have retired before tensor memory is released.
      tc_commit(bar(DONE));
      int never = 0;                       // this wait runs even after an abort, with its own limit
      mbar_wait(bar(DONE), 0, &never, p.status, 1 + DONE, WAIT_LIMIT_NS);
    }
  } else {
    // ================================ drain + softmax + epilogue ============================
    const int qd = warp & 3, grp = warp >> 2;
    const int row_t = qd * 32 + lane;                                  // tensor-memory lane = query row (or key row of P2)
    const uint32_t lane_base = ((uint32_t)(qd * 32)) << 16;
    const uint32_t tS = tmem + lane_base + TM_S + KPT * grp;
    const uint32_t tO = tmem + lane_base + TM_O + OPT * grp;
    const uint32_t tP = tmem + lane_base + TM_P + (KPT / 2) * grp;
    const float sl2 = p.sm_scale * 1.4426950408889634f;
    // staging rows: c2p row i holds band columns [32*qd, +160); p2c row j holds band columns [96 - 32*(j/32), +160)
    // c2p rows are laid out in pairs (656 bytes per pair, the odd row 320 bytes in): 16-byte row stores of a warp
    // hit eight different 16-byte slots, and the skewed 32-bit reads (one row per lane, two bytes further per
    // lane) hit 32 different banks.
    const uint32_t c_row = stC + (uint32_t)(row_t >> 1) * 656u + (uint32_t)(row_t & 1) * 320u;
    const uint32_t p_row = stP + (uint32_t)row_t * STG_STRIDE;
    const uint32_t c_read = c_row + 2u * (uint32_t)(lane + (BK - 1) - KPT * grp);          // key e of this thread: c_read - 2e
    const uint32_t p_read = stP + (uint32_t)(KPT * grp) * STG_STRIDE + 2u * (uint32_t)(row_t + 31);  // + e*STRIDE - 2*(e%32)
    const uint32_t x_mine = sX + 4u * (uint32_t)(grp * BQ + row_t);
    int drains = 0;

    // Drain the band buffer into this warp's share of the staging rows.  kind 0: c2p (window starts at 32*qd),
    // kind 1: p2c (96 - 32*qd).
    auto drain_band = [&](int kind) {
      wait(BAND_FULL, (uint32_t)(drains & 1));
      ++drains;
      tc_fence_after();
      // The 160 staged columns of a row are split evenly over the four warps that own the row: 40 columns each.
      const int local = (STG_COLS / GROUPS) * grp;                     // position inside the staging row
      const uint32_t src = tmem + lane_base + TM_RING + (uint32_t)((kind == 0 ? 32 * qd : 96 - 32 * qd) + local);
      const uint32_t dst = (kind == 0 ? c_row : p_row) + 2u * (uint32_t)local;
      drain_chunk(src, dst);
      uint32_t r[8];
      tmem_ld8(src + 32, r);
      tmem_ld_wait8(r);
      sts_128(dst + 64, pack_bf16x2(__uint_as_float(r[0]), __uint_as_float(r[1])),
              pack_bf16x2(__uint_as_float(r[2]), __uint_as_float(r[3])),
              pack_bf16x2(__uint_as_float(r[4]), __uint_as_float(r[5])),
              pack_bf16x2(__uint_as_float(r[6]), __uint_as_float(r[7])));
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(BAND_FREE));
    };
    // Saturated tiles have no bands (their position terms are part of the score product).
    auto drain_c = [&](bool sat) { if (C2P && !sat) drain_band(0); };
    auto drain_p2 = [&](bool sat) { if (P2C && !sat) drain_band(1); };

    // The CUDA-core warps walk one flat stream of key tiles.  Thread 0 copies the work items from the scheduler's
    // ring into four slots, two items ahead of the one being processed, so that every warp takes its trip counts
    // from the same copy (also after an abort) and an item switch needs no extra barrier: a slot is written at
    // least one CTA-wide barrier before anybody reads it, and rewritten only after its last reader has passed one.
    static_assert(sizeof(Work) == 32, "work items are copied as two 16-byte vectors");
    const uint32_t slots = sbase + OFF_CUR + 16;                       // four items of 32 bytes
    volatile Work* const item_slots = reinterpret_cast<volatile Work*>(gbase + OFF_CUR + 16);
    auto load_item = [&](int n, Work& k) {                             // every field (epilogue)
      const uint4 a = lds_128(slots + 32u * (uint32_t)(n & 3)), b = lds_128(slots + 32u * (uint32_t)(n & 3) + 16u);
      k.q0 = (int)a.x; k.len = (int)a.y; k.rows = (int)a.z; k.bcoord = (int)a.w; k.h = (int)b.x; k.n_kv = (int)b.y;
      k.tok0 = (int64_t)(((uint64_t)b.w << 32) | b.z);
    };
    auto leader_publish = [&](int n) {                                 // thread 0 only
      uint4 a = make_uint4(0, 0, 0, 0), b = make_uint4(0, 0xffffffffu, 0, 0);   // end marker: n_kv = -1
      if (n == 0 || item_slots[(n - 1) & 3].n_kv > 0) {                // nothing follows the end marker
        wait(WORK_FULL0 + (n % WORK_RING), (uint32_t)((n / WORK_RING) & 1));
        const uint32_t src = sbase + OFF_WORK + 32u * (uint32_t)(n % WORK_RING);
        a = lds_128(src); b = lds_128(src + 16u);
        if (*abort_flag) b.y = 0xffffffffu;
        release(n);
      }
      sts_128(slots + 32u * (uint32_t)(n & 3), a.x, a.y, a.z, a.w);
      sts_128(slots + 32u * (uint32_t)(n & 3) + 16u, b.x, b.y, b.z, b.w);
    };
    const uint32_t lx_mine = sbase + OFF_LX + 4u * (uint32_t)(grp * BQ + row_t);      // + parity * GROUPS * BQ * 4
    const uint32_t mx_row = sbase + OFF_MX + 4u * (uint32_t)row_t;                     // + parity * BQ * 4

    // Epilogue of item pn, whose last key tile was number gl of the stream: O / l -> global.  Runs during the first
    // key tile of the item after it (so the wait for its last P.V product is off the critical path), or at the end.
    auto finish_item = [&](int pn, int gl) {
      Work w;
      load_item(pn, w);
      const uint32_t par = (uint32_t)(pn & 1);
      float l_tot = 0.f;
#pragma unroll
      for (int gg = 0; gg < GROUPS; ++gg)
        l_tot += lds_f32(sbase + OFF_LX + 4u * (uint32_t)((par * GROUPS + gg) * BQ + row_t));
      wait(O_FULL, (uint32_t)(gl & 1));
      tc_fence_after();
      uint32_t r[OPT];
      tmem_ld_cols<OPT>(tO, r);
      tc_fence_before();
      float inv;
      asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(inv) : "f"(l_tot));
      // The normalised rows go through shared memory (the quadrant's part of the p2c staging area, which nobody
      // uses between the barrier that closed this tile's p2c reads and the next drain) so that each store
      // instruction writes four whole 128-byte rows instead of 32 separate 16-byte pieces.
      {
        const bool valid = w.q0 + row_t < w.len;
        uint32_t outw[OPT / 2];
#pragma unroll
        for (int e = 0; e < OPT; e += 2)
          outw[e / 2] = valid ? pack_bf16x2(__uint_as_float(r[e]) * inv, __uint_as_float(r[e + 1]) * inv) : 0u;
        const uint32_t obuf = stP + (uint32_t)(32 * qd) * STG_STRIDE;          // 32 rows, 144-byte pitch
        const uint32_t mine = obuf + (uint32_t)lane * 144u + (uint32_t)(OPT * 2 * grp);
#pragma unroll
        for (int i = 0; i < OPT / 8; ++i)
          sts_128(mine + 16u * i, outw[4 * i], outw[4 * i + 1], outw[4 * i + 2], outw[4 * i + 3]);
        bar_quadrant(qd);
        __nv_bfloat16* const obase = reinterpret_cast<__nv_bfloat16*>(p.o) + (int64_t)w.bcoord * p.o_sb +
                                     (int64_t)w.h * p.o_sh + 8 * (lane & 7);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int rq = 8 * grp + 4 * i + (lane >> 3);                        // row inside the quadrant
          const int row = w.q0 + 32 * qd + rq;
          const uint4 v = lds_128(obuf + (uint32_t)rq * 144u + 16u * (uint32_t)(lane & 7));
          if (row < w.rows) *reinterpret_cast<uint4*>(obase + (w.tok0 + row) * p.o_st) = v;
        }
        if (p.lse && grp == 0) {
          const int row = w.q0 + row_t;
          if (row < w.rows)
            p.lse[(int64_t)w.bcoord * p.lse_sb + (int64_t)w.h * p.lse_sh + w.tok0 + row] =
                valid ? (lds_f32(mx_row + par * (BQ * 4)) * 0.6931471805599453f + logf(l_tot)) : 0.f;
        }
        bar_quadrant(qd);                                                      // the staging rows may be drained into again
      }
    };

    if (tid == 0) { leader_publish(0); leader_publish(1); }
    bar_all_cuda_warps();
    struct { int q0, len, n_kv; } cur;
    auto switch_item = [&](int n) {
      volatile Work* w = item_slots + (n & 3);
      cur.q0 = w->q0; cur.len = w->len; cur.n_kv = w->n_kv;
    };
    switch_item(0);
    if (cur.n_kv > 0) {
      if (tid == 0) leader_publish(2);
      {                                                                // c2p band of the very first key tile
        const bool sat0 = LONG && tile_saturated(p, cur.q0, 0);
        drain_c(sat0);
        bar_all_cuda_warps();
      }
      float m_run = 0.f, l_part = 0.f;
      int n = 0, it = 0, g = 0;
      while (true) {
        const bool last_of_item = (it + 1 == cur.n_kv);
        const bool has_next = !last_of_item || item_slots[(n + 1) & 3].n_kv > 0;
        const int nvalid = cur.len - it * BK - KPT * grp;            // keys e >= nvalid of this thread are masked
        const bool sat = LONG && tile_saturated(p, cur.q0, it * BK);   // this key tile, and the one after it
        const bool sat_n = LONG && (!last_of_item ? tile_saturated(p, cur.q0, (it + 1) * BK)
                                                  : tile_saturated(p, item_slots[(n + 1) & 3].q0, 0));
        // The next tile's c2p band is drained inside this tile's exponential loop (eight columns at a time between the
        // loop's steps: that loop is bound by the special-function unit and has issue slots to spare, and the
        // tensor-memory loads' latency disappears behind it); a saturated tile has no band, and the tile before or after
        // one drains in one piece instead.
        const bool fuse = C2P && has_next && !sat && !sat_n;
        // Likewise this tile's own p2c band is drained inside the c2p loop just below (it was issued as soon as the c2p
        // band of this tile had been drained, during the tile before).
        const bool fuse_p = C2P && P2C && !sat;
        uint32_t dr[8];
        auto drain_begin = [&](uint32_t src) {
          wait(BAND_FULL, (uint32_t)(drains & 1));
          ++drains;
          tc_fence_after();
          tmem_ld8(src, dr);
        };
        // step c (0..4) of a fused drain: store the eight columns that have arrived, ask for the next eight; the band
        // buffer is handed back as soon as the last load has completed
        auto drain_step = [&](int c, uint32_t src, uint32_t dst) {
          tmem_ld_wait8(dr);
          sts_128(dst + 16u * (uint32_t)c, pack_bf16x2(__uint_as_float(dr[0]), __uint_as_float(dr[1])),
                  pack_bf16x2(__uint_as_float(dr[2]), __uint_as_float(dr[3])),
                  pack_bf16x2(__uint_as_float(dr[4]), __uint_as_float(dr[5])),
                  pack_bf16x2(__uint_as_float(dr[6]), __uint_as_float(dr[7])));
          if (c + 1 < STG_COLS / GROUPS / 8) {
            tmem_ld8(src + 8u * (uint32_t)(c + 1), dr);
          } else {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(BAND_FREE));
          }
        };
        const uint32_t dc_src = tmem + lane_base + TM_RING + (uint32_t)(32 * qd + (STG_COLS / GROUPS) * grp);
        const uint32_t dc_dst = c_row + 2u * (uint32_t)((STG_COLS / GROUPS) * grp);
        const uint32_t dp_src = tmem + lane_base + TM_RING + (uint32_t)(96 - 32 * qd + (STG_COLS / GROUPS) * grp);
        const uint32_t dp_dst = p_row + 2u * (uint32_t)((STG_COLS / GROUPS) * grp);
        if (fuse_p) drain_begin(dp_src);
        wait(S_FULL, (uint32_t)(g & 1));
        tc_fence_after();
        float s[KPT];
        {
          tmem_ld_cols<KPT>(tS, reinterpret_cast<uint32_t*>(s));
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(S_TAKEN));
        // Phase 1: add the content->position term, then hand the c2p staging rows (shared only inside the
        // quadrant) to the next key tile at once, so that its position->content products can run during phase 2.
        if (C2P) {
          // The 32 values sit at descending addresses from c_read; read them as 17 aligned 32-bit words and
          // realign odd lanes with a funnel shift (half the shared-memory wavefronts of 16-bit loads).
          if (sat) {
            // nothing to add: the score product of a saturated tile already holds all three terms
          } else {
            const uint32_t lo_addr = (c_read - 2u * (KPT - 1)) & ~3u;
            const uint32_t sh = (uint32_t)(lane & 1) * 16u;
            uint32_t wv[KPT / 2 + 1];
#pragma unroll
            for (int k = 0; k <= KPT / 2; ++k) wv[k] = lds_u32(lo_addr + 4u * k);
#pragma unroll
            for (int k = 0; k < KPT / 2; ++k) {
              const uint32_t v = __funnelshift_r(wv[k], wv[k + 1], sh);       // (element 2k, element 2k+1) ascending
              uint16_t lo, hi;
              asm("mov.b32 {%0, %1}, %2;" : "=h"(lo), "=h"(hi) : "r"(v));
              s[KPT - 1 - 2 * k] = add_bf16(s[KPT - 1 - 2 * k], lo);
              s[KPT - 2 - 2 * k] = add_bf16(s[KPT - 2 - 2 * k], hi);
              if ((k & 1) && k / 2 < STG_COLS / GROUPS / 8 && fuse_p) drain_step(k / 2, dp_src, dp_dst);
            }
          }
        }
        if (P2C && !fuse_p) drain_p2(sat);
        // Closes the reads of the c2p staging rows (the next tile's band is drained into them during phase 2) and
        // completes the p2c staging rows, which phase 2 reads across quadrants.
        bar_all_cuda_warps();
        // The copy of the item two ahead goes into the slot of the item two back, whose last reader (that item's
        // epilogue, inside the first tile of the item before this one) lies behind the barrier above.
        if (tid == 0 && it == 0 && n > 0) leader_publish(n + 2);
        // Phase 2.  Scores stay unscaled in s[]; the exponentials are taken at once against the reference exponent
        // of the previous tiles (0 on the first tile) so that the MUFU work overlaps the shared-memory reads, and
        // are redone only for rows whose new maximum is more than 2^8 above (or, on the first tile, 2^64 below) it.
        const float m_prev = (it > 0) ? m_run : 0.f;
        float lsum = 0.f;
        uint32_t pk[KPT / 2];
        // P of this tile goes to tensor memory while it is being formed, eight keys at a time, so the P.V product of
        // the tile before must have finished with the buffer (it has, long ago: it was issued when that tile ended).
        if (g > 0) {
          wait(O_FULL, (uint32_t)((g - 1) & 1));
          tc_fence_after();
        }
        if (sat) {
          // Saturated tile: the scores are complete; masking is applied unconditionally (not the common path).
#pragma unroll
          for (int e = 0; e < KPT; e += 2) {
            const float x0 = (e < nvalid) ? s[e] : -CUDART_INF_F;
            const float x1 = (e + 1 < nvalid) ? s[e + 1] : -CUDART_INF_F;
            s[e] = x0; s[e + 1] = x1;
            const float a = ex2(fmaf(x0, sl2, -m_prev)), b = ex2(fmaf(x1, sl2, -m_prev));
            lsum += a + b;
            pk[e / 2] = pack_bf16x2(a, b);
          }
          tmem_st_cols<KPT / 2>(tP, pk);
        } else if (nvalid >= KPT) {
#pragma unroll
          for (int e = 0; e < KPT; e += 2) {
            float x0 = s[e], x1 = s[e + 1];
            if (P2C) {
              x0 = add_bf16(x0, lds_u16(p_read + (uint32_t)(e * STG_STRIDE - 2 * (e & 31))));
              x1 = add_bf16(x1, lds_u16(p_read + (uint32_t)((e + 1) * STG_STRIDE - 2 * ((e + 1) & 31))));
            }
            s[e] = x0; s[e + 1] = x1;
            const float a = ex2(fmaf(x0, sl2, -m_prev)), b = ex2(fmaf(x1, sl2, -m_prev));
            lsum += a + b;
            pk[e / 2] = pack_bf16x2(a, b);
            if ((e / 2) % 4 == 3) tmem_st4(tP + (uint32_t)(e / 2 - 3), pk[e / 2 - 3], pk[e / 2 - 2], pk[e / 2 - 1], pk[e / 2]);
            if (fuse && e / 2 == FCB) drain_begin(dc_src);
            if (fuse && e / 2 > FCB && e / 2 <= FCB + STG_COLS / GROUPS / 8) drain_step(e / 2 - FCB - 1, dc_src, dc_dst);
          }
        } else {
#pragma unroll
          for (int e = 0; e < KPT; e += 2) {
            float x0 = s[e], x1 = s[e + 1];
            if (P2C) {
              x0 = add_bf16(x0, lds_u16(p_read + (uint32_t)(e * STG_STRIDE - 2 * (e & 31))));
              x1 = add_bf16(x1, lds_u16(p_read + (uint32_t)((e + 1) * STG_STRIDE - 2 * ((e + 1) & 31))));
            }
            x0 = (e < nvalid) ? x0 : -CUDART_INF_F;                      // keys beyond the sequence end
            x1 = (e + 1 < nvalid) ? x1 : -CUDART_INF_F;
            s[e] = x0; s[e + 1] = x1;
            const float a = ex2(fmaf(x0, sl2, -m_prev)), b = ex2(fmaf(x1, sl2, -m_prev));
            lsum += a + b;
            pk[e / 2] = pack_bf16x2(a, b);
            if ((e / 2) % 4 == 3) tmem_st4(tP + (uint32_t)(e / 2 - 3), pk[e / 2 - 3], pk[e / 2 - 2], pk[e / 2 - 1], pk[e / 2]);
            if (fuse && e / 2 == FCB) drain_begin(dc_src);
            if (fuse && e / 2 > FCB && e / 2 <= FCB + STG_COLS / GROUPS / 8) drain_step(e / 2 - FCB - 1, dc_src, dc_dst);
          }
        }
        // Tiles around a saturated one drain the next c2p band here, in one piece (the band product was issued when
        // this tile's p2c band left the buffer, at the top of the tile, and needs about this long).
        if (C2P && has_next && !fuse) drain_c(sat_n);
        // The barrier below closes the reads of the p2c staging rows of this key tile (so the next tile's band can
        // be drained into them) and carries a vote: only when some thread of the CTA saw a score far from the
        // reference exponent do the rows exchange their maxima and move the exponent; otherwise it simply stays.
        // The vote reads the row sums: an exponential above 2^8 (or an overflow) shows as a large sum, a first tile
        // far below the exponent as a vanishing one.  The maxima themselves are only formed when the vote passes.
        const bool vote = (lsum > 256.f) || (it == 0 && nvalid > 0 && lsum < 1.7e-18f);
        const bool moved = bar_all_cuda_warps_or(vote);
        float m_new = m_prev, alpha = 1.f;
        if (moved) {
          float mx = -CUDART_INF_F;
#pragma unroll
          for (int e = 0; e < KPT; ++e) mx = fmaxf(mx, s[e]);
          sts_f32(x_mine, mx);
          bar_all_cuda_warps();
#pragma unroll
          for (int gg = 0; gg < GROUPS; ++gg) mx = fmaxf(mx, lds_f32(sX + 4u * (uint32_t)(gg * BQ + row_t)));
          const float row_max = mx * sl2;                              // sl2 > 0
          const float excess = row_max - m_prev;
          const bool redo = (excess > 8.f) || (it == 0 && excess < -64.f);
          if (__any_sync(0xffffffffu, redo)) {
            // The store to tensor memory is a warp-wide instruction, so the whole warp forms its P again (rows that
            // keep their exponent get the same values as before) and overwrites what the loop stored.
            if (redo) {
              m_new = row_max;
              alpha = ex2(m_prev - m_new);
            }
            lsum = 0.f;
#pragma unroll
            for (int e = 0; e < KPT; e += 2) {
              const float a = ex2(fmaf(s[e], sl2, -m_new)), b = ex2(fmaf(s[e + 1], sl2, -m_new));
              lsum += a + b;
              pk[e / 2] = pack_bf16x2(a, b);
            }
            tmem_st_wait();
            tmem_st_cols<KPT / 2>(tP, pk);
          }
        }
        if (it > 0) {
          if (moved && __any_sync(0xffffffffu, alpha != 1.f)) {
            uint32_t r[OPT];
            tmem_ld_cols<OPT>(tO, r);
#pragma unroll
            for (int e = 0; e < OPT; ++e) r[e] = __float_as_uint(__uint_as_float(r[e]) * alpha);
            tmem_st_cols<OPT>(tO, r);
          }
        } else if (n > 0) {
          finish_item(n - 1, g - 1);       // also frees O and P for this tile's P.V (announced by P_READY below)
        }
        // A key tile with fewer than 128 valid keys: the probabilities of the keys beyond the sequence are exact zeros,
        // but what the caller left in the padding of V need not be finite, and 0 x NaN would reach every query row
        // of the tile.  The softmax threads zero those rows of the V tile (it has landed long ago) before they
        // announce P; the announcement orders the zeros before the product reads them.
        {
          const int nv_tile = cur.len - it * BK;
          if (nv_tile < BK) {
            wait(V_FULL, (uint32_t)(g & 1));
            for (int idx = tid; idx < (BK - nv_tile) * 8; idx += NCT)
              sts_128(sV + (uint32_t)(nv_tile + (idx >> 3)) * 128u + 16u * (uint32_t)(idx & 7), 0u, 0u, 0u, 0u);
            fence_proxy_async_smem();
          }
        }
        l_part = (it > 0 ? l_part * alpha : 0.f) + lsum;
        m_run = m_new;
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(P_READY));
        if (last_of_item) {                                            // what the item's epilogue needs from this thread
          sts_f32(lx_mine + (uint32_t)(n & 1) * (GROUPS * BQ * 4), l_part);
          if (grp == 0) sts_f32(mx_row + (uint32_t)(n & 1) * (BQ * 4), m_run);
        }
        ++g;
        if (!last_of_item) { ++it; continue; }
        ++n;
        it = 0;
        switch_item(n);
        if (cur.n_kv <= 0) break;
      }
      bar_all_cuda_warps();                                            // the last tile's row sums are in shared memory
      finish_item(n - 1, g - 1);
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
  if (warp == NCW + 1) tmem_dealloc(tmem, TM_COLS);
}

// ---------------------------------------------------------------------------------------------
PFN_cuTensorMapEncodeTiled_v12000 get_encode_fn() {
  // initialised once, by whichever thread comes first (function-local statics are thread-safe)
  static const PFN_cuTensorMapEncodeTiled_v12000 fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      return reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
    return static_cast<PFN_cuTensorMapEncodeTiled_v12000>(nullptr);
  }();
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

int table_map(CUtensorMap* m, const void* ptr, int rows, int H, int box_rows, const char* what) {
  uint64_t dims[3] = {(uint64_t)HD, (uint64_t)rows, (uint64_t)H};
  uint64_t strides[2] = {(uint64_t)HD * 2, (uint64_t)rows * HD * 2};
  uint32_t box[3] = {HD, (uint32_t)box_rows, 1};
  return encode_map(m, ptr, 3, dims, strides, box, what);
}

// The kernel needs more dynamic shared memory than the default limit; the attribute is per device and per
// instantiation, so it is set once for each pair, under a lock (entry points may be called from several host threads).
template <bool C2P, bool P2C, bool LONG>
int launch_variant(const AttnParams& p, dim3 grid, const CUtensorMap* maps, cudaStream_t s) {
  auto kern = attn_umma_kernel<C2P, P2C, LONG>;
  constexpr int MAX_DEV = 64;
  static std::mutex mu;
  static bool configured[MAX_DEV] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dev < 0 || dev >= MAX_DEV || !configured[dev]) {
      e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
      if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(max dynamic shared memory)");
      if (dev >= 0 && dev < MAX_DEV) configured[dev] = true;
    }
  }
  kern<<<grid, NTHREADS, SMEM_BYTES, s>>>(p, maps[0], maps[1], maps[2], maps[3], maps[4], maps[5], maps[6]);
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
  CUtensorMap maps[7];
  memset(maps, 0, sizeof(maps));
  const int64_t tokens = p.varlen ? p.total_tokens : p.L;
  const int B = p.varlen ? 1 : p.n_seqs;
  int rc;
  if ((rc = token_map(&maps[0], p.q, tokens, p.H, B, p.q_sb, p.q_st, p.q_sh, "q"))) return rc;
  if ((rc = token_map(&maps[1], p.k, tokens, p.H, B, p.k_sb, p.k_st, p.k_sh, "k"))) return rc;
  if ((rc = token_map(&maps[2], p.v, tokens, p.H, B, p.v_sb, p.v_st, p.v_sh, "v"))) return rc;
  if (p.flags & TDB_FLAG_C2P) {
    if ((rc = table_map(&maps[3], p.kr_exp, p.exp_rows, p.H, BAND, "kr_exp"))) return rc;
    if ((rc = table_map(&maps[5], p.kr_exp, p.exp_rows, p.H, SATN, "kr_exp (saturated tiles)"))) return rc;
  } else { maps[3] = maps[0]; maps[5] = maps[0]; }
  if (p.flags & TDB_FLAG_P2C) {
    if ((rc = table_map(&maps[4], p.qr_exp, p.exp_rows, p.H, BAND, "qr_exp"))) return rc;
    if ((rc = table_map(&maps[6], p.qr_exp, p.exp_rows, p.H, SATN, "qr_exp (saturated tiles)"))) return rc;
  } else { maps[4] = maps[0]; maps[6] = maps[0]; }

  // Persistent CTAs: one per SM (201 KB of shared memory and all 512 tensor-memory columns each), never more
  // than there are work items (query tiles x heads).
  int dev = 0, sms = 0;
  if ((rc = cuda_fail(cudaGetDevice(&dev), "cudaGetDevice"))) return rc;
  if ((rc = cuda_fail(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev), "cudaDeviceGetAttribute"))) return rc;
  int64_t tiles;
  if (p.varlen) {
    tiles = (p.total_tokens + BQ - 1) / BQ + p.n_seqs + 1;           // upper bound; the device list has the real count
    if (tiles * p.H > 0x7fffffff) { set_error("too many tiles"); return TDB_ERR_SHAPE; }
    build_tile_list_kernel<<<1, 1024, 0, s>>>(p.cu_seqlens, p.n_seqs, p.total_tokens,
                                              reinterpret_cast<int32_t*>(p.workspace), (int)tiles, p.status);
    if ((rc = cuda_fail(cudaGetLastError(), "build_tile_list launch"))) return rc;
  } else {
    tiles = (int64_t)p.n_seqs * ((p.L + BQ - 1) / BQ);
    if (tiles * p.H > 0x7fffffff) { set_error("too many tiles"); return TDB_ERR_SHAPE; }
  }
  const int64_t items = tiles * p.H;
  dim3 grid((unsigned)(items < sms ? items : sms), 1, 1);
  // status word 2 is the device-wide work counter of this launch; start it at zero even if the caller reuses the words
  if ((rc = cuda_fail(cudaMemsetAsync(p.status + 2, 0, sizeof(int32_t), s), "cudaMemsetAsync(work counter)"))) return rc;
  const bool c2p = p.flags & TDB_FLAG_C2P, p2c = p.flags & TDB_FLAG_P2C;
  // Saturated tiles exist only if a sequence exceeds the saturation distance by a tile; the variant that handles
  // them specially is a little slower on ordinary tiles, so it is used from twice that length on (p.L is the
  // padded length or the caller's max_seqlen).
  const bool lng = (c2p || p2c) && p.L >= 2 * (p.exp_delta_max - TDB_EXPAND_MARGIN) + BK;
  if (c2p && p2c) return lng ? launch_variant<true, true, true>(p, grid, maps, s) : launch_variant<true, true, false>(p, grid, maps, s);
  if (c2p) return lng ? launch_variant<true, false, true>(p, grid, maps, s) : launch_variant<true, false, false>(p, grid, maps, s);
  if (p2c) return lng ? launch_variant<false, true, true>(p, grid, maps, s) : launch_variant<false, true, false>(p, grid, maps, s);
  return launch_variant<false, false, false>(p, grid, maps, s);
}

}  // namespace tdb
