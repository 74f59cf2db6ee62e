// Flash-attention forward for sm_100a: TMA-staged tiles, tcgen05 MMAs with
// accumulators in tensor memory, warp-specialised roles.
//
// One CTA owns 256 query rows of one (batch, query head) as two 128-row tiles
// that ping-pong on the tensor core: while the softmax warps of one tile work on
// its scores, the MMAs of the other tile run.  K and V tiles are loaded once per
// CTA and used by both query tiles.
//
//   warp 0      TMA producer (one lane): Q tiles, then a K ring and a V ring
//   warp 1      MMA issuer (one lane): S_t = Q_t.K^T (both operands in shared
//               memory), O_t += P_t.V (P_t read from tensor memory, V in shared
//               memory, MN-major)
//   warps 2-5   softmax of tile 0: one thread per query row, the row's scores held
//               in registers (all tensor-memory loads in flight at once)
//   warps 6-9   softmax of tile 1
//
// Tensor memory (columns): S0 | S1 | O0 | O1, 128 lanes = 128 query rows.  P_t is
// written over S_t as packed 16-bit pairs, so the next S_t MMA is issued only
// after the P_t.V MMAs (same issuing thread, executed in order).
//
// Softmax arithmetic is the reference kernel's
// (probjax/nn/pallas_kernels/kernels/attention.py:456-529): fp32 scores, scale,
// bias, mask, exp2 domain, P rounded to the input dtype, O divided by the row sum
// at the end.  The running maximum is only advanced when it grew by more than 8
// (a factor 256), which leaves the result unchanged and skips most rescales.
//
// Every barrier wait is bounded: on expiry the role raises the CTA abort flag,
// all roles drain, tensor memory is freed and the status word gets
// PJX_ERR_DEVICE_TIMEOUT.
#include <atomic>
#include <cstdlib>
#include <mutex>
#include <type_traits>

#include "pjx_common.cuh"
#include "sm100_ptx.cuh"

namespace pjx {
namespace {

using namespace sm100;

// Timing experiments (python -m probjax_b200.build --what-if N): 0 = the shipped kernel.
#ifndef PJX_EXP_VARIANT
#define PJX_EXP_VARIANT 0
#endif

constexpr int BM = 128;          // rows per query tile (= tensor-memory lanes)
constexpr int NTHREADS = 320;    // 10 warps

// Optional phase timeline of one CTA (debug builds only, -DPJX_TRACE): role r
// (0/1 = softmax of tile 0/1, 2 = MMA issuer) stamps clock64() at point `pt` of KV
// iteration j.
#ifdef PJX_TRACE
__device__ long long g_trace[3][64][8];
#define PJX_TRACE_AT(r, j, pt)                                                                   \
  do {                                                                                           \
    if (blockIdx.x == gridDim.x / 2 && (j) < 64 &&                                               \
        ((r) == 2 || (threadIdx.x & 127) == 64))                                                 \
      g_trace[(r)][(j)][(pt)] = clock64();                                                       \
  } while (0)
// Per-CTA timeline: [0] SM id, then clock64 at [1] entry, [2] first S MMA issued, [3] last MMA
// issued, [4] epilogue of tile 1 begins, [5] exit; [6] globaltimer at entry.
__device__ long long g_cta[8192][8];
#define PJX_CTA_AT(slot)                                                        \
  do {                                                                          \
    if (blockIdx.x < 8192) g_cta[blockIdx.x][(slot)] = clock64();               \
  } while (0)
#else
#define PJX_TRACE_AT(r, j, pt) do {} while (0)
#define PJX_CTA_AT(slot) do {} while (0)
#endif

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float y;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(y) : "f"(a), "f"(b), "f"(c));
  return y;
}

template <int DQK, int DV, int BN, int KST, int VST, bool BIAS_STAGED = false, bool REL_STAGED = false>
struct Cfg {
  static constexpr int Q_SUB = DQK / 64, V_SUB = DV / 64;
  static constexpr int Q_TILE_BYTES = Q_SUB * BM * 128;
  static constexpr int K_TILE_BYTES = Q_SUB * BN * 128;
  static constexpr int V_TILE_BYTES = V_SUB * BN * 128;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + 2 * Q_TILE_BYTES;
  static constexpr int OFF_V = OFF_K + KST * K_TILE_BYTES;
  // staged bias: per query tile one fp32 [128 rows x BN keys] tile as BN/32 boxes of 128 x 32 (128-byte rows)
  static constexpr int BIAS_TILE_BYTES = BIAS_STAGED ? (BN / 32) * BM * 128 : 0;
  static constexpr int OFF_BIAS = OFF_V + VST * V_TILE_BYTES;
  // window of a relative-position table that one (query tile, KV tile) pair uses: 2 BM - 1 entries per query
  // tile, one buffer each.  Only the instantiation that reads it reserves it, and only 2 KB: at (128,128) a
  // double-buffered 4 KB pushed the CTA from the 196 KB shared-memory configuration to the 228 KB one, and
  // the 32 KB of L1 that takes away made every variant that spills 12-20 % slower when all of them carried it.
  static constexpr int REL_BYTES = REL_STAGED ? 2 * (2 * BM) * 4 : 0;
  static constexpr int OFF_REL = OFF_BIAS + 2 * BIAS_TILE_BYTES;
  static constexpr int OFF_BAR = OFF_REL + REL_BYTES;
  static constexpr int N_BAR = 2 + 2 * KST + 2 * VST + 6 + 4 + 2 + 1 + 2;
  static constexpr int SMEM_BYTES = OFF_BAR + N_BAR * 8 + 16 + 1024;  // + alignment slack
  static constexpr int TMEM_USED = 2 * BN + 2 * DV;
  static constexpr int TMEM_COLS = TMEM_USED <= 128 ? 128 : (TMEM_USED <= 256 ? 256 : 512);
  static_assert(TMEM_USED <= 512, "tensor memory has 512 columns");
  static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
};

template <bool BF16>
__device__ __forceinline__ uint32_t pack16(float lo, float hi) {
  if constexpr (BF16) {
    __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&t);
  } else {
    __half2 t = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&t);
  }
}

// p = exp2(x * cs - m) for one row of BN scores, running sums, pack to 16 bits and
// store over the scores in tensor memory. All exponentials of the row form one
// straight-line block (the stores come last) so that the scheduler can overlap the
// latencies of independent elements.
template <int BN, bool BF16>
__device__ __forceinline__ void exp_pack_store(const float (&s)[BN], float2 cs2, float2 nm2, float2& sum0,
                                               float2& sum1, uint32_t s_addr) {
  uint32_t pk[BN / 2];
#pragma unroll
  for (int i = 0; i < BN / 2; i += 2) {
    const float2 x0 = __ffma2_rn(make_float2(s[2 * i], s[2 * i + 1]), cs2, nm2);
    const float2 x1 = __ffma2_rn(make_float2(s[2 * i + 2], s[2 * i + 3]), cs2, nm2);
    const float2 p0 = make_float2(ex2_approx(x0.x), ex2_approx(x0.y));
    const float2 p1 = make_float2(ex2_approx(x1.x), ex2_approx(x1.y));
    sum0 = __fadd2_rn(sum0, p0);
    sum1 = __fadd2_rn(sum1, p1);
    pk[i] = pack16<BF16>(p0.x, p0.y);
    pk[i + 1] = pack16<BF16>(p1.x, p1.y);
  }
#if PJX_EXP_VARIANT == 11
#pragma unroll
  for (int i = 0; i < BN / 2; ++i) asm volatile("" ::"r"(pk[i]));
#else
#pragma unroll
  for (int c = 0; c < BN / 64; ++c) tmem_st32(s_addr + c * 32, *reinterpret_cast<const uint32_t(*)[32]>(&pk[c * 32]));
#endif
}

// The same with EMU of every 4 score pairs exponentiated on the FMA pipe instead of the
// special-function unit: x = n + f with n = round(x), f in [-0.5, 0.5]; 2^f as a degree-3
// polynomial (max relative error 7.5e-5, far below the 16-bit rounding of P); n is added to the
// exponent field.  x is clamped at -126, so the result is never exactly 0: only for tiles that
// need no mask (a masked score must give exactly 0).
template <int BN, bool BF16, int EMU>
__device__ __forceinline__ void exp_pack_store_emu(const float (&s)[BN], float2 cs2, float2 nm2, float2& sum0,
                                                   float2& sum1, uint32_t s_addr) {
  uint32_t pk[BN / 2];
  const float2 magic = make_float2(12582912.f, 12582912.f), nmagic = make_float2(-12582912.f, -12582912.f);
  const float2 neg1 = make_float2(-1.f, -1.f);
  const float2 c0 = make_float2(0.9999280572f, 0.9999280572f), c1 = make_float2(0.6932609677f, 0.6932609677f);
  const float2 c2 = make_float2(0.2426111251f, 0.2426111251f), c3 = make_float2(0.0551716648f, 0.0551716648f);
#pragma unroll
  for (int i = 0; i < BN / 2; ++i) {
    float2 x = __ffma2_rn(make_float2(s[2 * i], s[2 * i + 1]), cs2, nm2);
    float2 p;
    if ((i & 3) < EMU) {
      x.x = fmaxf(x.x, -126.f);
      x.y = fmaxf(x.y, -126.f);
      const float2 r = __fadd2_rn(x, magic);
      const float2 f = __ffma2_rn(__fadd2_rn(r, nmagic), neg1, x);
      float2 q = __ffma2_rn(f, c3, c2);
      q = __ffma2_rn(q, f, c1);
      q = __ffma2_rn(q, f, c0);
      p.x = __uint_as_float(__float_as_uint(q.x) + (__float_as_uint(r.x) << 23));
      p.y = __uint_as_float(__float_as_uint(q.y) + (__float_as_uint(r.y) << 23));
    } else {
#if PJX_EXP_VARIANT == 9
      p = x;
#else
      p = make_float2(ex2_approx(x.x), ex2_approx(x.y));
#endif
    }
    if (i & 1) sum1 = __fadd2_rn(sum1, p); else sum0 = __fadd2_rn(sum0, p);
    pk[i] = pack16<BF16>(p.x, p.y);
  }
#pragma unroll
  for (int c = 0; c < BN / 64; ++c) tmem_st32(s_addr + c * 32, *reinterpret_cast<const uint32_t(*)[32]>(&pk[c * 32]));
}

// The same with a multiplier per probability applied after it has been added to the row sum
// (dropout): dmul(i) is the multiplier of score column i.
template <int BN, bool BF16, typename F>
__device__ __forceinline__ void exp_pack_store_scaled(const float (&s)[BN], float2 cs2, float2 nm2, float2& sum0,
                                                      float2& sum1, uint32_t s_addr, F dmul) {
  uint32_t pk[BN / 2];
#pragma unroll
  for (int i = 0; i < BN / 2; i += 2) {
    const float2 x0 = __ffma2_rn(make_float2(s[2 * i], s[2 * i + 1]), cs2, nm2);
    const float2 x1 = __ffma2_rn(make_float2(s[2 * i + 2], s[2 * i + 3]), cs2, nm2);
    const float2 p0 = make_float2(ex2_approx(x0.x), ex2_approx(x0.y));
    const float2 p1 = make_float2(ex2_approx(x1.x), ex2_approx(x1.y));
    sum0 = __fadd2_rn(sum0, p0);
    sum1 = __fadd2_rn(sum1, p1);
    pk[i] = pack16<BF16>(p0.x * dmul(2 * i), p0.y * dmul(2 * i + 1));
    pk[i + 1] = pack16<BF16>(p1.x * dmul(2 * i + 2), p1.y * dmul(2 * i + 3));
  }
#pragma unroll
  for (int c = 0; c < BN / 64; ++c) tmem_st32(s_addr + c * 32, *reinterpret_cast<const uint32_t(*)[32]>(&pk[c * 32]));
}

// BIAS: 0 = no bias, 1 = bias read by each thread from global memory, 2 = bias tiles
// staged in shared memory by TMA (one row per thread out of global memory costs one
// L1 transaction per lane and instruction; the staged tile is read conflict-free).
//
// BAND: the mask is a band of visible keys around each query row (row + band_lo <= key <=
// row + band_hi) instead of the causal flag.  The KV loop then starts at the first tile that
// any row of the CTA can see; a query tile whose band begins later meets leading tiles it
// masks completely, which leaves its running state untouched.
//
// MOD (implies BAND): structured masks and score modifiers (score_mod.cuh) are evaluated by the
// softmax threads: level 1 holds the masks only (segment ids, per-row key limits, prefix), level 2
// also passes the scaled score of (row, key) through the score terms and applies dropout, level 3 is
// the masks and a relative-position table alone (every path that shares an instantiation costs the
// others registers: with the table's path inside level 2 its other terms ran 12-20 % slower).  No tile
// beyond the band / prefix range is visited; under a segment mask the launcher also gives every
// query tile the key range its ids can match, so tiles outside the range are skipped.
//
// SPLIT: the CTA takes one HALF of the KV tiles of its work item (two CTAs per item, blockIdx.x & 1 = the
// half) and leaves an fp32 partial -- O normalised by its own sum, base-2 log-sum-exp -- in a workspace
// (p.o / p.lse then point there); the half that finishes second merges the two and writes the result.  Used for the work items of a last, partly
// filled wave of a grid of equal items: 512 items on 148 SMs are 3.46 waves and cost 4; with the last 68
// items cut in two, 136 CTAs of half length fill that wave.
//
// `order_item0` packs the order block width (low 8 bits) and the index of the grid's first work item.
template <int DQK, int DV, int BN, int KST, int VST, bool BF16, int BIAS, bool BAND, int MOD = 0, bool SPLIT = false>
__global__ void __launch_bounds__(NTHREADS, 1)
attn_fwd_sm100_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_b,
                      const __grid_constant__ CUtensorMap tm_o, const FwdParamsCore p, const int order_item0,
                      const ScoreMod smod) {
  constexpr bool HAS_BIAS = BIAS != 0;
  static_assert(!SPLIT || (!BAND && !MOD && BIAS == 0), "KV halves are built for the plain variant");
  const int order_w = order_item0 & 0xff;
  const int item = (order_item0 >> 8) + (SPLIT ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x));
  const int half = SPLIT ? static_cast<int>(blockIdx.x & 1) : 0;
  static_assert(!MOD || (BAND && BIAS != 2), "the modifier variant builds on the band variant without staged bias");
  using C = Cfg<DQK, DV, BN, KST, VST, BIAS == 2, MOD == 3>;
  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar0 = sbase + C::OFF_BAR;
  auto BAR = [&](int i) { return bar0 + 8u * i; };
  // barrier indices
  const int Q_FULL = 0;                   // [2]
  const int K_FULL = 2;                   // [KST]
  const int K_EMPTY = K_FULL + KST;       // [KST]
  const int V_FULL = K_EMPTY + KST;       // [VST]
  const int V_EMPTY = V_FULL + VST;       // [VST]
  const int S_FULL = V_EMPTY + VST;       // [2]
  const int P_FULL = S_FULL + 2;          // [2]
  const int O_FULL = P_FULL + 2;          // [2]
  const int B_FULL = O_FULL + 2;          // [2] staged bias tile landed
  const int B_EMPTY = B_FULL + 2;         // [2] staged bias tile consumed (128 arrivals)
  const int O_STAGED = B_EMPTY + 2;       // [2] output tile written to shared memory (128 arrivals)
  const int V_CLEAN = O_STAGED + 2;       // rows past the valid length cleared in the last V tile (32 arrivals)
  [[maybe_unused]] const int REL_SYNC = V_CLEAN + 1;  // [2] table window of a query tile staged (128 arrivals)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + C::OFF_BAR + C::N_BAR * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Work order: the (batch, head) pairs are taken in blocks of `order_w`; inside a block the
  // query-tile index is the slow, descending axis. Under a causal mask the long CTAs of a
  // block therefore start first and its short ones fill the gaps; unmasked grids use blocks
  // of one pair, whose CTAs in flight share few K/V heads.
  const int n_bh = p.Hq * p.B;
  const int n_qt = (p.Lq + 2 * BM - 1) / (2 * BM);
  const int blk = item / (order_w * n_qt);
  const int rem = item - blk * (order_w * n_qt);
  const int wc = min(order_w, n_bh - blk * order_w);
  const int qt = n_qt - 1 - rem / wc;
  const int bh = blk * order_w + rem % wc;
  const int h = bh % p.Hq, b = bh / p.Hq;
  const int hk = h / (p.Hq / p.Hkv);
  const int q0 = qt * 2 * BM;

  int kv_len = p.Lkv;
  if constexpr (!SPLIT) {  // (a SPLIT launch has no key lengths; the field carries its arrival counters)
    if (p.kv_lengths) kv_len = max(0, min(kv_len, p.kv_lengths[b]));
  }
  int n_t[2];
  int j_base = 0;  // first KV tile of the loop (BAND only)
  if constexpr (BAND) {
    int lo_t[2], hi_t[2];
    j_base = 0x7fffffff;
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      const int qs = q0 + t * BM;
      lo_t[t] = hi_t[t] = 0;
      if (qs < p.Lq) {
        int end = max(0, min(kv_len, min(qs + BM, p.Lq) + p.band_hi));
        int begin = max(0, qs + p.band_lo);
        if constexpr (MOD) {
          if (smod.q_tile_range) {  // keys that can share a segment with a row of this tile
            const int32_t* r = smod.q_tile_range + ((int64_t)b * smod.q_tile_range_bs + qs / BM) * 2;
            begin = max(begin, r[0]);
            end = min(end, r[1]);
          }
          if (smod.prefix_len) {  // prefix keys are visible to every row
            const int pre = min(kv_len, smod.prefix_len[b]);
            if (pre > 0) {
              end = max(end, pre);
              begin = 0;
            }
          }
        }
        if (begin < end) {
          lo_t[t] = begin / BN;
          hi_t[t] = (end + BN - 1) / BN;
          j_base = min(j_base, lo_t[t]);
        }
      }
    }
#pragma unroll
    for (int t = 0; t < 2; ++t) n_t[t] = hi_t[t] > 0 ? hi_t[t] - j_base : 0;
    if (j_base == 0x7fffffff) j_base = 0;
  } else {
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      const int qs = q0 + t * BM;
      if (qs >= p.Lq) {
        n_t[t] = 0;
      } else {
        const int lim = p.causal ? min(kv_len, min(qs + BM, p.Lq)) : kv_len;
        n_t[t] = (lim + BN - 1) / BN;
      }
    }
    if constexpr (SPLIT) {  // this CTA's half of the tiles (the launcher takes unmasked problems only: equal counts)
      const int all = max(n_t[0], n_t[1]);
      j_base = half ? all / 2 : 0;
      const int mine = half ? all - all / 2 : all / 2;
#pragma unroll
      for (int t = 0; t < 2; ++t) n_t[t] = n_t[t] > 0 ? mine : 0;
    }
  }
  const int n = max(n_t[0], n_t[1]);
  // The last KV tile of the loop may reach past the valid length. Probabilities are exactly 0
  // there, but those rows may hold anything (a cache tail that was never written) and 0 x NaN
  // inside the P.V product is not 0: the producer warp clears them in shared memory once the
  // tile has landed, and the MMA issuer waits for that before the tile's P.V.
  const int clean_j = (n > 0 && (j_base + n) * BN > kv_len) ? n - 1 : -1;

  if (threadIdx.x == 0) {
#ifdef PJX_TRACE
    if (blockIdx.x < 8192) {
      unsigned smid;
      unsigned long long gt;
      asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt));
      g_cta[blockIdx.x][0] = smid;
      g_cta[blockIdx.x][6] = (long long)gt;
    }
#endif
    PJX_CTA_AT(1);
    for (int i = 0; i < C::N_BAR; ++i)
      mbar_init(BAR(i), i == V_CLEAN ? 32u : (((i >= P_FULL && i < P_FULL + 2) || i >= B_EMPTY) ? 128u : 1u));
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(tmem_slot), C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0 && n > 0) {
      prefetch_tmap(&tm_q);
      prefetch_tmap(&tm_k);
      prefetch_tmap(&tm_v);
      if constexpr (BIAS == 2) prefetch_tmap(&tm_b);
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        if (n_t[t] == 0) continue;
        mbar_arrive_expect_tx(BAR(Q_FULL + t), C::Q_TILE_BYTES);
#pragma unroll
        for (int s = 0; s < C::Q_SUB; ++s)
          tma_load_4d(sbase + C::OFF_Q + t * C::Q_TILE_BYTES + s * BM * 128, &tm_q, BAR(Q_FULL + t), s * 64, h,
                      q0 + t * BM, b);
      }
      for (int j = 0; j < n; ++j) {
        const int ks = j % KST, vs = j % VST;
        if (!mbar_wait(BAR(K_EMPTY + ks), ((j / KST) & 1) ^ 1, abort_flag)) break;
        mbar_arrive_expect_tx(BAR(K_FULL + ks), C::K_TILE_BYTES);
#pragma unroll
        for (int s = 0; s < C::Q_SUB; ++s)
          tma_load_4d(sbase + C::OFF_K + ks * C::K_TILE_BYTES + s * BN * 128, &tm_k, BAR(K_FULL + ks), s * 64, hk,
                      (j_base + j) * BN, b);
        if (!mbar_wait(BAR(V_EMPTY + vs), ((j / VST) & 1) ^ 1, abort_flag)) break;
        mbar_arrive_expect_tx(BAR(V_FULL + vs), C::V_TILE_BYTES);
#pragma unroll
        for (int s = 0; s < C::V_SUB; ++s)
          tma_load_4d(sbase + C::OFF_V + vs * C::V_TILE_BYTES + s * BN * 128, &tm_v, BAR(V_FULL + vs), s * 64, hk,
                      (j_base + j) * BN, b);
        if constexpr (BIAS == 2) {
          bool okb = true;
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            if (j >= n_t[t]) continue;
            okb = mbar_wait(BAR(B_EMPTY + t), (j & 1) ^ 1, abort_flag);
            if (!okb) break;
            mbar_arrive_expect_tx(BAR(B_FULL + t), C::BIAS_TILE_BYTES);
#pragma unroll
            for (int c = 0; c < BN / 32; ++c)
              tma_load_4d(sbase + C::OFF_BIAS + t * C::BIAS_TILE_BYTES + c * BM * 128, &tm_b, BAR(B_FULL + t),
                          (j_base + j) * BN + c * 32, q0 + t * BM, p.bias_hs ? h : 0, p.bias_bs ? b : 0);
          }
          if (!okb) break;
        }
      }
    }
    __syncwarp();
    if (clean_j >= 0) {
      const int vs = clean_j % VST;
      if (mbar_wait(BAR(V_FULL + vs), (clean_j / VST) & 1, abort_flag)) {
        for (int r = kv_len - (j_base + clean_j) * BN + lane; r < BN; r += 32) {
          const uint32_t vrow = sbase + C::OFF_V + vs * C::V_TILE_BYTES + r * 128;
#pragma unroll
          for (int sub = 0; sub < C::V_SUB; ++sub)
#pragma unroll
            for (int u = 0; u < 8; ++u)
              asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};\n" ::"r"(vrow + sub * BN * 128 + u * 16), "r"(0) : "memory");
        }
        fence_proxy_async();
      }
      mbar_arrive(BAR(V_CLEAN));
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0 && n > 0) {
      constexpr uint32_t idesc_s = make_idesc(BM, BN, BF16, false, false);
      constexpr uint32_t idesc_o = make_idesc(BM, DV, BF16, false, true);
      auto issue_s = [&](int t, int j) {
        const uint32_t qa = sbase + C::OFF_Q + t * C::Q_TILE_BYTES;
        const uint32_t ka = sbase + C::OFF_K + (j % KST) * C::K_TILE_BYTES;
#pragma unroll
        for (int s = 0; s < C::Q_SUB; ++s)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            mma_ss(tmem + t * BN, make_smem_desc(qa + s * BM * 128 + kk * 32, 16, 1024),
                   make_smem_desc(ka + s * BN * 128 + kk * 32, 16, 1024), idesc_s, (s | kk) != 0);
      };
      auto issue_pv = [&](int t, int j) {
        const uint32_t va = sbase + C::OFF_V + (j % VST) * C::V_TILE_BYTES;
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk)
          mma_ts(tmem + 2 * BN + t * DV, tmem + t * BN + kk * 8, make_smem_desc(va + kk * 2048, BN * 128, 1024),
                 idesc_o, (j | kk) != 0);
      };
      bool ok = true;
#pragma unroll
      for (int t = 0; t < 2; ++t)
        if (ok && n_t[t] > 0) ok = mbar_wait(BAR(Q_FULL + t), 0, abort_flag);
      if (ok) ok = mbar_wait(BAR(K_FULL + 0), 0, abort_flag);
      if (ok) {
        tc_fence_after();
#pragma unroll
        for (int t = 0; t < 2; ++t)
          if (n_t[t] > 0) {
            issue_s(t, 0);
            mma_commit(BAR(S_FULL + t));
          }
        mma_commit(BAR(K_EMPTY + 0));
        PJX_CTA_AT(2);
      }
      for (int j = 0; ok && j < n; ++j) {
        const bool have_next = j + 1 < n;
        ok = mbar_wait(BAR(V_FULL + j % VST), (j / VST) & 1, abort_flag);
        if (ok && j == clean_j) ok = mbar_wait(BAR(V_CLEAN), 0, abort_flag);
        if (ok && have_next) ok = mbar_wait(BAR(K_FULL + (j + 1) % KST), ((j + 1) / KST) & 1, abort_flag);
        if (!ok) break;
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (j < n_t[t]) {
            PJX_TRACE_AT(2, j, 4 * t + 0);
            ok = mbar_wait(BAR(P_FULL + t), j & 1, abort_flag);
            if (!ok) break;
            tc_fence_after();
            PJX_TRACE_AT(2, j, 4 * t + 1);
            issue_pv(t, j);
            PJX_TRACE_AT(2, j, 4 * t + 2);
            if (j == n_t[t] - 1) mma_commit(BAR(O_FULL + t));
          }
          if (j + 1 < n_t[t]) {
            issue_s(t, j + 1);
            mma_commit(BAR(S_FULL + t));
            PJX_TRACE_AT(2, j, 4 * t + 3);
          }
        }
        if (!ok) break;
        mma_commit(BAR(V_EMPTY + j % VST));
        if (have_next) mma_commit(BAR(K_EMPTY + (j + 1) % KST));
      }
      PJX_CTA_AT(3);
    }
  } else {
    // ------------------------------------------------------------ softmax warps
    const int t = (warp - 2) >> 2;
    const int quarter = warp & 3;  // tensor-memory lane quarter this warp may access
    const int r_in = quarter * 32 + lane;
    const int row = q0 + t * BM + r_in;
    const bool row_ok = row < p.Lq;
    const int my_n = t ? n_t[1] : n_t[0];
    const uint32_t lane_sel = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t s_addr = tmem + lane_sel + t * BN;
    const uint32_t o_addr = tmem + lane_sel + 2 * BN + t * DV;
    const float c1 = p.sm_scale * kLog2e;
    const float* bias_row = nullptr;
    if (BIAS == 1 && row_ok) bias_row = p.bias + (int64_t)b * p.bias_bs + (int64_t)h * p.bias_hs + (int64_t)row * p.Lkv;
    const bool bias_vec = BIAS == 1 && (p.Lkv % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.bias) & 15) == 0) &&
                          (p.bias_bs % 4 == 0) && (p.bias_hs % 4 == 0);
    ScoreModView mv = {};
    int my_seg = 0, my_limit = 0x7fffffff;
    bool mod_terms = false;  // a modifier changes the scores (not only the mask)
    [[maybe_unused]] int mod_kind = 0;
    bool seg_vec = false;    // the key-side segment ids can be read four at a time
    if constexpr (MOD) {
      mv = view_of(smod, b, h, p.Lq);
      if (row_ok && mv.seg_q) my_seg = mv.seg_q[row];
      if (row_ok && mv.row_limit) my_limit = mv.row_limit[row];
      if constexpr (MOD >= 2) {  // which score terms are on: head scale 1, soft cap 2, relative table 4, ALiBi 8 / 16
        mod_kind = (mv.hscale_m1 != 0.f ? 1 : 0) | (mv.softcap > 0.f ? 2 : 0) | (mv.rel != nullptr ? 4 : 0) | (mv.alibi_mode << 3);
        mod_terms = mod_kind != 0;
      }
      seg_vec = mv.seg_k != nullptr && (reinterpret_cast<uintptr_t>(mv.seg_k) & 15) == 0;
    }
    // scores reach the exponential already in the exp2 domain when a bias or a score modifier was applied
    // (a positive per-head scale alone is folded into that multiplier: the row maximum is taken before it)
    const bool hs_fold = MOD == 2 && !HAS_BIAS && mod_kind == 1 && mv.hscale_m1 > -1.f;
    const float cs = HAS_BIAS ? 1.f : hs_fold ? c1 * (1.f + mv.hscale_m1) : (MOD >= 2 && mod_terms) ? 1.f : c1;

    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < my_n; ++j) {
      PJX_TRACE_AT(t, j, 0);
      ok = mbar_wait(BAR(S_FULL + t), j & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      PJX_TRACE_AT(t, j, 1);
#if PJX_EXP_VARIANT == 12
      l = 1.f;
      tc_fence_before();
      mbar_arrive(BAR(P_FULL + t));
      continue;
#endif
      constexpr int NCH = BN / 32;
      const int k0 = (j_base + j) * BN;
      bool need_mask;
      if constexpr (MOD) {  // band, lengths, per-row limits and the prefix; the segment test comes after it
        const bool band_cut = (k0 + BN - 1 > q0 + t * BM + p.band_hi) || (k0 < q0 + t * BM + BM - 1 + p.band_lo);
        // (a tile inside the prefix is visible whatever the band says; a row limit matters to the rows it cuts)
        need_mask = (k0 + BN > kv_len) || (band_cut && k0 + BN > mv.prefix) || my_limit < k0 + BN;
      } else if constexpr (BAND) {
        need_mask = (k0 + BN > kv_len) || (k0 + BN - 1 > q0 + t * BM + p.band_hi) ||
                    (k0 < q0 + t * BM + BM - 1 + p.band_lo);
      } else {
        need_mask = (k0 + BN > kv_len) || (p.causal && k0 + BN - 1 > q0 + t * BM);
      }

      // The whole row of scores in registers: all loads in flight at once.
      float s[BN];
#if PJX_EXP_VARIANT == 10
#pragma unroll
      for (int i = 0; i < BN; ++i) s[i] = __int_as_float(0x3c000000 + ((i * 37 + j * 11 + lane) & 0xffff));
#else
#pragma unroll
      for (int c = 0; c < NCH; ++c) tmem_ld32f(s_addr + c * 32, &s[c * 32]);
      tmem_wait_ld();
#endif
      PJX_TRACE_AT(t, j, 2);

      if (MOD == 2 && mod_terms) {
        // scaled score -> modifiers -> exp2 domain; a dense bias (BIAS == 1) is added below on top.
        // One term alone (the usual case) has a loop of its own with no test per element; the values
        // written for rows past Lq and keys past kv_len are never used (not stored / masked below).
        const bool plain = !HAS_BIAS;
        if (plain && (mod_kind == 8 || mod_kind == 16)) {  // ALiBi: s - slope * distance
          // float arithmetic throughout (an integer-to-float conversion per element runs at a quarter of
          // the rate); a tile on one side of the diagonal has a distance that is linear in the key
          const float sl2 = mv.slope * kLog2e;
          const int d0 = row - k0;  // row - key at the tile's first key
          const float d0f = (float)d0;
          if (d0 >= BN - 1) {  // every key at or before the row
            const float base = -sl2 * d0f;
#pragma unroll
            for (int i = 0; i < BN; ++i) s[i] = fmaf(s[i], c1, fmaf(sl2, (float)i, base));
          } else if (d0 <= 0) {  // every key at or after the row: no penalty (causal form) or slope * (key - row)
            const float sl = mod_kind == 8 ? 0.f : sl2;
            const float base = sl * d0f;
#pragma unroll
            for (int i = 0; i < BN; ++i) s[i] = fmaf(s[i], c1, fmaf(-sl, (float)i, base));
          } else if (mod_kind == 8) {
#pragma unroll
            for (int i = 0; i < BN; ++i) s[i] = fmaf(s[i], c1, -sl2 * fmaxf(d0f - (float)i, 0.f));
          } else {
#pragma unroll
            for (int i = 0; i < BN; ++i) s[i] = fmaf(s[i], c1, -sl2 * fabsf(d0f - (float)i));
          }
        } else if (plain && mod_kind == 1) {  // per-head scale: folded into the multiplier of the exponential if positive
          if (!hs_fold) {
            const float c = c1 * (1.f + mv.hscale_m1);
#pragma unroll
            for (int i = 0; i < BN; ++i) s[i] *= c;
          }
        } else if (plain && mod_kind == 2) {  // soft cap: cap * tanh(s / cap)
          const float a = p.sm_scale / mv.softcap, c = mv.softcap * kLog2e;
#pragma unroll
          for (int i = 0; i < BN; ++i) {
            float th;
            asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(s[i] * a));
            s[i] = c * th;
          }
        } else {
#pragma unroll
          for (int i = 0; i < BN; ++i) {
            const int key = k0 + i;
            const float sc = s[i] * p.sm_scale;
            const float md = (row_ok && key < kv_len) ? mod_score<false>(mv, sc, row, key, nullptr) : sc;
            // the bias branch multiplies by c1 = sm_scale * log2(e) itself: hand it md / sm_scale
            s[i] = plain ? md * kLog2e : md / p.sm_scale;
          }
        }
      }
      if constexpr (MOD == 3 && C::REL_BYTES > 0) {  // a relative-position table alone, no dense bias
        // The 128 x 128 scores of a tile pair use 2 BM - 1 consecutive entries, table[key - row]: the tile's
        // 128 softmax threads stage them (times log2 e) in shared memory, meet at a bounded barrier, and row
        // r reads entry BM - 1 - r + i for key i -- consecutive lanes read consecutive words.  One buffer per
        // query tile and two phases of one barrier per KV tile: "window written" (waited for at once) and
        // "window read" (arrived at after the reads, waited for a whole tile later, before the next write).
        static_assert(BN == BM, "the window is laid out for square tile pairs");
        float* win = reinterpret_cast<float*>(smem + C::OFF_REL) + t * (2 * BM);
        if (j > 0) {
          ok = mbar_wait(BAR(REL_SYNC + t), 1, abort_flag);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
        }
        const int base = k0 - (q0 + t * BM) - (BM - 1);  // win[x] = table[base + x]
        for (int x = r_in; x < 2 * BM - 1; x += BM) {
          const int idx = base + x;
          win[x] = (idx > -p.Lq && idx < p.Lkv) ? __ldg(mv.rel + idx) * kLog2e : 0.f;
        }
        mbar_arrive(BAR(REL_SYNC + t));
        ok = mbar_wait(BAR(REL_SYNC + t), 0, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const float* mine = win + (BM - 1 - r_in);
#pragma unroll
        for (int i = 0; i < BN; ++i) s[i] = fmaf(s[i], c1, mine[i]);
        mbar_arrive(BAR(REL_SYNC + t));
      }
      if constexpr (BIAS == 2) {
        ok = mbar_wait(BAR(B_FULL + t), j & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const uint32_t brow = sbase + C::OFF_BIAS + t * C::BIAS_TILE_BYTES + r_in * 128;
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            float4 bv;
            asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];\n"
                         : "=f"(bv.x), "=f"(bv.y), "=f"(bv.z), "=f"(bv.w)
                         : "r"(brow + c * BM * 128 + ((i ^ (r_in & 7)) << 4)));
            s[c * 32 + 4 * i + 0] = fmaf(bv.x, kLog2e, s[c * 32 + 4 * i + 0] * c1);
            s[c * 32 + 4 * i + 1] = fmaf(bv.y, kLog2e, s[c * 32 + 4 * i + 1] * c1);
            s[c * 32 + 4 * i + 2] = fmaf(bv.z, kLog2e, s[c * 32 + 4 * i + 2] * c1);
            s[c * 32 + 4 * i + 3] = fmaf(bv.w, kLog2e, s[c * 32 + 4 * i + 3] * c1);
          }
        }
        mbar_arrive(BAR(B_EMPTY + t));
      } else if constexpr (BIAS == 1) {
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          const int kc = k0 + c * 32;
          if (bias_row && bias_vec && kc + 32 <= p.Lkv) {
            const float4* bp = reinterpret_cast<const float4*>(bias_row + kc);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float4 bv = __ldg(bp + i);
              s[c * 32 + 4 * i + 0] = fmaf(bv.x, kLog2e, s[c * 32 + 4 * i + 0] * c1);
              s[c * 32 + 4 * i + 1] = fmaf(bv.y, kLog2e, s[c * 32 + 4 * i + 1] * c1);
              s[c * 32 + 4 * i + 2] = fmaf(bv.z, kLog2e, s[c * 32 + 4 * i + 2] * c1);
              s[c * 32 + 4 * i + 3] = fmaf(bv.w, kLog2e, s[c * 32 + 4 * i + 3] * c1);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const float bv = (bias_row && kc + i < p.Lkv) ? __ldg(bias_row + kc + i) : 0.f;
              s[c * 32 + i] = fmaf(bv, kLog2e, s[c * 32 + i] * c1);
            }
          }
        }
      }
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < BN; ++i) {
          const int key = k0 + i;
          bool keep;
          if constexpr (MOD) {
            keep = (key <= row + p.band_hi && key >= row + p.band_lo) || key < mv.prefix;
            keep = keep && key < kv_len && key < my_limit;
          } else if constexpr (BAND) {
            keep = key < kv_len && key <= row + p.band_hi && key >= row + p.band_lo;
          } else {
            keep = key < kv_len && (!p.causal || key <= row);
          }
          s[i] = keep ? s[i] : -INFINITY;
        }
      }
      if constexpr (MOD) {
        if (mv.seg_k) {
          // Same-segment test, one load per warp and tile: lane L reads the ids of keys k0 + 4 L .. + 3, and
          // for every distinct row id in the warp four ballots give the 128 keep bits of the rows that carry
          // it.  A row whose bits are all set (the tile lies inside its segment) has nothing to mask.  Keys
          // at and past kv_len are masked above: every tile that holds one needs the mask.
          static_assert(BN == 128, "four keys per lane");
          int4 g = make_int4(0, 0, 0, 0);
          if (seg_vec && k0 + BN <= p.Lkv) {
            g = __ldg(reinterpret_cast<const int4*>(mv.seg_k + k0) + lane);
          } else {
            const int kk = k0 + 4 * lane;
            if (kk + 0 < p.Lkv) g.x = __ldg(mv.seg_k + kk + 0);
            if (kk + 1 < p.Lkv) g.y = __ldg(mv.seg_k + kk + 1);
            if (kk + 2 < p.Lkv) g.z = __ldg(mv.seg_k + kk + 2);
            if (kk + 3 < p.Lkv) g.w = __ldg(mv.seg_k + kk + 3);
          }
          uint32_t bits0 = 0, bits1 = 0, bits2 = 0, bits3 = 0;
          uint32_t remaining = 0xffffffffu;
          while (remaining) {  // warp-uniform
            const int v = __shfl_sync(0xffffffffu, my_seg, __ffs(remaining) - 1);
            const uint32_t b0 = __ballot_sync(0xffffffffu, g.x == v), b1 = __ballot_sync(0xffffffffu, g.y == v);
            const uint32_t b2 = __ballot_sync(0xffffffffu, g.z == v), b3 = __ballot_sync(0xffffffffu, g.w == v);
            if (my_seg == v) {
              bits0 = b0; bits1 = b1; bits2 = b2; bits3 = b3;
            }
            remaining &= ~__ballot_sync(0xffffffffu, my_seg == v);
          }
          if ((bits0 & bits1 & bits2 & bits3) != 0xffffffffu) {
#pragma unroll
            for (int i = 0; i < BN / 4; ++i) {
              s[4 * i + 0] = (bits0 >> i) & 1u ? s[4 * i + 0] : -INFINITY;
              s[4 * i + 1] = (bits1 >> i) & 1u ? s[4 * i + 1] : -INFINITY;
              s[4 * i + 2] = (bits2 >> i) & 1u ? s[4 * i + 2] : -INFINITY;
              s[4 * i + 3] = (bits3 >> i) & 1u ? s[4 * i + 3] : -INFINITY;
            }
          }
        }
      }

      float mx;
      {
        float m[8];  // independent chains
#pragma unroll
        for (int i = 0; i < 8; ++i) m[i] = fmaxf(s[2 * i], s[2 * i + 1]);
#pragma unroll
        for (int i = 1; i < BN / 16; ++i)
#pragma unroll
          for (int u = 0; u < 8; ++u) m[u] = fmax3(m[u], s[16 * i + 2 * u], s[16 * i + 2 * u + 1]);
        mx = fmaxf(fmaxf(fmaxf(m[0], m[1]), fmaxf(m[2], m[3])), fmaxf(fmaxf(m[4], m[5]), fmaxf(m[6], m[7])));
      }
      mx *= cs;  // cs > 0
#if PJX_EXP_VARIANT == 13
      mx = 4.f;
#endif

      // lazy running maximum: advance only when it grew by more than 8 (base 2)
      const bool need = (mx > m_ref + 8.f) || (m_ref == -INFINITY && mx > -INFINITY);
      const bool rescale = __any_sync(0xffffffffu, need);
      float corr = 1.f;
      if (rescale) {
        const float m_new = fmaxf(m_ref, mx);
        corr = (m_new == -INFINITY) ? 1.f : exp2f(m_ref - m_new);
        m_ref = m_new;
        l *= corr;
      }

      // p = exp2(x * cs - m), row sum, pack to 16 bits, store over S
      const float neg_m = (m_ref == -INFINITY) ? 0.f : -m_ref;
      const float2 cs2 = make_float2(cs, cs), nm2 = make_float2(neg_m, neg_m);
      float2 sum0 = make_float2(0.f, 0.f), sum1 = make_float2(0.f, 0.f);
      PJX_TRACE_AT(t, j, 3);
      if constexpr (MOD == 2) {
        if (mv.drop_rate > 0.f)
          exp_pack_store_scaled<BN, BF16>(s, cs2, nm2, sum0, sum1, s_addr, [&](int i) { return mod_dropout(mv, row, k0 + i); });
        else
          exp_pack_store<BN, BF16>(s, cs2, nm2, sum0, sum1, s_addr);
      } else {
#if PJX_EXP_VARIANT == 0 || PJX_EXP_VARIANT >= 10
        exp_pack_store<BN, BF16>(s, cs2, nm2, sum0, sum1, s_addr);
#elif PJX_EXP_VARIANT == 9
        exp_pack_store_emu<BN, BF16, 0>(s, cs2, nm2, sum0, sum1, s_addr);
#else
        if (need_mask)
          exp_pack_store<BN, BF16>(s, cs2, nm2, sum0, sum1, s_addr);
        else
          exp_pack_store_emu<BN, BF16, PJX_EXP_VARIANT>(s, cs2, nm2, sum0, sum1, s_addr);
#endif
      }
      PJX_TRACE_AT(t, j, 4);
      const float lsum = (sum0.x + sum0.y) + (sum1.x + sum1.y);

      // rescale O only now: the score registers are free again (the previous P.V of this
      // tile completed before these scores became visible)
      if (rescale && j > 0) {
#pragma unroll
        for (int c = 0; c < DV / 32; ++c) {
          float o[32];
          tmem_ld32f(o_addr + c * 32, o);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] *= corr;
          tmem_st32f(o_addr + c * 32, o);
        }
      }
      l += lsum;
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(BAR(P_FULL + t));
      PJX_TRACE_AT(t, j, 5);
    }

    if (ok && (q0 + t * BM) < p.Lq) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      if (my_n > 0) {
        ok = mbar_wait(BAR(O_FULL + t), 0, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
      }
      // SPLIT: this half's fp32 partial goes to the workspace; the half that arrives second (a counter per work
      // item and query tile) merges both and writes the final rows, so no CTA ever waits for another.
      float ca = inv, cb = 0.f;          // final value = O_tmem * ca + other_partial * cb
      const float* other = nullptr;
      float lse_final = 0.f;
      bool writes_out = true;
      if constexpr (SPLIT) {
        if (ok) {
          tc_fence_after();
          const int64_t slot = ((int64_t)(blockIdx.x >> 1) * 2 + t) * BM + r_in;
          const int64_t slots = (int64_t)(gridDim.x >> 1) * 2 * BM;
          float* po = static_cast<float*>(p.o) + ((int64_t)half * slots + slot) * DV;
#pragma unroll
          for (int c = 0; c < DV / 32; ++c) {
            float o[32];
            tmem_ld32f(o_addr + c * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 8; ++i)
              *reinterpret_cast<float4*>(po + c * 32 + 4 * i) =
                  make_float4(o[4 * i] * inv, o[4 * i + 1] * inv, o[4 * i + 2] * inv, o[4 * i + 3] * inv);
          }
          const float lse_self = l > 0.f ? m_ref + log2f(l) : -INFINITY;
          p.lse[half * slots + slot] = lse_self;
          __threadfence();
          // rendezvous of the tile's 128 threads (the bias barrier of this tile is free in this variant), one
          // counter increment, second rendezvous to hand its result round
          volatile int* arrived = reinterpret_cast<volatile int*>(tmem_slot + 2 + t);
          mbar_arrive(BAR(B_EMPTY + t));
          ok = mbar_wait(BAR(B_EMPTY + t), 0, abort_flag);
          ok = __all_sync(0xffffffffu, ok);
          if (ok) {
            if (r_in == 0)
              *arrived = atomicAdd(const_cast<int32_t*>(p.kv_lengths) + (blockIdx.x >> 1) * 2 + t, 1);
            mbar_arrive(BAR(B_EMPTY + t));
            ok = mbar_wait(BAR(B_EMPTY + t), 1, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
          }
          writes_out = ok && *arrived == 1;
          if (writes_out) {
            __threadfence();
            const int64_t oslot = (int64_t)(half ^ 1) * slots + slot;
            other = static_cast<const float*>(p.o) + oslot * DV;
            const float lse_other = p.lse[oslot];
            const float mx = fmaxf(lse_self, lse_other);
            const float ws = mx == -INFINITY ? 0.f : exp2f(lse_self - mx), wo = mx == -INFINITY ? 0.f : exp2f(lse_other - mx);
            const float den = ws + wo;
            ca = ws;  // weights of this half and of the other; the merge below is written in half order,
            cb = wo;  // so that the result does not depend on which half arrived second
            lse_final = den > 0.f ? (mx + log2f(den)) * kLn2 : INFINITY;
          }
        }
      }
      if (ok && !writes_out) {
        // first half to arrive: nothing more to do
      } else if (ok) {
        tc_fence_after();
        if (threadIdx.x == 320 - 128) PJX_CTA_AT(4);
        // O leaves through shared memory: every thread writes its row (16-bit, 128-byte-swizzled
        // like the tensor map expects) over the query tile, which the MMAs no longer read, and one
        // thread hands the tile to a TMA store, which clips rows past Lq. Stores straight from the
        // registers would touch 32 separate rows per instruction.
        const uint32_t stage = sbase + C::OFF_Q + t * C::Q_TILE_BYTES;
        const float out_scale = SPLIT ? 1.f : inv;  // a merged value carries its normalisation already
        const float iden = (ca + cb) > 0.f ? 1.f / (ca + cb) : 0.f;  // SPLIT: 1 / (sum of the halves' weights)
#pragma unroll
        for (int c = 0; c < DV / 32; ++c) {
          float o[32];
          if (my_n > 0) {
            tmem_ld32f(o_addr + c * 32, o);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = 0.f;
          }
          if constexpr (SPLIT) {  // merged value of the two halves, the other half's partial read back from L2
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float4 w = *reinterpret_cast<const float4*>(other + c * 32 + 4 * i);
              const float ov[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float mine = __fmul_rn(__fmul_rn(o[4 * i + e], inv), ca);  // o * inv is what this half stored
                const float theirs = __fmul_rn(ov[e], cb);
                const float sum = half ? __fadd_rn(theirs, mine) : __fadd_rn(mine, theirs);
                o[4 * i + e] = __fmul_rn(sum, iden);
              }
            }
          }
          // columns 32c .. 32c+31 = 16-byte units 4(c%2) .. 4(c%2)+3 of the 128-byte row in block c/2
          const uint32_t rbase = stage + (c >> 1) * (BM * 128) + r_in * 128;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t unit = static_cast<uint32_t>((c & 1) * 4 + i) ^ static_cast<uint32_t>(r_in & 7);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};\n" ::"r"(rbase + unit * 16),
                         "r"(pack16<BF16>(o[8 * i + 0] * out_scale, o[8 * i + 1] * out_scale)),
                         "r"(pack16<BF16>(o[8 * i + 2] * out_scale, o[8 * i + 3] * out_scale)),
                         "r"(pack16<BF16>(o[8 * i + 4] * out_scale, o[8 * i + 5] * out_scale)),
                         "r"(pack16<BF16>(o[8 * i + 6] * out_scale, o[8 * i + 7] * out_scale))
                         : "memory");
          }
        }
        fence_proxy_async();
        mbar_arrive(BAR(O_STAGED + t));
        if (r_in == 0 && mbar_wait(BAR(O_STAGED + t), 0, abort_flag)) {
#pragma unroll
          for (int s = 0; s < DV / 64; ++s) tma_store_4d(&tm_o, stage + s * (BM * 128), s * 64, h, q0 + t * BM, b);
          tma_store_commit();
          tma_store_wait_read();
        }
        if constexpr (SPLIT) {  // p.bias carries the caller's LSE pointer in this variant
          float* lse_out = const_cast<float*>(p.bias);
          if (lse_out && row_ok) lse_out[((int64_t)b * p.Hq + h) * p.Lq + row] = lse_final;
        } else {
          if (p.lse && row_ok)
            p.lse[((int64_t)b * p.Hq + h) * p.Lq + row] = l > 0.f ? (m_ref + log2f(l)) * kLn2 : INFINITY;
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    __syncwarp();
    tmem_dealloc(tmem, C::TMEM_COLS);
    if (lane == 0) PJX_CTA_AT(5);
    if (lane == 0 && *abort_flag && p.status) atomicExch(p.status, (int)PJX_ERR_DEVICE_TIMEOUT);
  }
}

// ---------------------------------------------------------------------------
// Host side: tensor maps and launch
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      f = nullptr;
    return reinterpret_cast<EncodeTiledFn>(f);
  }();
  return fn;
}

}  // namespace

// [B, L, H, Dim] row-major 16-bit tensor, box = 64 elements x 1 head x `rows` tokens.
int make_tmap_blhd(CUtensorMap* m, const void* base, int dtype, int B, int L, int H, int Dim, int rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(PJX_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[4] = {(cuuint64_t)Dim, (cuuint64_t)H, (cuuint64_t)L, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)Dim * 2, (cuuint64_t)H * Dim * 2, (cuuint64_t)L * H * Dim * 2};
  cuuint32_t box[4] = {64, 1, (cuuint32_t)rows, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(m, dtype == PJX_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                  const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(PJX_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return PJX_OK;
}

namespace {

// fp32 bias [Bb, Hb, Lq, Lkv] (strides in elements, 0 = broadcast): box = 32 keys x 128 rows.
int make_tmap_bias(CUtensorMap* m, const FwdParams& p) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(PJX_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  const cuuint64_t hb = p.bias_hs ? p.Hq : 1, bb = p.bias_bs ? p.B : 1;
  const cuuint64_t plane = (cuuint64_t)p.Lq * p.Lkv;
  cuuint64_t dims[4] = {(cuuint64_t)p.Lkv, (cuuint64_t)p.Lq, hb, bb};
  cuuint64_t strides[3] = {(cuuint64_t)p.Lkv * 4, (p.bias_hs ? (cuuint64_t)p.bias_hs : plane) * 4,
                           (p.bias_bs ? (cuuint64_t)p.bias_bs : plane * hb) * 4};
  cuuint32_t box[4] = {32, (cuuint32_t)BM, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(p.bias), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(PJX_ERR_CUDA, "cuTensorMapEncodeTiled (bias) failed with CUresult %d", (int)r);
  return PJX_OK;
}

bool bias_can_be_staged(const FwdParams& p) {
  return p.bias && p.Lkv % 4 == 0 && (reinterpret_cast<uintptr_t>(p.bias) & 15) == 0 && p.bias_hs % 4 == 0 &&
         p.bias_bs % 4 == 0;
}

// The partials of the KV halves come from the stream-ordered allocator.  Its default pool hands freed memory
// back to the driver at every synchronisation, which would make each call pay for a fresh mapping: keep it.
void keep_pool_memory() {
  static std::atomic<bool> done[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64 || done[dev].exchange(true)) return;
  cudaMemPool_t pool;
  if (cudaDeviceGetDefaultMemPool(&pool, dev) == cudaSuccess) {
    uint64_t keep = 256ull << 20;  // the partials are at most 74 items x 2 halves x 256 rows x Dv floats (< 40 MB)
    uint64_t cur = 0;
    if (cudaMemPoolGetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &cur) == cudaSuccess && cur < keep)
      cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
  }
}

// A second stream per device for the halves: they do not depend on the full-length CTAs, and launched beside
// them their CTAs take over SMs one by one as the last full wave drains, instead of waiting for all of it.
struct SideStream {
  cudaStream_t stream = nullptr;
  cudaEvent_t fork = nullptr, join = nullptr;
  std::mutex mu;  // held while one call enqueues its fork / launch / join
};
SideStream* side_stream() {
  static SideStream side[64];
  static std::mutex create_mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  SideStream& s = side[dev];
  std::lock_guard<std::mutex> lock(create_mu);
  if (!s.stream) {
    if (cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&s.fork, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&s.join, cudaEventDisableTiming) != cudaSuccess) {
      (void)cudaGetLastError();
      s.stream = nullptr;
      return nullptr;
    }
  }
  return &s;
}

int sm_count() {
  int dev = 0, v = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v < 1)
    v = 148;
  return v;
}

// Key range per tile of 128 query rows under a segment mask (ScoreMod::q_tile_range): one CTA per
// (tile, batch row of the ids).
__global__ void __launch_bounds__(128) seg_tile_range_kernel(const int32_t* __restrict__ seg_q, const int32_t* __restrict__ seg_k,
                                                             int64_t sq_bs, int64_t sk_bs, int Lq, int Lkv,
                                                             int32_t* __restrict__ out) {
  __shared__ int red[4][2];
  const int tile = blockIdx.x, bs = blockIdx.y, tid = threadIdx.x;
  const int32_t* sq = seg_q + (int64_t)bs * sq_bs;
  const int32_t* sk = seg_k + (int64_t)bs * sk_bs;
  auto block_min_max = [&](int& lo, int& hi) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, o));
      hi = max(hi, __shfl_xor_sync(0xffffffffu, hi, o));
    }
    __syncthreads();  // the previous round's values have been read
    if ((tid & 31) == 0) {
      red[tid >> 5][0] = lo;
      red[tid >> 5][1] = hi;
    }
    __syncthreads();
    lo = min(min(red[0][0], red[1][0]), min(red[2][0], red[3][0]));
    hi = max(max(red[0][1], red[1][1]), max(red[2][1], red[3][1]));
  };
  const int row = tile * 128 + tid;
  int smin = 0x7fffffff, smax = (int)0x80000000;
  if (row < Lq) smin = smax = sq[row];
  block_min_max(smin, smax);
  int first = 0x7fffffff, last = -1;
  for (int j = tid; j < Lkv; j += 128) {
    const int s = sk[j];
    if (s >= smin && s <= smax) {
      first = min(first, j);
      last = max(last, j);
    }
  }
  block_min_max(first, last);
  if (tid == 0) {
    int32_t* r = out + ((int64_t)bs * gridDim.x + tile) * 2;
    r[0] = last < 0 ? 0 : first;
    r[1] = last + 1;
  }
}

template <int DQK, int DV, int BN, int KST, int VST, bool BF16, int BIAS, bool BAND = false, int MOD = 0>
int launch_one(const FwdParams& p, int dtype, cudaStream_t stream) {
  using C = Cfg<DQK, DV, BN, KST, VST, BIAS == 2, MOD == 3>;
  CUtensorMap tq, tk, tv, tb;
  int rc;
  if ((rc = make_tmap_blhd(&tq, p.q, dtype, p.B, p.Lq, p.Hq, DQK, BM))) return rc;
  if ((rc = make_tmap_blhd(&tk, p.k, dtype, p.B, p.Lkv, p.Hkv, DQK, BN))) return rc;
  if ((rc = make_tmap_blhd(&tv, p.v, dtype, p.B, p.Lkv, p.Hkv, DV, BN))) return rc;
  if (BIAS == 2) {
    if ((rc = make_tmap_bias(&tb, p))) return rc;
  } else {
    tb = tq;  // unused
  }
  CUtensorMap to;
  if ((rc = make_tmap_blhd(&to, p.o, dtype, p.B, p.Lq, p.Hq, DV, BM))) return rc;
  auto kern = attn_fwd_sm100_kernel<DQK, DV, BN, KST, VST, BF16, BIAS, BAND, MOD>;
  if ((rc = check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES),
                       "cudaFuncSetAttribute(sm100 fwd)")))
    return rc;
  dim3 grid((unsigned)(((p.Lq + 2 * BM - 1) / (2 * BM)) * (int64_t)p.Hq * p.B));
  // Triangular work (an upper bound on the keys only): heavy-first order inside blocks of (batch, head) pairs.
  // Wider blocks balance better (causal headline shape, blocks of 4 / 8 / 16 / 32 / 64 / 128 pairs: 919 / 935 / 936 /
  // 940 / 947 / 948 TFLOP/s) until the K and V of the pairs in flight no longer fit the near L2 partition (latent
  // shape, 16 heads with K / V of their own: 64 pairs 0.333 ms, 16 pairs 0.320 ms): blocks whose K / V take 32 MB.
  int order_w = 1;
  if (p.band_hi < PJX_BAND_NO_UPPER && p.band_lo == PJX_BAND_NO_LOWER) {
    const double kv_bytes_per_pair = (double)p.Lkv * (DQK + DV) * 2.0 * p.Hkv / p.Hq;
    order_w = 4;
    while (order_w < 128 && 2.0 * order_w * kv_bytes_per_pair <= 32.0 * 1024 * 1024) order_w *= 2;
  }
  if constexpr (BIAS == 0 && !BAND && !MOD && DQK == DV) {
    // Equal work items (no mask, no key lengths) come in waves of one CTA per SM; a last wave that fills at
    // most half of the SMs is cut into KV halves (two CTAs per item, fp32 partials, one small merge kernel).
    const int64_t n_items = grid.x;
    const int sms = sm_count();
    const int64_t full = n_items / sms * sms;
    const int tail = (int)(n_items - full);
    const int n_kv = (p.Lkv + BN - 1) / BN;
    static const bool off = getenv("PJX_FWD_SPLIT_TAIL") && atoi(getenv("PJX_FWD_SPLIT_TAIL")) == 0;
    if (!off && !p.causal && !p.kv_lengths && tail > 0 && 2 * tail <= sms && n_kv >= 8 && n_items < (1 << 23)) {
      const size_t slots = (size_t)tail * 2 * BM;
      const size_t o_bytes = 2 * slots * DV * sizeof(float), l_bytes = 2 * slots * sizeof(float);
      const size_t c_bytes = (size_t)tail * 2 * sizeof(int32_t);  // arrivals per (work item, query tile)
      void* ws = nullptr;
      keep_pool_memory();
      if (cudaMallocAsync(&ws, o_bytes + l_bytes + c_bytes, stream) == cudaSuccess) {
        int32_t* counters = reinterpret_cast<int32_t*>(static_cast<char*>(ws) + o_bytes + l_bytes);
        rc = check_cuda(cudaMemsetAsync(counters, 0, c_bytes, stream), "clear arrival counters");
        auto kern_h = attn_fwd_sm100_kernel<DQK, DV, BN, KST, VST, BF16, 0, false, false, true>;
        if (!rc)
          rc = check_cuda(cudaFuncSetAttribute(kern_h, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES),
                          "cudaFuncSetAttribute(sm100 fwd, KV halves)");
        SideStream* side = (!rc && full > 0) ? side_stream() : nullptr;
        cudaStream_t hstream = stream;  // where the halves go
        std::unique_lock<std::mutex> side_lock;
        if (side) {
          side_lock = std::unique_lock<std::mutex>(side->mu);
          if (cudaEventRecord(side->fork, stream) == cudaSuccess && cudaStreamWaitEvent(side->stream, side->fork, 0) == cudaSuccess)
            hstream = side->stream;
          else
            (void)cudaGetLastError();
        }
        if (!rc) {
          if (full > 0) {
            kern<<<dim3((unsigned)full), NTHREADS, C::SMEM_BYTES, stream>>>(tq, tk, tv, tb, to,
                                                                            static_cast<const FwdParamsCore&>(p), order_w, p.mod);
            count_launch();
          }
          // the halves: partials and their LSE in the workspace; the fields this variant does not use carry the
          // arrival counters (kv_lengths) and the caller's LSE pointer (bias)
          FwdParamsCore ph = static_cast<const FwdParamsCore&>(p);
          ph.o = ws;
          ph.lse = reinterpret_cast<float*>(static_cast<char*>(ws) + o_bytes);
          ph.kv_lengths = counters;
          ph.bias = p.lse;
          kern_h<<<dim3(2u * (unsigned)tail), NTHREADS, C::SMEM_BYTES, hstream>>>(tq, tk, tv, tb, to, ph,
                                                                                order_w | ((int)full << 8), p.mod);
          count_launch();
          rc = check_cuda(cudaGetLastError(), "sm100 forward launch (with KV halves)");
          if (hstream != stream) {  // the caller's stream continues after both grids
            if (!rc) rc = check_cuda(cudaEventRecord(side->join, hstream), "record the halves' completion");
            if (!rc) rc = check_cuda(cudaStreamWaitEvent(stream, side->join, 0), "join the halves");
          }
        }
        cudaFreeAsync(ws, stream);
        return rc;
      }
      (void)cudaGetLastError();  // no memory for the partials: one grid as usual
    }
  }
  if constexpr (MOD) {
    // Segment masks: the KV loop of a query tile is cut to the keys whose ids can match (worth a small
    // kernel of its own from a few KV tiles on; without memory for the ranges every tile is visited).
    if (p.mod.seg_q && p.mod.seg_k && !p.mod.prefix_len && p.Lkv > 2 * BN) {
      const int tiles = (p.Lq + BM - 1) / BM;
      const int nb = (p.mod.seg_q_bs == 0 && p.mod.seg_k_bs == 0) ? 1 : p.B;
      void* ranges = nullptr;
      keep_pool_memory();
      if (nb <= 65535 && cudaMallocAsync(&ranges, (size_t)nb * tiles * 2 * sizeof(int32_t), stream) == cudaSuccess) {
        seg_tile_range_kernel<<<dim3(tiles, nb), 128, 0, stream>>>(p.mod.seg_q, p.mod.seg_k, p.mod.seg_q_bs, p.mod.seg_k_bs,
                                                                   p.Lq, p.Lkv, static_cast<int32_t*>(ranges));
        count_launch();
        ScoreMod mod = p.mod;
        mod.q_tile_range = static_cast<const int32_t*>(ranges);
        mod.q_tile_range_bs = nb == 1 ? 0 : tiles;
        kern<<<grid, NTHREADS, C::SMEM_BYTES, stream>>>(tq, tk, tv, tb, to, static_cast<const FwdParamsCore&>(p), order_w, mod);
        count_launch();
        rc = check_cuda(cudaGetLastError(), "sm100 forward launch (segment ranges)");
        cudaFreeAsync(ranges, stream);
        return rc;
      }
      (void)cudaGetLastError();
    }
  }
  kern<<<grid, NTHREADS, C::SMEM_BYTES, stream>>>(tq, tk, tv, tb, to, static_cast<const FwdParamsCore&>(p), order_w, p.mod);
  count_launch();
  return check_cuda(cudaGetLastError(), "sm100 forward launch");
}

template <int DQK, int DV, int BN, int KST, int VST, bool BF16>
int launch_cfg(const FwdParams& p, int dtype, cudaStream_t stream) {
  if (p.mod.on) {
    // level 1: masks only (segments, per-row limits, prefix); level 2: score terms and dropout as well
    const bool terms = p.mod.rel_bias || p.mod.alibi_slopes || p.mod.head_scale || p.mod.softcap > 0.f || p.mod.dropout_rate > 0.f;
    // level 3: a relative-position table as the only score term and no dense bias (the table's window is staged)
    if (p.mod.rel_bias && !p.mod.alibi_slopes && !p.mod.head_scale && !(p.mod.softcap > 0.f) && !(p.mod.dropout_rate > 0.f) && !p.bias)
      return launch_one<DQK, DV, BN, KST, VST, BF16, 0, true, 3>(p, dtype, stream);
    if (!terms) {
      if (!p.bias) return launch_one<DQK, DV, BN, KST, VST, BF16, 0, true, 1>(p, dtype, stream);
      return launch_one<DQK, DV, BN, KST, VST, BF16, 1, true, 1>(p, dtype, stream);
    }
    if (!p.bias) return launch_one<DQK, DV, BN, KST, VST, BF16, 0, true, 2>(p, dtype, stream);
    return launch_one<DQK, DV, BN, KST, VST, BF16, 1, true, 2>(p, dtype, stream);
  }
  if (p.banded()) {
    if (!p.bias) return launch_one<DQK, DV, BN, KST, VST, BF16, 0, true>(p, dtype, stream);
    return launch_one<DQK, DV, BN, KST, VST, BF16, 1, true>(p, dtype, stream);
  }
  if (!p.bias) return launch_one<DQK, DV, BN, KST, VST, BF16, 0>(p, dtype, stream);
  return launch_one<DQK, DV, BN, KST, VST, BF16, 1>(p, dtype, stream);
}

template <bool BF16>
int launch_by_shape(const FwdParams& p, int dtype, cudaStream_t stream) {
  if (p.D == 128 && p.Dv == 128) return launch_cfg<128, 128, 128, 2, 2, BF16>(p, dtype, stream);
  if (p.D == 64 && p.Dv == 64) {
    // with a bias that TMA can address, two K/V stages leave room for the staged bias tiles
    if (bias_can_be_staged(p) && !p.banded() && !p.mod.on) return launch_one<64, 64, 128, 2, 2, BF16, 2>(p, dtype, stream);
    return launch_cfg<64, 64, 128, 3, 3, BF16>(p, dtype, stream);
  }
  if (p.D == 192 && p.Dv == 128) return launch_cfg<192, 128, 128, 1, 2, BF16>(p, dtype, stream);
  return fail(PJX_ERR_UNSUPPORTED, "tcgen05 forward: head dims (%d, %d) not built", p.D, p.Dv);
}

}  // namespace

bool fwd_sm100_supported(const FwdParams& p, int dtype, const char** why) {
  const char* w = nullptr;
  if (dtype != PJX_BF16 && dtype != PJX_F16) w = "dtype must be bf16 or fp16";
  else if (!((p.D == 128 && p.Dv == 128) || (p.D == 64 && p.Dv == 64) || (p.D == 192 && p.Dv == 128)))
    w = "head dims must be (64,64), (128,128) or (192,128)";
  else if (!(p.sm_scale > 0.f)) w = "sm_scale must be positive";
  else if (p.B < 1 || p.Lq < 1 || p.Lkv < 1) w = "empty problem";
  else if (((p.Lq + 2 * BM - 1) / (2 * BM)) * (int64_t)p.Hq * p.B > 0x7fffffffLL) w = "grid too large";
  else if ((reinterpret_cast<uintptr_t>(p.q) | reinterpret_cast<uintptr_t>(p.k) | reinterpret_cast<uintptr_t>(p.v) |
            reinterpret_cast<uintptr_t>(p.o)) & 15)
    w = "q, k, v, o must be 16-byte aligned";
  if (why) *why = w;
  return w == nullptr;
}

#ifdef PJX_TRACE
extern "C" int pjx_debug_read_trace(long long* host_out) {
  return (int)cudaMemcpyFromSymbol(host_out, g_trace, sizeof(long long) * 3 * 64 * 8);
}
extern "C" int pjx_debug_read_cta(long long* host_out) {
  return (int)cudaMemcpyFromSymbol(host_out, g_cta, sizeof(long long) * 8192 * 8);
}
#endif

int launch_fwd_sm100(const FwdParams& p, int dtype, cudaStream_t stream) {
  const char* why = nullptr;
  if (!fwd_sm100_supported(p, dtype, &why)) return fail(PJX_ERR_UNSUPPORTED, "tcgen05 forward: %s", why);
  return dtype == PJX_BF16 ? launch_by_shape<true>(p, dtype, stream) : launch_by_shape<false>(p, dtype, stream);
}

}  // namespace pjx
