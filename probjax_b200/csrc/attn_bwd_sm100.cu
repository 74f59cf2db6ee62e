// Flash-attention backward for sm_100a: TMA-staged tiles, tcgen05 MMAs with accumulators in
// tensor memory.  Two kernels without atomics (the reference splits its backward the same way,
// probjax/nn/pallas_kernels/kernels/attention.py:1189-1483 `mha_backward_kernel_split_dkdv` and
// `_split_dq`), both recomputing P = exp(s - lse) from the forward's log-sum-exp:
//
//   dQ kernel     one CTA per 128-row query tile of a (batch, query head), walking the KV tiles:
//                   S = Q.K^T, dP = dO.V^T            (both operands in shared memory)
//                   dS = P o (dP - delta)              (compute warps, one thread per query row)
//                   dQ += dS.K                         (dS read from tensor memory, K MN-major)
//   dK/dV kernel  one CTA per 128-key tile of a (batch, KV head), walking the query tiles of all
//                 query heads of the group (GQA gradients are summed inside the CTA):
//                   S^T = K.Q^T, dP^T = V.dO^T
//                   P^T, dS^T                          (compute warps, one thread per key row)
//                   dV += P^T.dO,  dK += dS^T.Q       (A from tensor memory, dO / Q MN-major)
//
// Transposed scores in the dK/dV kernel put the keys on the tensor-memory lanes, so P^T and dS^T
// are already laid out as the A operand of the two accumulating products.  P and dS are rounded
// to the input dtype before those products, as the reference does.  Scaling by sm_scale is
// applied once, when dQ and dK leave tensor memory.
//
// Warps: 0 = TMA producer, 1 = MMA issuer (one lane), 2-5 and 6-9 = two compute groups; a group
// has one thread per tensor-memory lane (query row, or key row in the dK/dV kernel) and takes
// one half of the 128 score columns, so that every scheduler has two compute warps to
// interleave.  A group writes its 16-bit results over the first 32 columns of its own half,
// which it has read already.  The MMA issuer works in half steps: the score products of half A of
// the next step are issued as soon as half A of this step has been accumulated, so the tensor
// core works on one half while a compute group works on the other.  Every barrier wait is
// bounded; on expiry the CTA drains, frees tensor memory and reports PJX_ERR_DEVICE_TIMEOUT.
#include "pjx_common.cuh"
#include "sm100_ptx.cuh"

namespace pjx {

int make_tmap_blhd(CUtensorMap* m, const void* base, int dtype, int B, int L, int H, int Dim, int rows);

namespace {

using namespace sm100;

constexpr int BM = 128;        // query rows per tile
constexpr int BN = 128;        // keys per tile
constexpr int NTHREADS = 320;  // 10 warps

// Optional phase timeline of one CTA of the dQ kernel (debug builds only, -DPJX_TRACE).
#ifdef PJX_TRACE
__device__ long long g_btrace[4][64][8];
#define PJX_BTRACE(r, j, pt)                                                                     \
  do {                                                                                           \
    if (blockIdx.x == gridDim.x / 2 && (j) < 64)                                                 \
      g_btrace[(r)][(j)][(pt)] = clock64();                                                      \
  } while (0)
#define PJX_KTRACE(r, j, pt)                                                                     \
  do {                                                                                           \
    if (blockIdx.x == gridDim.x / 2 && (j) < 64)                                                 \
      g_btrace[2 + (r)][(j)][(pt)] = clock64();                                                  \
  } while (0)
#else
#define PJX_BTRACE(r, j, pt) do {} while (0)
#define PJX_KTRACE(r, j, pt) do {} while (0)
#endif

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

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

// Work order of a 1-D grid over (tile, pair) with `n_tiles` tiles per pair and `n_pairs` pairs
// (a pair is a (batch, head)): pairs are taken in blocks of `order_w`; inside a block the tile
// index is the slow axis, so that under a causal band the long CTAs of a block start first
// (callers number the tiles heaviest-first) while the CTAs in flight share few K/V heads.
__device__ __forceinline__ void work_item(int id, int n_tiles, int n_pairs, int order_w, int& tile, int& pair) {
  const int blk = id / (order_w * n_tiles);
  const int rem = id - blk * (order_w * n_tiles);
  const int wc = min(order_w, n_pairs - blk * order_w);
  tile = rem / wc;
  pair = blk * order_w + rem % wc;
}

// dS of 32 score columns of one query row: p = exp2(s c1 - lse2), dS = p (dP - delta), packed to
// 16 bits.  Straight-line over independent elements so that the scheduler can overlap them.
template <bool BF16>
__device__ __forceinline__ void ds_row_chunk(const float (&s)[32], const float (&dp)[32], float c1, float neg_lse2,
                                             float neg_delta, float (&d)[32]) {
  const float2 c2 = make_float2(c1, c1), nl2 = make_float2(neg_lse2, neg_lse2), nd2 = make_float2(neg_delta, neg_delta);
#pragma unroll
  for (int i = 0; i < 16; i += 2) {
    const float2 x0 = __ffma2_rn(make_float2(s[2 * i], s[2 * i + 1]), c2, nl2);
    const float2 x1 = __ffma2_rn(make_float2(s[2 * i + 2], s[2 * i + 3]), c2, nl2);
    const float2 p0 = make_float2(ex2_approx(x0.x), ex2_approx(x0.y));
    const float2 p1 = make_float2(ex2_approx(x1.x), ex2_approx(x1.y));
    const float2 e0 = __fadd2_rn(make_float2(dp[2 * i], dp[2 * i + 1]), nd2);
    const float2 e1 = __fadd2_rn(make_float2(dp[2 * i + 2], dp[2 * i + 3]), nd2);
    const float2 d0 = __fmul2_rn(p0, e0), d1 = __fmul2_rn(p1, e1);
    d[2 * i] = d0.x;
    d[2 * i + 1] = d0.y;
    d[2 * i + 2] = d1.x;
    d[2 * i + 3] = d1.y;
  }
}

// Rows of `Dh` 16-bit elements leave tensor memory (32 columns at a time), are scaled and
// written to a [.., rows, heads, Dh] tensor; `dst` points at this thread's row.
template <int Dh, bool BF16>
__device__ __forceinline__ void store_row(uint32_t taddr, unsigned char* dst, float scale, bool have_acc, bool row_ok) {
#pragma unroll
  for (int c = 0; c < Dh / 32; ++c) {
    float o[32];
    if (have_acc) {
      tmem_ld32f(taddr + c * 32, o);
      tmem_wait_ld();
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) o[i] = 0.f;
    }
    if (row_ok) {
      uint4* d4 = reinterpret_cast<uint4*>(dst + c * 64);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        uint4 w;
        w.x = pack16<BF16>(o[8 * i + 0] * scale, o[8 * i + 1] * scale);
        w.y = pack16<BF16>(o[8 * i + 2] * scale, o[8 * i + 3] * scale);
        w.z = pack16<BF16>(o[8 * i + 4] * scale, o[8 * i + 5] * scale);
        w.w = pack16<BF16>(o[8 * i + 6] * scale, o[8 * i + 7] * scale);
        d4[i] = w;
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// dQ kernel
// ---------------------------------------------------------------------------------------------
template <int D>
struct DqCfg {
  static constexpr int SUB = D / 64;               // 64-element (128-byte) column blocks of a row
  static constexpr int TILE = SUB * 128 * 128;     // bytes of a 128-row tile
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_DO = TILE;
  static constexpr int OFF_K = 2 * TILE;           // 2 stages
  static constexpr int OFF_V = 4 * TILE;           // 2 stages
  static constexpr int OFF_BAR = 6 * TILE;
  // barriers: QDO_FULL, K_FULL[2], K_EMPTY[2], V_FULL[2], V_EMPTY[2], SP_FULL[2], DS_FULL[2], DQ_FULL, K_CLEAN
  static constexpr int N_BAR = 15;
  static constexpr int SMEM_BYTES = OFF_BAR + N_BAR * 8 + 16 + 1024;
  static constexpr int TMEM_COLS = 512;            // S 128 | dP 128 | dQ D
  static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
};

template <int D, bool BF16>
__global__ void __launch_bounds__(NTHREADS, 1)
bwd_dq_sm100_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                    const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                    const BwdParams p, const int order_w) {
  using C = DqCfg<D>;
  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar0 = sbase + C::OFF_BAR;
  auto BAR = [&](int i) { return bar0 + 8u * i; };
  const int QDO_FULL = 0, K_FULL = 1, K_EMPTY = 3, V_FULL = 5, V_EMPTY = 7, SP_FULL = 9, DS_FULL = 11, DQ_FULL = 13,
            K_CLEAN = 14;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + C::OFF_BAR + C::N_BAR * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qt = (p.Lq + BM - 1) / BM;
  int tile, pair;
  work_item(blockIdx.x, n_qt, p.Hq * p.B, order_w, tile, pair);
  const int qt = n_qt - 1 - tile;  // the last query tiles see the most keys under a causal band
  const int h = pair % p.Hq, b = pair / p.Hq;
  const int hk = h / (p.Hq / p.Hkv);
  const int q0 = qt * BM;

  int kv_len = p.Lkv;
  if (p.kv_lengths) kv_len = max(0, min(kv_len, p.kv_lengths[b]));
  // KV tiles any row of this query tile can see
  const int kv_end = max(0, min(kv_len, min(q0 + BM, p.Lq) + p.band_hi));
  const int kv_begin = max(0, q0 + p.band_lo);
  const int j_lo = kv_begin / BN;
  const int n = kv_begin < kv_end ? (kv_end + BN - 1) / BN - j_lo : 0;
  // The last KV tile may reach past the valid length: dS is exactly 0 there, but those K rows may
  // hold anything and 0 x NaN inside dQ += dS.K is not 0. The producer warp clears them in shared
  // memory once the tile has landed; the MMA issuer waits for that before it uses the tile.
  const int clean_j = (n > 0 && (j_lo + n) * BN > kv_len) ? n - 1 : -1;

  if (threadIdx.x == 0) {
    for (int i = 0; i < C::N_BAR; ++i)
      mbar_init(BAR(i), i == K_CLEAN ? 32u : ((i == DS_FULL || i == DS_FULL + 1) ? 128u : 1u));
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
  const uint32_t T_S = tmem, T_DP = tmem + BN, T_DQ = tmem + 2 * BN;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0 && n > 0) {
      prefetch_tmap(&tm_q);
      prefetch_tmap(&tm_do);
      prefetch_tmap(&tm_k);
      prefetch_tmap(&tm_v);
      mbar_arrive_expect_tx(BAR(QDO_FULL), 2 * C::TILE);
#pragma unroll
      for (int s = 0; s < C::SUB; ++s) {
        tma_load_4d(sbase + C::OFF_Q + s * BM * 128, &tm_q, BAR(QDO_FULL), s * 64, h, q0, b);
        tma_load_4d(sbase + C::OFF_DO + s * BM * 128, &tm_do, BAR(QDO_FULL), s * 64, h, q0, b);
      }
      for (int j = 0; j < n; ++j) {
        const int st = j & 1;
        if (!mbar_wait(BAR(K_EMPTY + st), ((j >> 1) & 1) ^ 1, abort_flag)) break;
        mbar_arrive_expect_tx(BAR(K_FULL + st), C::TILE);
#pragma unroll
        for (int s = 0; s < C::SUB; ++s)
          tma_load_4d(sbase + C::OFF_K + st * C::TILE + s * BN * 128, &tm_k, BAR(K_FULL + st), s * 64, hk,
                      (j_lo + j) * BN, b);
        if (!mbar_wait(BAR(V_EMPTY + st), ((j >> 1) & 1) ^ 1, abort_flag)) break;
        mbar_arrive_expect_tx(BAR(V_FULL + st), C::TILE);
#pragma unroll
        for (int s = 0; s < C::SUB; ++s)
          tma_load_4d(sbase + C::OFF_V + st * C::TILE + s * BN * 128, &tm_v, BAR(V_FULL + st), s * 64, hk,
                      (j_lo + j) * BN, b);
      }
    }
    __syncwarp();
    if (clean_j >= 0) {
      const int st = clean_j & 1;
      if (mbar_wait(BAR(K_FULL + st), (clean_j >> 1) & 1, abort_flag)) {
        for (int r = kv_len - (j_lo + clean_j) * BN + lane; r < BN; r += 32) {
          const uint32_t krow = sbase + C::OFF_K + st * C::TILE + r * 128;
#pragma unroll
          for (int sub = 0; sub < C::SUB; ++sub)
#pragma unroll
            for (int u = 0; u < 8; ++u)
              asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};\n" ::"r"(krow + sub * BN * 128 + u * 16), "r"(0) : "memory");
        }
        fence_proxy_async();
      }
      mbar_arrive(BAR(K_CLEAN));
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && n > 0) {
      constexpr uint32_t idesc_s = make_idesc(BM, BN / 2, BF16, false, false);
      constexpr uint32_t idesc_q = make_idesc(BM, D, BF16, false, true);
      const uint32_t qa = sbase + C::OFF_Q, doa = sbase + C::OFF_DO;
      // S and dP of one half (64 keys) of KV tile j: the B operands start 64 rows into the tiles
      auto issue_sdp = [&](int half, int j) {
        const uint32_t ka = sbase + C::OFF_K + (j & 1) * C::TILE + half * 64 * 128;
        const uint32_t va = sbase + C::OFF_V + (j & 1) * C::TILE + half * 64 * 128;
#pragma unroll
        for (int s = 0; s < C::SUB; ++s)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            mma_ss(T_S + half * 64, make_smem_desc(qa + s * BM * 128 + kk * 32, 16, 1024),
                   make_smem_desc(ka + s * BN * 128 + kk * 32, 16, 1024), idesc_s, (s | kk) != 0);
#pragma unroll
        for (int s = 0; s < C::SUB; ++s)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            mma_ss(T_DP + half * 64, make_smem_desc(doa + s * BM * 128 + kk * 32, 16, 1024),
                   make_smem_desc(va + s * BN * 128 + kk * 32, 16, 1024), idesc_s, (s | kk) != 0);
        mma_commit(BAR(SP_FULL + half));
      };
      // dQ += dS.K over one half: A = dS (16-bit pairs at the first 32 columns of the half of S),
      // B = the K tile read MN-major
      auto issue_acc = [&](int half, int j) {
        const uint32_t ka = sbase + C::OFF_K + (j & 1) * C::TILE;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          mma_ts(T_DQ, T_S + half * 64 + kk * 8, make_smem_desc(ka + (half * 4 + kk) * 2048, BN * 128, 1024), idesc_q,
                 (j | half | kk) != 0);
      };
      bool ok = mbar_wait(BAR(QDO_FULL), 0, abort_flag);
      if (ok) ok = mbar_wait(BAR(K_FULL), 0, abort_flag);
      if (ok && clean_j == 0) ok = mbar_wait(BAR(K_CLEAN), 0, abort_flag);
      if (ok) ok = mbar_wait(BAR(V_FULL), 0, abort_flag);
      if (ok) {
        tc_fence_after();
        issue_sdp(0, 0);
        issue_sdp(1, 0);
        mma_commit(BAR(V_EMPTY));
      }
      for (int j = 0; ok && j < n; ++j) {
        const int st = j & 1;
        const bool next = j + 1 < n;
        PJX_BTRACE(0, j, 0);
        ok = mbar_wait(BAR(DS_FULL + 0), j & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        PJX_BTRACE(0, j, 1);
        issue_acc(0, j);
        if (next) {
          ok = mbar_wait(BAR(K_FULL + (st ^ 1)), ((j + 1) >> 1) & 1, abort_flag);
          if (ok && j + 1 == clean_j) ok = mbar_wait(BAR(K_CLEAN), 0, abort_flag);
          if (ok) ok = mbar_wait(BAR(V_FULL + (st ^ 1)), ((j + 1) >> 1) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
          issue_sdp(0, j + 1);  // over dS of half 0, which the MMAs just issued consume first
        }
        PJX_BTRACE(0, j, 2);
        ok = mbar_wait(BAR(DS_FULL + 1), j & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        issue_acc(1, j);
        mma_commit(BAR(K_EMPTY + st));
        if (next) {
          issue_sdp(1, j + 1);
          mma_commit(BAR(V_EMPTY + (st ^ 1)));
        }
        PJX_BTRACE(0, j, 3);
      }
      if (ok) mma_commit(BAR(DQ_FULL));
    }
  } else {
    // --------------------------------------------------------------- compute warps
    const int grp = (warp - 2) >> 2;  // which half of the score columns
    const int quarter = warp & 3;
    const int r_in = quarter * 32 + lane;
    const int row = q0 + r_in;
    const bool row_ok = row < p.Lq;
    const uint32_t lane_sel = static_cast<uint32_t>(quarter * 32) << 16;
    const float c1 = p.sm_scale * kLog2e;
    // padded per-row vectors: +inf / 0 for rows past Lq and +inf for rows without keys, so P = 0 there
    const int64_t at = ((int64_t)b * p.Hq + h) * p.Lq_pad + row;
    const float lse2 = p.lse2[at], delta = p.delta[at];
    const uint32_t s_addr = T_S + lane_sel + grp * 64, dp_addr = T_DP + lane_sel + grp * 64;
    bool ok = true;
    for (int j = 0; j < n; ++j) {
      if (r_in == 64 && grp == 0) PJX_BTRACE(1, j, 0);
      ok = mbar_wait(BAR(SP_FULL + grp), j & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      if (r_in == 64 && grp == 0) PJX_BTRACE(1, j, 1);
      const int k0 = (j_lo + j) * BN + grp * 64;  // first key of this group's columns
      const bool need_mask = (k0 + 64 > kv_len) || (k0 + 63 > q0 + p.band_hi) || (k0 < q0 + BM - 1 + p.band_lo);
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        float s[32], dp[32], d[32];
        tmem_ld32f(s_addr + c * 32, s);
        tmem_ld32f(dp_addr + c * 32, dp);
        tmem_wait_ld();
        if (r_in == 64 && grp == 0) PJX_BTRACE(1, j, 2 + 2 * c);
        ds_row_chunk<BF16>(s, dp, c1, -lse2, -delta, d);
        if (need_mask) {  // selects, not products: masked scores may be anything
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int key = k0 + c * 32 + i;
            const bool keep = key < kv_len && key <= row + p.band_hi && key >= row + p.band_lo;
            d[i] = keep ? d[i] : 0.f;
          }
        }
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) pk[i] = pack16<BF16>(d[2 * i], d[2 * i + 1]);
        // over columns of this group's half that were read already (chunk 0: 0-15, chunk 1: 16-31)
        tmem_st16(s_addr + c * 16, pk);
        if (r_in == 64 && grp == 0) PJX_BTRACE(1, j, 3 + 2 * c);
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(BAR(DS_FULL + grp));
      if (r_in == 64 && grp == 0) PJX_BTRACE(1, j, 6);
    }
    if (ok && q0 < p.Lq) {
      if (n > 0) {
        ok = mbar_wait(BAR(DQ_FULL), 0, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
      }
      if (ok) {
        tc_fence_after();
        // each group stores one half of the row's D columns
        unsigned char* dst = static_cast<unsigned char*>(p.dq) + ((((int64_t)b * p.Lq + row) * p.Hq + h) * D) * 2;
        store_row<D / 2, BF16>(T_DQ + lane_sel + grp * (D / 2), dst + grp * D, p.sm_scale, n > 0, row_ok);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    __syncwarp();
    tmem_dealloc(tmem, C::TMEM_COLS);
    if (lane == 0 && *abort_flag && p.status) atomicExch(p.status, (int)PJX_ERR_DEVICE_TIMEOUT);
  }
}

// ---------------------------------------------------------------------------------------------
// dK/dV kernel
// ---------------------------------------------------------------------------------------------
template <int D>
struct DkvCfg {
  static constexpr int SUB = D / 64;
  static constexpr int TILE = SUB * 128 * 128;
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = TILE;
  static constexpr int OFF_Q = 2 * TILE;            // 2 stages
  static constexpr int OFF_DO = 4 * TILE;           // 2 stages
  static constexpr int OFF_ROW = 6 * TILE;          // 2 stages x { float lse2[128]; float delta[128]; }
  static constexpr int OFF_BAR = OFF_ROW + 2 * 2 * BM * 4;
  // barriers: KV_FULL, QDO_FULL[2], QDO_EMPTY[2], SP_FULL[2], PDS_FULL[2], ACC_FULL
  static constexpr int N_BAR = 10;
  static constexpr int SMEM_BYTES = OFF_BAR + N_BAR * 8 + 16 + 1024;
  static constexpr int TMEM_COLS = 512;             // S^T 128 | dP^T 128 | dV D | dK D
  static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
  static_assert(2 * BM + 2 * D <= 512, "tensor memory has 512 columns");
};

template <int D, bool BF16>
__global__ void __launch_bounds__(NTHREADS, 1)
bwd_dkdv_sm100_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                      const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                      const BwdParams p, const int order_w) {
  using C = DkvCfg<D>;
  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar0 = sbase + C::OFF_BAR;
  auto BAR = [&](int i) { return bar0 + 8u * i; };
  const int KV_FULL = 0, QDO_FULL = 1, QDO_EMPTY = 3, SP_FULL = 5, PDS_FULL = 7, ACC_FULL = 9;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + C::OFF_BAR + C::N_BAR * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* row_s = reinterpret_cast<float*>(smem + C::OFF_ROW);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int kt, pair;  // the first key tiles are seen by the most queries under a causal band
  work_item(blockIdx.x, (p.Lkv + BN - 1) / BN, p.Hkv * p.B, order_w, kt, pair);
  const int hk = pair % p.Hkv, b = pair / p.Hkv;
  const int G = p.Hq / p.Hkv;
  const int k0 = kt * BN;

  int kv_len = p.Lkv;
  if (p.kv_lengths) kv_len = max(0, min(kv_len, p.kv_lengths[b]));
  // query tiles that see a key of this tile: rows in [first key - band_hi, last valid key - band_lo]
  const int q_begin = max(0, k0 - p.band_hi);
  const int q_end = min(p.Lq, min(k0 + BN, kv_len) - p.band_lo);
  const int t_lo = q_begin / BM;
  const int n_t = (k0 < kv_len && q_begin < q_end) ? (q_end + BM - 1) / BM - t_lo : 0;
  const int n = n_t * G;  // steps: query heads of the group outer, query tiles inner

  if (threadIdx.x == 0) {
    for (int i = 0; i < C::N_BAR; ++i)
      mbar_init(BAR(i), (i == PDS_FULL || i == PDS_FULL + 1) ? 128u : 1u);
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
  const uint32_t T_S = tmem, T_DP = tmem + BM, T_DV = tmem + 2 * BM, T_DK = tmem + 2 * BM + D;

  if (warp == 0) {
    // ------------------------------------------------------------------- TMA producer
    if (lane == 0 && n > 0) {
      prefetch_tmap(&tm_q);
      prefetch_tmap(&tm_do);
      prefetch_tmap(&tm_k);
      prefetch_tmap(&tm_v);
      mbar_arrive_expect_tx(BAR(KV_FULL), 2 * C::TILE);
#pragma unroll
      for (int s = 0; s < C::SUB; ++s) {
        tma_load_4d(sbase + C::OFF_K + s * BN * 128, &tm_k, BAR(KV_FULL), s * 64, hk, k0, b);
        tma_load_4d(sbase + C::OFF_V + s * BN * 128, &tm_v, BAR(KV_FULL), s * 64, hk, k0, b);
      }
      for (int it = 0; it < n; ++it) {
        const int st = it & 1;
        const int h = hk * G + it / n_t;
        const int q0 = (t_lo + it % n_t) * BM;
        if (!mbar_wait(BAR(QDO_EMPTY + st), ((it >> 1) & 1) ^ 1, abort_flag)) break;
        mbar_arrive_expect_tx(BAR(QDO_FULL + st), 2 * C::TILE + 2 * BM * 4);
#pragma unroll
        for (int s = 0; s < C::SUB; ++s) {
          tma_load_4d(sbase + C::OFF_Q + st * C::TILE + s * BM * 128, &tm_q, BAR(QDO_FULL + st), s * 64, h, q0, b);
          tma_load_4d(sbase + C::OFF_DO + st * C::TILE + s * BM * 128, &tm_do, BAR(QDO_FULL + st), s * 64, h, q0, b);
        }
        // the 128 query rows' log-sum-exp (base 2) and delta out of the padded workspace arrays
        const int64_t at = ((int64_t)b * p.Hq + h) * p.Lq_pad + q0;
        bulk_load(sbase + C::OFF_ROW + st * 2 * BM * 4, p.lse2 + at, BM * 4, BAR(QDO_FULL + st));
        bulk_load(sbase + C::OFF_ROW + st * 2 * BM * 4 + BM * 4, p.delta + at, BM * 4, BAR(QDO_FULL + st));
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && n > 0) {
      constexpr uint32_t idesc_s = make_idesc(BN, BM / 2, BF16, false, false);
      constexpr uint32_t idesc_acc = make_idesc(BN, D, BF16, false, true);
      const uint32_t ka = sbase + C::OFF_K, va = sbase + C::OFF_V;
      // S^T and dP^T of one half (64 query rows) of step `it`: keys on the lanes, query rows on
      // the columns; the B operands start 64 rows into the Q / dO tiles
      auto issue_sdp = [&](int half, int it) {
        const uint32_t qa = sbase + C::OFF_Q + (it & 1) * C::TILE + half * 64 * 128;
        const uint32_t doa = sbase + C::OFF_DO + (it & 1) * C::TILE + half * 64 * 128;
#pragma unroll
        for (int s = 0; s < C::SUB; ++s)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            mma_ss(T_S + half * 64, make_smem_desc(ka + s * BN * 128 + kk * 32, 16, 1024),
                   make_smem_desc(qa + s * BM * 128 + kk * 32, 16, 1024), idesc_s, (s | kk) != 0);
#pragma unroll
        for (int s = 0; s < C::SUB; ++s)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            mma_ss(T_DP + half * 64, make_smem_desc(va + s * BN * 128 + kk * 32, 16, 1024),
                   make_smem_desc(doa + s * BM * 128 + kk * 32, 16, 1024), idesc_s, (s | kk) != 0);
        mma_commit(BAR(SP_FULL + half));
      };
      // dV += P^T.dO and dK += dS^T.Q over one half: A from tensor memory (16-bit pairs at the
      // first 32 columns of the half), dO / Q tiles read MN-major
      auto issue_acc = [&](int half, int it) {
        const uint32_t qa = sbase + C::OFF_Q + (it & 1) * C::TILE, doa = sbase + C::OFF_DO + (it & 1) * C::TILE;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          mma_ts(T_DV, T_S + half * 64 + kk * 8, make_smem_desc(doa + (half * 4 + kk) * 2048, BM * 128, 1024), idesc_acc,
                 (it | half | kk) != 0);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          mma_ts(T_DK, T_DP + half * 64 + kk * 8, make_smem_desc(qa + (half * 4 + kk) * 2048, BM * 128, 1024), idesc_acc,
                 (it | half | kk) != 0);
      };
      bool ok = mbar_wait(BAR(KV_FULL), 0, abort_flag);
      if (ok) ok = mbar_wait(BAR(QDO_FULL), 0, abort_flag);
      if (ok) {
        tc_fence_after();
        issue_sdp(0, 0);
        issue_sdp(1, 0);
      }
      for (int it = 0; ok && it < n; ++it) {
        const int st = it & 1;
        const bool next = it + 1 < n;
        PJX_KTRACE(0, it, 0);
        ok = mbar_wait(BAR(PDS_FULL + 0), it & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        PJX_KTRACE(0, it, 1);
        issue_acc(0, it);
        if (next) {
          ok = mbar_wait(BAR(QDO_FULL + (st ^ 1)), ((it + 1) >> 1) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
          issue_sdp(0, it + 1);  // over P^T / dS^T of half 0, which the MMAs just issued consume first
        }
        PJX_KTRACE(0, it, 2);
        ok = mbar_wait(BAR(PDS_FULL + 1), it & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        issue_acc(1, it);
        mma_commit(BAR(QDO_EMPTY + st));
        if (next) issue_sdp(1, it + 1);
        PJX_KTRACE(0, it, 3);
      }
      if (ok) mma_commit(BAR(ACC_FULL));
    }
  } else {
    // --------------------------------------------------------------- compute warps
    const int grp = (warp - 2) >> 2;  // which half of the query columns
    const int quarter = warp & 3;
    const int r_in = quarter * 32 + lane;
    const int key = k0 + r_in;
    const bool key_ok = key < kv_len;
    const uint32_t lane_sel = static_cast<uint32_t>(quarter * 32) << 16;
    const float c1 = p.sm_scale * kLog2e;
    const float2 c2 = make_float2(c1, c1);
    const uint32_t s_addr = T_S + lane_sel + grp * 64, dp_addr = T_DP + lane_sel + grp * 64;
    bool ok = true;
    for (int it = 0; it < n; ++it) {
      const int st = it & 1;
      const int q0 = (t_lo + it % n_t) * BM + grp * 64;  // first query row of this group's columns
      if (r_in == 64 && grp == 0) PJX_KTRACE(1, it, 0);
      ok = mbar_wait(BAR(SP_FULL + grp), it & 1, abort_flag);
      if (r_in == 64 && grp == 0) PJX_KTRACE(1, it, 1);
      if (ok) ok = mbar_wait(BAR(QDO_FULL + st), (it >> 1) & 1, abort_flag);  // the row vectors landed with Q and dO
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      if (r_in == 64 && grp == 0) PJX_KTRACE(1, it, 2);
      const float* lse2_s = row_s + st * 2 * BM + grp * 64;
      const float* delta_s = lse2_s + BM;
      // this key row against query rows q0 .. q0+63: visible iff q + band_lo <= key <= q + band_hi
      const bool need_mask = !key_ok || (key > q0 + p.band_hi) || (key < q0 + 63 + p.band_lo);
#pragma unroll
      for (int c = 0; c < 2; ++c) {  // 32 query columns at a time
        float s[32], dp[32];
        tmem_ld32f(s_addr + c * 32, s);
        tmem_ld32f(dp_addr + c * 32, dp);
        tmem_wait_ld();
        float pr[32], ds[32];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float4 l4 = *reinterpret_cast<const float4*>(lse2_s + c * 32 + 4 * i);
          const float4 d4 = *reinterpret_cast<const float4*>(delta_s + c * 32 + 4 * i);
          const float2 x0 = __ffma2_rn(make_float2(s[4 * i], s[4 * i + 1]), c2, make_float2(-l4.x, -l4.y));
          const float2 x1 = __ffma2_rn(make_float2(s[4 * i + 2], s[4 * i + 3]), c2, make_float2(-l4.z, -l4.w));
          const float2 p0 = make_float2(ex2_approx(x0.x), ex2_approx(x0.y));
          const float2 p1 = make_float2(ex2_approx(x1.x), ex2_approx(x1.y));
          const float2 e0 = __fadd2_rn(make_float2(dp[4 * i], dp[4 * i + 1]), make_float2(-d4.x, -d4.y));
          const float2 e1 = __fadd2_rn(make_float2(dp[4 * i + 2], dp[4 * i + 3]), make_float2(-d4.z, -d4.w));
          const float2 g0 = __fmul2_rn(p0, e0), g1 = __fmul2_rn(p1, e1);
          pr[4 * i] = p0.x; pr[4 * i + 1] = p0.y; pr[4 * i + 2] = p1.x; pr[4 * i + 3] = p1.y;
          ds[4 * i] = g0.x; ds[4 * i + 1] = g0.y; ds[4 * i + 2] = g1.x; ds[4 * i + 3] = g1.y;
        }
        if (need_mask) {  // selects, not products: masked scores may be anything
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int qrow = q0 + c * 32 + i;
            const bool keep = key_ok && key <= qrow + p.band_hi && key >= qrow + p.band_lo;
            pr[i] = keep ? pr[i] : 0.f;
            ds[i] = keep ? ds[i] : 0.f;
          }
        }
        uint32_t pkp[16], pkd[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          pkp[i] = pack16<BF16>(pr[2 * i], pr[2 * i + 1]);
          pkd[i] = pack16<BF16>(ds[2 * i], ds[2 * i + 1]);
        }
        // over columns of this group's half that were read already (chunk 0: 0-15, chunk 1: 16-31)
        tmem_st16(s_addr + c * 16, pkp);
        tmem_st16(dp_addr + c * 16, pkd);
        if (r_in == 64 && grp == 0) PJX_KTRACE(1, it, 3 + c);
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(BAR(PDS_FULL + grp));
      if (r_in == 64 && grp == 0) PJX_KTRACE(1, it, 5);
    }
    if (ok && k0 < p.Lkv) {
      if (n > 0) {
        ok = mbar_wait(BAR(ACC_FULL), 0, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
      }
      if (ok) {
        tc_fence_after();
        const bool row_ok = key < p.Lkv;
        const int64_t at = (((int64_t)b * p.Lkv + key) * p.Hkv + hk) * D * 2;
        // group 0 stores the dV row, group 1 the dK row
        if (grp == 0) store_row<D, BF16>(T_DV + lane_sel, static_cast<unsigned char*>(p.dv) + at, 1.f, n > 0, row_ok);
        else store_row<D, BF16>(T_DK + lane_sel, static_cast<unsigned char*>(p.dk) + at, p.sm_scale, n > 0, row_ok);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    __syncwarp();
    tmem_dealloc(tmem, C::TMEM_COLS);
    if (lane == 0 && *abort_flag && p.status) atomicExch(p.status, (int)PJX_ERR_DEVICE_TIMEOUT);
  }
}

template <int D, bool BF16>
int launch_both(const BwdParams& p, cudaStream_t stream) {
  CUtensorMap tq, tdo, tk, tv;
  int rc;
  if ((rc = make_tmap_blhd(&tq, p.q, p.dtype, p.B, p.Lq, p.Hq, D, BM))) return rc;
  if ((rc = make_tmap_blhd(&tdo, p.d_o, p.dtype, p.B, p.Lq, p.Hq, D, BM))) return rc;
  if ((rc = make_tmap_blhd(&tk, p.k, p.dtype, p.B, p.Lkv, p.Hkv, D, BN))) return rc;
  if ((rc = make_tmap_blhd(&tv, p.v, p.dtype, p.B, p.Lkv, p.Hkv, D, BN))) return rc;
  auto kq = bwd_dq_sm100_kernel<D, BF16>;
  if ((rc = check_cuda(cudaFuncSetAttribute(kq, cudaFuncAttributeMaxDynamicSharedMemorySize, DqCfg<D>::SMEM_BYTES),
                       "cudaFuncSetAttribute(sm100 dq)")))
    return rc;
  // triangular work (an upper bound on the keys only): heavy-first order in blocks of 16 pairs
  const int order_w = (p.band_hi < PJX_BAND_NO_UPPER && p.band_lo == PJX_BAND_NO_LOWER) ? 16 : 1;
  const int64_t n_dq = (int64_t)((p.Lq + BM - 1) / BM) * p.Hq * p.B;
  kq<<<dim3((unsigned)n_dq), NTHREADS, DqCfg<D>::SMEM_BYTES, stream>>>(tq, tdo, tk, tv, p, order_w);
  count_launch();
  if ((rc = check_cuda(cudaGetLastError(), "sm100 dq launch"))) return rc;
  auto kk = bwd_dkdv_sm100_kernel<D, BF16>;
  if ((rc = check_cuda(cudaFuncSetAttribute(kk, cudaFuncAttributeMaxDynamicSharedMemorySize, DkvCfg<D>::SMEM_BYTES),
                       "cudaFuncSetAttribute(sm100 dk/dv)")))
    return rc;
  const int64_t n_dkv = (int64_t)((p.Lkv + BN - 1) / BN) * p.Hkv * p.B;
  kk<<<dim3((unsigned)n_dkv), NTHREADS, DkvCfg<D>::SMEM_BYTES, stream>>>(tq, tdo, tk, tv, p, order_w);
  count_launch();
  return check_cuda(cudaGetLastError(), "sm100 dk/dv launch");
}

}  // namespace

bool bwd_sm100_supported(const BwdParams& p, const char** why) {
  const char* w = nullptr;
  if (p.dtype != PJX_BF16 && p.dtype != PJX_F16) w = "dtype must be bf16 or fp16";
  else if (!(p.D == p.Dv && (p.D == 64 || p.D == 128))) w = "head dims must be (64,64) or (128,128)";
  else if (p.bias) w = "a dense bias is taken by the CUDA-core kernels only";
  else if (p.B < 1 || p.Lq < 1 || p.Lkv < 1) w = "empty problem";
  else if ((int64_t)((p.Lq + BM - 1) / BM) * p.Hq * p.B > 0x7fffffffLL ||
           (int64_t)((p.Lkv + BN - 1) / BN) * p.Hkv * p.B > 0x7fffffffLL)
    w = "grid too large";
  else if ((reinterpret_cast<uintptr_t>(p.q) | reinterpret_cast<uintptr_t>(p.k) | reinterpret_cast<uintptr_t>(p.v) |
            reinterpret_cast<uintptr_t>(p.d_o) | reinterpret_cast<uintptr_t>(p.dq) | reinterpret_cast<uintptr_t>(p.dk) |
            reinterpret_cast<uintptr_t>(p.dv)) & 15)
    w = "q, k, v, d_o, dq, dk, dv must be 16-byte aligned";
  else if (reinterpret_cast<uintptr_t>(p.delta) & 15) w = "the workspace must be 16-byte aligned";
  if (why) *why = w;
  return w == nullptr;
}

#ifdef PJX_TRACE
extern "C" int pjx_debug_read_bwd_trace(long long* host_out) {
  return (int)cudaMemcpyFromSymbol(host_out, g_btrace, sizeof(long long) * 4 * 64 * 8);
}
#endif

int launch_bwd_sm100(const BwdParams& p, cudaStream_t stream) {
  const char* why = nullptr;
  if (!bwd_sm100_supported(p, &why)) return fail(PJX_ERR_UNSUPPORTED, "tcgen05 backward: %s", why);
  const bool bf16 = p.dtype == PJX_BF16;
  if (p.D == 128) return bf16 ? launch_both<128, true>(p, stream) : launch_both<128, false>(p, stream);
  return bf16 ? launch_both<64, true>(p, stream) : launch_both<64, false>(p, stream);
}

}  // namespace pjx
