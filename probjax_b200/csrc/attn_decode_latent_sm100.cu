// Split-KV decode over a latent cache on the tcgen05 tensor cores (absorbed latent attention,
// K = V = C; probjax/nn/pallas_kernels/kernels/latent_attention.py:604-607, 204-244).
//
// The mma.sync kernel of attn_decode_latent.cu is bound by the legacy tensor path (its 576 tensor
// steps per 64 keys keep that pipe busy ~80 % of the time at 3.8 TB/s).  Here both products run as
// tcgen05 MMAs with the KEYS on the M axis, so that 16 query rows cost an N = 16 instruction
// instead of a padded M:
//
//   S^T [128 keys x 16 rows]  = C_tile [128 x R] . Q^T [R x 16]         (A, B K-major in shared memory)
//   O^T [R x 16 rows]        += C_tile^T [R x 128 keys] . P^T [128 x 16]  (A = the same tile, MN-major)
//
// The latent tile [128 keys x R] comes in by TMA as R / 64 sub-tiles [128 keys x 64 columns] (128-byte
// swizzle), TWICE: once from HBM into the score ring (4 slots; a slot is free again as soon as its four
// score MMAs have run, so this stream never waits for a softmax), and a few microseconds later, as
// pairs of sub-tiles = the A operand of one 128-column output block, from L2 into the output ring.
// Keeping a tile resident from its first use to its second would leave room for three sub-tiles in
// flight, which is what bounded the first version of this kernel at 3.0 TB/s; HBM still sees every
// byte once.
//
//   warp 0      TMA producer of the score ring (one lane)
//   warp 6      TMA producer of the output ring (one lane); the whole warp clears the rows past the valid
//               length in the pairs of a split's last tile (0 x NaN is not 0 inside the second product)
//   warp 1      MMA issuer of the scores (one lane): S^T(0), S^T(1), then S^T(t+2) once P(t) has been written
//               (the softmax has then read S^T[t % 2])
//   warp 7      MMA issuer of the output (one lane): the pairs of P(t).C(t).  Two issuers, because an N = 16
//               MMA takes 32 cycles and one thread cannot issue them that fast, and because either ring
//               would otherwise wait for the other's data
//   warps 2-5   softmax: one thread per key (= tensor-memory lane).  The maximum over the keys of a
//               tile is a reduction ACROSS threads: a 16-value butterfly per warp (16 shuffles), then
//               shared memory across the four warps.  P^T goes to shared memory as the B operand.  The
//               running maximum only advances when it grew by more than 8 (base 2), so O^T is rarely
//               rescaled, and then only after the previous tile's second product has completed.
//
// Tensor memory: two S^T buffers of 16 columns, O^T ceil(R / 128) blocks of 16 columns.  S^T, P^T and
// the reduction scratch are double-buffered, so the softmax of tile t + 1 overlaps the second product
// of tile t.  The partials have the layout of the other decode kernels (O normalised by its own sum,
// base-2 LSE), so the same combine finishes the job.  Every wait is bounded; on expiry the status word
// gets PJX_ERR_DEVICE_TIMEOUT.
#include <type_traits>

#include "pjx_common.cuh"
#include "sm100_ptx.cuh"

namespace pjx {

// gemm_sm100.cu: row-major [rows, cols] 16-bit matrix, box = 64 columns x box_rows rows, 128-byte swizzle
int make_tmap_2d(CUtensorMap* m, const void* base, int dtype, int64_t rows, int64_t cols, int box_rows, int64_t pitch);

namespace {

using namespace sm100;

constexpr int TK = 128;              // keys per tile (= tensor-memory lanes)
constexpr int SUB_BYTES = TK * 128;  // one sub-tile: 128 keys x 64 columns of 16 bits
#ifndef PJX_LD_NQ
#define PJX_LD_NQ 4
#define PJX_LD_NP 4
#endif
constexpr int NQ = PJX_LD_NQ;        // slots of the score ring (one sub-tile each)
constexpr int NP = PJX_LD_NP;        // slots of the output ring (a pair of sub-tiles each)
constexpr int NROW = 16;             // query rows per CTA (the N of both products)
constexpr int TC_THREADS = 256;      // producers (warps 0, 6), MMA issuers (warps 1, 7), softmax (warps 2-5)

template <int R>
struct TCfg {
  static constexpr int NSUB = R / 64;
  static constexpr int NBLK = (NSUB + 1) / 2;          // output blocks of 128 latent columns
  static constexpr int OFF_QRING = 0;
  static constexpr int OFF_PRING = NQ * SUB_BYTES;
  static constexpr int OFF_Q = OFF_PRING + NP * 2 * SUB_BYTES;  // [NSUB][16 rows][128 B], swizzled
  static constexpr int OFF_P = OFF_Q + NSUB * 2048;    // 2 x [2 key blocks][16 rows][128 B], swizzled
  static constexpr int OFF_RED = OFF_P + 2 * 4096;     // 2 x [4 warps][16] floats
  static constexpr int OFF_BAR = OFF_RED + 2 * 4 * 16 * 4;
  static constexpr int N_BAR = 2 * NQ + 3 * NP + 7;
  static constexpr int SMEM = OFF_BAR + N_BAR * 8 + 16 + 1024;  // + alignment slack
  static constexpr int TMEM_COLS = 128;
  static constexpr int O_COL = 32;
  static_assert(R % 64 == 0 && NSUB >= 2 && NSUB <= 9, "latent width: a multiple of 64 in 128 .. 576");
  static_assert(O_COL + NBLK * 16 <= TMEM_COLS, "tensor memory columns");
  static_assert(SMEM <= 227 * 1024, "shared memory budget");
};

__device__ __forceinline__ void tmem_ld16f(uint32_t taddr, float* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
      : "=f"(r[0]), "=f"(r[1]), "=f"(r[2]), "=f"(r[3]), "=f"(r[4]), "=f"(r[5]), "=f"(r[6]), "=f"(r[7]), "=f"(r[8]),
        "=f"(r[9]), "=f"(r[10]), "=f"(r[11]), "=f"(r[12]), "=f"(r[13]), "=f"(r[14]), "=f"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st16f(uint32_t taddr, const float* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n" ::"r"(taddr),
      "f"(r[0]), "f"(r[1]), "f"(r[2]), "f"(r[3]), "f"(r[4]), "f"(r[5]), "f"(r[6]), "f"(r[7]), "f"(r[8]), "f"(r[9]),
      "f"(r[10]), "f"(r[11]), "f"(r[12]), "f"(r[13]), "f"(r[14]), "f"(r[15])
      : "memory");
}

// Reduction of 16 per-thread values over the 32 lanes of a warp in 16 shuffles: every step halves
// the values a lane still carries and doubles the lanes folded into each.  Afterwards lane l holds
// the result of value index ((l >> 4) & 1) * 8 + ((l >> 3) & 1) * 4 + ((l >> 2) & 1) * 2 + ((l >> 1) & 1).
template <bool MAX>
__device__ __forceinline__ float warp_reduce16(const float (&x)[16], int lane) {
  auto op = [](float a, float b) { return MAX ? fmaxf(a, b) : a + b; };
  float v8[8], v4[4], v2[2], v1;
  const bool b16 = lane & 16, b8 = lane & 8, b4 = lane & 4, b2 = lane & 2;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float send = b16 ? x[j] : x[j + 8];
    const float recv = __shfl_xor_sync(0xffffffffu, send, 16);
    v8[j] = op(b16 ? x[j + 8] : x[j], recv);
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float send = b8 ? v8[j] : v8[j + 4];
    const float recv = __shfl_xor_sync(0xffffffffu, send, 8);
    v4[j] = op(b8 ? v8[j + 4] : v8[j], recv);
  }
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const float send = b4 ? v4[j] : v4[j + 2];
    const float recv = __shfl_xor_sync(0xffffffffu, send, 4);
    v2[j] = op(b4 ? v4[j + 2] : v4[j], recv);
  }
  {
    const float send = b2 ? v2[0] : v2[1];
    const float recv = __shfl_xor_sync(0xffffffffu, send, 2);
    v1 = op(b2 ? v2[1] : v2[0], recv);
  }
  return op(v1, __shfl_xor_sync(0xffffffffu, v1, 1));
}
__device__ __forceinline__ int reduce16_index(int lane) {
  return ((lane >> 4) & 1) * 8 + ((lane >> 3) & 1) * 4 + ((lane >> 2) & 1) * 2 + ((lane >> 1) & 1);
}

template <bool BF16, int R>
__global__ void __launch_bounds__(TC_THREADS, 1)
decode_latent_tc_kernel(const __grid_constant__ CUtensorMap tm_c, const DecodeParams p) {
  using C = TCfg<R>;
  using T = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
  constexpr int NSUB = C::NSUB, NBLK = C::NBLK;
  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar0 = sbase + C::OFF_BAR;
  auto BAR = [&](int i) { return bar0 + 8u * i; };
  // barrier indices
  const int QF = 0;                    // [NQ] score-ring slot filled
  const int QE = NQ;                   // [NQ] ... consumed
  const int PF = 2 * NQ;               // [NP] output-ring slot filled
  const int PE = 2 * NQ + NP;          // [NP] ... consumed
  const int S_FULL = 2 * NQ + 2 * NP;  // [2]
  const int P_FULL = S_FULL + 2;       // [2] 128 arrivals
  // [2] second product of tile t complete, on barrier t % 2.  Two barriers, as for S and P: a thread that
  // waits for tile t may be two tiles ahead of the issuer, and a parity wait on a single barrier cannot
  // tell "two phases behind" from "done".
  const int PV_DONE = P_FULL + 2;
  const int CLEAN = PV_DONE + 2;       // [NP] rows past the valid length cleared in the slot's pair (32 arrivals);
                                       // per slot, so that it cannot complete twice before the issuer looks
  const int RED = CLEAN + NP;          // rendezvous of the softmax threads (128 arrivals, one phase per tile)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + C::OFF_BAR + C::N_BAR * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* red = reinterpret_cast<float*>(smem + C::OFF_RED);

  const int split = blockIdx.x, grp = blockIdx.y;
  const DecodeSeq sq = decode_seq(p, blockIdx.z);
  const int b = sq.cache_b, len = sq.len;
  const int start = split * p.split_len;
  if (start >= len) return;  // the combine never reads this split
  const int end = min(len, start + p.split_len);
  // the combine of the splits, next on the stream, may become resident as SM slots free up (it waits
  // for this grid before it reads a partial)
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  const int n_tiles = (end - start + TK - 1) / TK;
  const int last_rows = end - start - (n_tiles - 1) * TK;  // valid rows of the last tile, 1 .. 128
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = p.Hq / p.Hkv;  // heads per row group

  if (tid == 0) {
    for (int i = 0; i < C::N_BAR; ++i)
      mbar_init(BAR(i), (i == P_FULL || i == P_FULL + 1 || i == RED) ? 128u : ((i >= CLEAN && i < CLEAN + NP) ? 32u : 1u));
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(tmem_slot), C::TMEM_COLS);
    tmem_relinquish();
  }
  // query rows of the group into the B-operand layout: packed row r = g * Lq + t, head grp * G + g;
  // rows past p.rows are zero.  Sub-block s = 64 columns: [16 rows][128 B], 16-byte chunks XOR-swizzled.
  {
    const T* q = static_cast<const T*>(p.q);
    for (int idx = tid; idx < NROW * (R / 8); idx += TC_THREADS) {
      const int r = idx / (R / 8), c = idx % (R / 8);
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (r < p.rows) {
        const int g = r / p.Lq, t = r % p.Lq;
        v = *reinterpret_cast<const uint4*>(q + ((sq.q_b * p.Lq + t) * p.Hq + grp * G + g) * R + c * 8);
      }
      const int sub = c >> 3, ch = c & 7;
      *reinterpret_cast<uint4*>(smem + C::OFF_Q + sub * 2048 + r * 128 + ((ch ^ (r & 7)) << 4)) = v;
    }
    fence_proxy_async();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const int row0 = (int)((int64_t)b * p.capacity + start);  // row of the 2-D view [B * capacity, R]

  if (warp == 0) {
    // -------------------------------------------- TMA producer, score ring (HBM)
    if (lane == 0) {
      prefetch_tmap(&tm_c);
      bool ok = true;
      for (int t = 0, n = 0; t < n_tiles && ok; ++t) {
        for (int i = 0; i < NSUB; ++i, ++n) {
          const int s = n % NQ;
          ok = mbar_wait(BAR(QE + s), ((n / NQ) & 1) ^ 1, abort_flag);
          if (!ok) break;
          mbar_arrive_expect_tx(BAR(QF + s), SUB_BYTES);
          tma_load_2d(sbase + C::OFF_QRING + s * SUB_BYTES, &tm_c, BAR(QF + s), i * 64, row0 + t * TK);
        }
      }
    }
  } else if (warp == 6) {
    // ------------------------------------------- TMA producer, output ring (L2)
    bool ok = true;
    for (int t = 0, n = 0; t < n_tiles && ok; ++t) {
      const bool dirty = (t == n_tiles - 1) && last_rows < TK;
      for (int m = 0; m < NBLK; ++m, ++n) {
        const int s = n % NP;
        const uint32_t dst = sbase + C::OFF_PRING + s * 2 * SUB_BYTES;
        const bool two = 2 * m + 1 < NSUB;
        if (lane == 0) {
          ok = mbar_wait(BAR(PE + s), ((n / NP) & 1) ^ 1, abort_flag);
          if (ok) {
            mbar_arrive_expect_tx(BAR(PF + s), two ? 2 * SUB_BYTES : SUB_BYTES);
            tma_load_2d(dst, &tm_c, BAR(PF + s), 2 * m * 64, row0 + t * TK);
            if (two) tma_load_2d(dst + SUB_BYTES, &tm_c, BAR(PF + s), (2 * m + 1) * 64, row0 + t * TK);
          }
        }
        ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
        if (!ok) break;
        if (dirty) {  // wait for the pair, clear its rows past the valid length, tell the issuer
          ok = mbar_wait(BAR(PF + s), (n / NP) & 1, abort_flag);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          unsigned char* base = smem + C::OFF_PRING + s * 2 * SUB_BYTES;
          const int per_half = (TK - last_rows) * 8;  // 16-byte units to clear in one sub-tile
          for (int idx = lane; idx < per_half * (two ? 2 : 1); idx += 32) {
            const int half = idx / per_half, rem = idx % per_half;
            *reinterpret_cast<uint4*>(base + half * SUB_BYTES + (last_rows + rem / 8) * 128 + (rem % 8) * 16) =
                make_uint4(0u, 0u, 0u, 0u);
          }
          fence_proxy_async();
          mbar_arrive(BAR(CLEAN + s));
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------ MMA issuer, scores
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc(TK, NROW, BF16, false, false);
      // descriptors differ only in the address field (bits 0-13, address >> 4): add to a base.  The address is
      // masked to the 18 bits of the field (bits above them would spill into the leading-offset field)
      const uint64_t kdesc = make_smem_desc(0, 16, 1024);
      const uint32_t ring16 = ((sbase + C::OFF_QRING) & 0x3FFFF) >> 4, q16 = ((sbase + C::OFF_Q) & 0x3FFFF) >> 4;
      bool ok = true;
      for (int t = 0, n = 0; t < n_tiles && ok; ++t) {
        if (t >= 2) {  // S^T[t % 2] is free once every softmax thread has written P(t - 2)
          ok = mbar_wait(BAR(P_FULL + (t & 1)), ((t - 2) >> 1) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
        }
        for (int i = 0; i < NSUB; ++i, ++n) {
          const int s = n % NQ;
          ok = mbar_wait(BAR(QF + s), (n / NQ) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
          const uint64_t ca = kdesc + (ring16 + s * (SUB_BYTES >> 4)), qa = kdesc + (q16 + i * (2048 >> 4));
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) mma_ss(tmem + (t & 1) * 16, ca + kk * 2, qa + kk * 2, idesc_s, (i | kk) != 0);
          mma_commit(BAR(QE + s));  // the slot is free again after its four MMAs
        }
        if (ok) mma_commit(BAR(S_FULL + (t & 1)));
      }
    }
  } else if (warp == 7) {
    // ------------------------------------------------------ MMA issuer, output
    if (lane == 0) {
      constexpr uint32_t idesc_o = make_idesc(128, NROW, BF16, true, false);
      const uint64_t adesc = make_smem_desc(0, SUB_BYTES, 1024), bdesc = make_smem_desc(0, 16, 1024);
      const uint32_t ring16 = ((sbase + C::OFF_PRING) & 0x3FFFF) >> 4, p16 = ((sbase + C::OFF_P) & 0x3FFFF) >> 4;
      bool ok = true;
      for (int t = 0, n = 0; t < n_tiles && ok; ++t) {
        ok = mbar_wait(BAR(P_FULL + (t & 1)), (t >> 1) & 1, abort_flag);
        if (!ok) break;
        const bool dirty = (t == n_tiles - 1) && last_rows < TK;
        const uint64_t pa = bdesc + (p16 + (t & 1) * (4096 >> 4));
        // O^T block m += C(t)^T [128 latent columns x 128 keys] . P^T
        for (int m = 0; m < NBLK; ++m, ++n) {
          const int s = n % NP;
          ok = mbar_wait(BAR(PF + s), (n / NP) & 1, abort_flag);
          if (ok && dirty) ok = mbar_wait(BAR(CLEAN + s), (m / NP) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
          const uint64_t ca = adesc + (ring16 + s * (2 * SUB_BYTES >> 4));
#pragma unroll
          for (int kk = 0; kk < TK / 16; ++kk)
            mma_ss(tmem + C::O_COL + m * 16, ca + kk * (2048 >> 4), pa + (kk >> 2) * (2048 >> 4) + (kk & 3) * 2, idesc_o,
                   (t | kk) != 0);
          mma_commit(BAR(PE + s));
        }
        if (ok) mma_commit(BAR(PV_DONE + (t & 1)));
      }
    }
  } else {
    // ------------------------------------------------------------ softmax warps
    const int quarter = warp & 3;           // tensor-memory lane quarter this warp may access
    const int kl = quarter * 32 + lane;     // key within the tile = tensor-memory lane
    const uint32_t lane_sel = static_cast<uint32_t>(quarter * 32) << 16;
    const float c1 = p.sm_scale * kLog2e;
    const int widx = warp - 2;              // 0 .. 3: row of `red`
    const int my_h = reduce16_index(lane);
    float m_run[NROW], l_part[NROW];
#pragma unroll
    for (int h = 0; h < NROW; ++h) {
      m_run[h] = -INFINITY;
      l_part[h] = 0.f;
    }
    bool ok = true;
    for (int t = 0; t < n_tiles; ++t) {
      const int buf = t & 1;
      ok = mbar_wait(BAR(S_FULL + buf), (t >> 1) & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      float x[NROW];
      tmem_ld16f(tmem + lane_sel + buf * 16, x);
      tmem_wait_ld();
      const bool valid = start + t * TK + kl < end;
#pragma unroll
      for (int h = 0; h < NROW; ++h) x[h] = valid ? x[h] * c1 : -INFINITY;
      // tile maximum of every row over the 128 keys
      float* rd = red + buf * 64;
      const float wmax = warp_reduce16<true>(x, lane);
      if ((lane & 1) == 0) rd[widx * 16 + my_h] = wmax;
      mbar_arrive(BAR(RED));  // bounded rendezvous of the 128 softmax threads (release / acquire on the barrier)
      ok = mbar_wait(BAR(RED), t & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      // lazy running maximum: advance only when some row grew by more than 8 (base 2); the same in every thread
      float tmx[NROW];
      bool need = false;
#pragma unroll
      for (int h = 0; h < NROW; ++h) {
        tmx[h] = fmaxf(fmaxf(rd[h], rd[16 + h]), fmaxf(rd[32 + h], rd[48 + h]));
        need = need || (tmx[h] > m_run[h] + 8.f) || (m_run[h] == -INFINITY && tmx[h] > -INFINITY);
      }
      if (need) {
        float corr[NROW];
#pragma unroll
        for (int h = 0; h < NROW; ++h) {
          const float mn = fmaxf(m_run[h], tmx[h]);
          corr[h] = (mn == -INFINITY) ? 1.f : exp2f(m_run[h] - mn);
          m_run[h] = mn;
          l_part[h] *= corr[h];
        }
        if (t > 0) {  // O^T holds tiles 0 .. t-1 once the previous second product has completed
          ok = mbar_wait(BAR(PV_DONE + ((t - 1) & 1)), ((t - 1) >> 1) & 1, abort_flag);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int m = 0; m < NBLK; ++m) {
            float o[NROW];
            tmem_ld16f(tmem + lane_sel + C::O_COL + m * 16, o);
            tmem_wait_ld();
#pragma unroll
            for (int h = 0; h < NROW; ++h) o[h] *= corr[h];
            tmem_st16f(tmem + lane_sel + C::O_COL + m * 16, o);
          }
          tmem_wait_st();
        }
      }
      // probabilities (rounded to the input dtype) into the B operand P^T[buf] [16 rows][128 keys], once the
      // second product of tile t - 2, which read this buffer, has completed
      if (t >= 2) {
        ok = mbar_wait(BAR(PV_DONE + buf), ((t - 2) >> 1) & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      {
        const int blk = kl >> 6, kin = kl & 63;
        unsigned char* prow = smem + C::OFF_P + buf * 4096 + blk * 2048 + (kin & 7) * 2;
#pragma unroll
        for (int h = 0; h < NROW; ++h) {
          const float mu = (m_run[h] == -INFINITY) ? 0.f : m_run[h];
          const float pv = exp2f(x[h] - mu);
          l_part[h] += pv;
          *reinterpret_cast<T*>(prow + h * 128 + (((kin >> 3) ^ (h & 7)) << 4)) = Elem<T>::from_f(pv);
        }
      }
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(BAR(P_FULL + buf));
    }

    if (ok) {
      ok = mbar_wait(BAR(PV_DONE + ((n_tiles - 1) & 1)), ((n_tiles - 1) >> 1) & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      // row sums over the 128 key lanes
      float* rd = red + (n_tiles & 1) * 64;
      const float wsum = warp_reduce16<false>(l_part, lane);
      if ((lane & 1) == 0) rd[widx * 16 + my_h] = wsum;
      mbar_arrive(BAR(RED));
      ok = mbar_wait(BAR(RED), n_tiles & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        float inv[NROW];
        float lsum_mine = 0.f;
#pragma unroll
        for (int h = 0; h < NROW; ++h) {
          const float ls = (rd[h] + rd[16 + h]) + (rd[32 + h] + rd[48 + h]);
          inv[h] = ls > 0.f ? 1.f / ls : 0.f;
          if (h == kl) lsum_mine = ls;
        }
        const int64_t part = (((int64_t)blockIdx.z * p.Hkv + grp) * p.num_splits + split) * p.rows;
#pragma unroll
        for (int m = 0; m < NBLK; ++m) {
          float o[NROW];
          tmem_ld16f(tmem + lane_sel + C::O_COL + m * 16, o);
          tmem_wait_ld();
          const int col = m * 128 + kl;  // this thread's latent column
          if (col < R) {
#pragma unroll
            for (int h = 0; h < NROW; ++h)
              if (h < p.rows) p.o_part[(part + h) * R + col] = o[h] * inv[h];
          }
        }
        if (kl < p.rows) {
          float mk = -INFINITY;
#pragma unroll
          for (int h = 0; h < NROW; ++h)
            if (h == kl) mk = m_run[h];
          p.lse_part[part + kl] = lsum_mine > 0.f ? mk + log2f(lsum_mine) : -INFINITY;
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, C::TMEM_COLS);
  if (tid == 0 && *abort_flag && p.status) atomicExch(p.status, PJX_ERR_DEVICE_TIMEOUT);
}

template <bool BF16, int R>
int launch_tc_t(const DecodeParams& p, int dtype, cudaStream_t stream) {
  using C = TCfg<R>;
  CUtensorMap tm;
  int rc = make_tmap_2d(&tm, p.k, dtype, decode_cache_rows(p) * p.capacity, R, TK, 0);
  if (rc) return rc;
  auto kern = decode_latent_tc_kernel<BF16, R>;
  rc = check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM),
                  "cudaFuncSetAttribute(latent decode, tcgen05)");
  if (rc) return rc;
  kern<<<dim3(p.num_splits, p.Hkv, p.B), TC_THREADS, C::SMEM, stream>>>(tm, p);
  count_launch();
  return check_cuda(cudaGetLastError(), "latent decode (tcgen05) launch");
}

template <bool BF16>
int launch_tc_r(const DecodeParams& p, int dtype, cudaStream_t stream) {
  switch (p.D) {
    case 128: return launch_tc_t<BF16, 128>(p, dtype, stream);
    case 256: return launch_tc_t<BF16, 256>(p, dtype, stream);
    case 512: return launch_tc_t<BF16, 512>(p, dtype, stream);
    case 576: return launch_tc_t<BF16, 576>(p, dtype, stream);
  }
  return fail(PJX_ERR_UNSUPPORTED, "latent decode (tcgen05): latent width %d is not built", p.D);
}

}  // namespace

// The tcgen05 kernel takes the same cases as the mma.sync one; it needs a status word for its
// bounded waits and a cache whose 2-D view [B * capacity, R] a tensor map can address.
bool decode_latent_tc_supported(const DecodeParams& p, int dtype) {
  return (dtype == PJX_BF16 || dtype == PJX_F16) && (p.D == 128 || p.D == 256 || p.D == 512 || p.D == 576) &&
         p.status != nullptr && p.rows <= NROW && decode_cache_rows(p) * p.capacity < (1LL << 31) &&
         (reinterpret_cast<uintptr_t>(p.k) & 15) == 0;
}

int launch_decode_latent_tc_splits(const DecodeParams& p, int dtype, cudaStream_t stream) {
  return dtype == PJX_BF16 ? launch_tc_r<true>(p, dtype, stream) : launch_tc_r<false>(p, dtype, stream);
}

}  // namespace pjx
