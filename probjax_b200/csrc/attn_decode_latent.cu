// Split-KV decode over a latent cache: absorbed latent attention, K = V = C.
//
// The decode-time form of latent attention reads one shared latent row per key,
// `cache [B, S, R]`, for all heads: the scores contract the query against the latent and the
// output is a weighted sum of the same latent rows (probjax/nn/pallas_kernels/kernels/
// latent_attention.py:604-607, the `mla_fwd_absorbed` primitive 204-244).  Each latent tile is
// therefore loaded once and used for both products, half the traffic of a decode that streams K
// and V, and R is large (512 + 64 rotary columns), which the head widths of the regular kernels
// do not cover.
//
// Grid (split, row group, batch).  The query rows of a sequence (heads x query tokens) are packed
// 16 to a group, the row count of one m16n8k16 operand, as in the GQA decode kernel.  A CTA of
// eight warps streams its split of the cache through a cp.async ring of 64-key tiles [64, R]
// (16-byte copies, XOR-swizzled 128-byte lines).  Per tile:
//   1. warp w forms the scores of keys 8w .. 8w+7 against all 16 rows (R / 16 tensor-core steps,
//      query fragments read from shared memory);
//   2. the row maxima are exchanged through shared memory, every warp rescales its accumulator,
//      and the probabilities (rounded to the input dtype) go to shared memory as the A operand of
//      the second product;
//   3. warp w accumulates output columns w R/8 .. (w+1) R/8 over the 64 keys of the tile, reading
//      the latent rows of the same tile transposed (ldmatrix.trans).
// The partial (O normalised by its own sum, base-2 LSE) has the layout of the GQA decode
// kernel's partials, so the same combine kernel finishes the job.
#include "mma_sync.cuh"
#include "pjx_common.cuh"

namespace pjx {
namespace {

using namespace mma_sync;

constexpr int LBK = 64;      // keys per tile
constexpr int LWARPS = 8;
constexpr int LTHR = LWARPS * 32;

// byte offset of 16-byte chunk c of row r in a tile with rows of `row_bytes` (a multiple of 128)
__device__ __forceinline__ uint32_t lswz(int r, int c, int row_bytes) {
  return static_cast<uint32_t>(r * row_bytes + (((c & ~7) | ((c ^ r) & 7)) << 4));
}

template <int R>
struct LCfg {
  static constexpr int ROW_BYTES = R * 2;
  static constexpr int TILE_BYTES = LBK * ROW_BYTES;
  static constexpr int NSTAGE = (3 * TILE_BYTES + 16 * ROW_BYTES + 4096 <= 220 * 1024) ? 3 : 2;
  static constexpr int OFF_Q = NSTAGE * TILE_BYTES;          // [16][R] query rows
  static constexpr int OFF_P = OFF_Q + 16 * ROW_BYTES;       // [16][64] probabilities (128-byte rows)
  static constexpr int OFF_RED = OFF_P + 16 * 128;           // [8 warps][16] row maxima, then [8][16] row sums
  static constexpr int SMEM = OFF_RED + 2 * LWARPS * 16 * 4;
  static constexpr int NT = R / 64;                          // output n-tiles (8 columns) per warp
  static_assert(R % 64 == 0 && R <= 576, "latent width: a multiple of 64, at most 576");
  static_assert(SMEM <= 227 * 1024, "shared memory budget");
};

template <typename T, int R>
__global__ void __launch_bounds__(LTHR, 1) decode_latent_kernel(const DecodeParams p) {
  using C = LCfg<R>;
  constexpr int CH = R / 8;  // 16-byte chunks per row
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const uint32_t sbase = smem_u32(smem_raw);
  float* red = reinterpret_cast<float*>(smem_raw + C::OFF_RED);

  const int split = blockIdx.x, grp = blockIdx.y;
  const DecodeSeq sq = decode_seq(p, blockIdx.z);
  const int b = sq.cache_b, len = sq.len;
  const int start = split * p.split_len;
  if (start >= len) return;  // the combine never reads this split
  const int end = min(len, start + p.split_len);
  // the combine of the splits, next on the stream, may become resident as SM slots free up (it waits
  // for this grid before it reads a partial)
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  const int n_tiles = (end - start + LBK - 1) / LBK;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = p.Hq / p.Hkv;  // heads per row group
  const T* cbase = static_cast<const T*>(p.k) + (int64_t)b * p.capacity * R;

  auto load_tile = [&](int t) {
    const uint32_t dst = sbase + (t % C::NSTAGE) * C::TILE_BYTES;
    const int key0 = start + t * LBK;
    // warp w copies rows 8w .. 8w+7, lanes take the 16-byte chunks lane, lane + 32, ... of a row: no
    // division, and the swizzle term (r & 7) is the unrolled loop index
    static_assert(LBK == 8 * LWARPS, "one warp per eight rows of a tile");
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int r = warp * 8 + i;
      const bool ok = key0 + r < end;  // rows past the valid length are zero-filled, never read
      const T* src = cbase + (int64_t)(key0 + (ok ? r : 0)) * R + lane * 8;
      const uint32_t drow = dst + r * C::ROW_BYTES;
#pragma unroll
      for (int c0 = 0; c0 < CH; c0 += 32) {
        const int c = c0 + lane;
        if (c0 + 32 <= CH || c < CH)
          cp_async16(drow + (((c & ~7) | ((c ^ i) & 7)) << 4), src + c0 * 8, ok ? 16 : 0);
      }
    }
  };
#pragma unroll
  for (int s = 0; s < C::NSTAGE - 1; ++s) {
    if (s < n_tiles) load_tile(s);
    cp_async_commit();
  }

  // query rows of the group: packed row r = g * Lq + t, head grp * G + g (rows past p.rows are zero)
  {
    const T* q = static_cast<const T*>(p.q);
    for (int idx = tid; idx < 16 * CH; idx += LTHR) {
      const int r = idx / CH, c = idx % CH;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (r < p.rows) {
        const int g = r / p.Lq, t = r % p.Lq;
        v = *reinterpret_cast<const uint4*>(q + ((sq.q_b * p.Lq + t) * p.Hq + grp * G + g) * R + c * 8);
      }
      *reinterpret_cast<uint4*>(smem_raw + C::OFF_Q + lswz(r, c, C::ROW_BYTES)) = v;
    }
  }

  const float c1 = p.sm_scale * kLog2e;
  float m_run[2] = {-INFINITY, -INFINITY};  // running maxima of rows lane/4 and lane/4 + 8 (CTA-wide values)
  float l_part[2] = {0.f, 0.f};             // this thread's share of the row sums
  float oacc[C::NT][4];
#pragma unroll
  for (int n = 0; n < C::NT; ++n)
#pragma unroll
    for (int e = 0; e < 4; ++e) oacc[n][e] = 0.f;
  const int row_lo = lane >> 2;

  for (int t = 0; t < n_tiles; ++t) {
    cp_async_wait<C::NSTAGE - 2>();
    __syncthreads();  // tile t has landed for everyone; everyone is done with tile t - 1 and its P
    if (t + C::NSTAGE - 1 < n_tiles) load_tile(t + C::NSTAGE - 1);
    cp_async_commit();
    const uint32_t tile = sbase + (t % C::NSTAGE) * C::TILE_BYTES;
    const int key0 = start + t * LBK;

    // ---- 1. scores of keys 8 warp .. 8 warp + 7 ----
    // four independent accumulators: one chain of R / 16 dependent tensor-core steps would run at the
    // latency of a step, not at its issue rate
    float sa[4][4];
#pragma unroll
    for (int c = 0; c < 4; ++c)
#pragma unroll
      for (int e = 0; e < 4; ++e) sa[c][e] = 0.f;
    const int arow = ((lane >> 3) & 1) * 8 + (lane & 7);
    static_assert((R / 32) % 2 == 0, "the score loop takes four 16-wide steps per iteration");
#pragma unroll 2
    for (int kp = 0; kp < R / 32; kp += 2) {  // four 16-wide steps per iteration, one per accumulator
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4(tile + lswz(warp * 8 + (lane & 7), (kp + u) * 4 + (lane >> 3), C::ROW_BYTES), b0, b1, b2, b3);
        uint32_t a[4], a2[4];
        ldsm_x4(sbase + C::OFF_Q + lswz(arow, (kp + u) * 4 + (lane >> 4), C::ROW_BYTES), a[0], a[1], a[2], a[3]);
        ldsm_x4(sbase + C::OFF_Q + lswz(arow, (kp + u) * 4 + 2 + (lane >> 4), C::ROW_BYTES), a2[0], a2[1], a2[2], a2[3]);
        mma16816<T>(sa[2 * u], a, b0, b1);
        mma16816<T>(sa[2 * u + 1], a2, b2, b3);
      }
    }
    float s[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) s[e] = (sa[0][e] + sa[1][e]) + (sa[2][e] + sa[3][e]);
    float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int key = key0 + warp * 8 + (lane & 3) * 2 + (e & 1);
      s[e] = key < end ? s[e] * c1 : -INFINITY;
      tmax[e >> 1] = fmaxf(tmax[e >> 1], s[e]);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      tmax[h] = fmaxf(tmax[h], __shfl_xor_sync(0xffffffffu, tmax[h], 1));
      tmax[h] = fmaxf(tmax[h], __shfl_xor_sync(0xffffffffu, tmax[h], 2));
    }
    if ((lane & 3) == 0) {
      red[warp * 16 + row_lo] = tmax[0];
      red[warp * 16 + row_lo + 8] = tmax[1];
    }
    __syncthreads();

    // ---- 2. new running maxima (the same in every warp), rescale, probabilities to shared memory ----
    float corr[2], mu[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float mx = m_run[h];
#pragma unroll
      for (int w = 0; w < LWARPS; ++w) mx = fmaxf(mx, red[w * 16 + row_lo + 8 * h]);
      corr[h] = (mx == -INFINITY) ? 1.f : exp2f(m_run[h] - mx);
      m_run[h] = mx;
      mu[h] = (mx == -INFINITY) ? 0.f : mx;
      l_part[h] *= corr[h];
    }
#pragma unroll
    for (int n = 0; n < C::NT; ++n) {
      oacc[n][0] *= corr[0];
      oacc[n][1] *= corr[0];
      oacc[n][2] *= corr[1];
      oacc[n][3] *= corr[1];
    }
    {
      const float p0 = exp2f(s[0] - mu[0]), p1 = exp2f(s[1] - mu[0]);
      const float p2 = exp2f(s[2] - mu[1]), p3 = exp2f(s[3] - mu[1]);
      l_part[0] += p0 + p1;
      l_part[1] += p2 + p3;
      // P [16 rows][64 keys] in the input dtype: 128-byte rows, 16-byte chunk = 8 keys = one warp's slice
      const uint32_t pb = sbase + C::OFF_P;
      const uint32_t off_lo = lswz(row_lo, warp, 128) + (lane & 3) * 4;
      const uint32_t off_hi = lswz(row_lo + 8, warp, 128) + (lane & 3) * 4;
      asm volatile("st.shared.b32 [%0], %1;\n" ::"r"(pb + off_lo), "r"(pack2<T>(p0, p1)) : "memory");
      asm volatile("st.shared.b32 [%0], %1;\n" ::"r"(pb + off_hi), "r"(pack2<T>(p2, p3)) : "memory");
    }
    __syncthreads();

    // ---- 3. O[:, warp's columns] += P . C_tile[:, warp's columns] ----
    uint32_t pf[4][4];
    {
      const int arow = ((lane >> 3) & 1) * 8 + (lane & 7);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks)
        ldsm_x4(sbase + C::OFF_P + lswz(arow, ks * 2 + (lane >> 4), 128), pf[ks][0], pf[ks][1], pf[ks][2], pf[ks][3]);
    }
    const int col_chunk0 = warp * C::NT;  // first 16-byte chunk (8 columns) of this warp's output slice
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      const int vrow = ks * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
#pragma unroll
      for (int np = 0; np < C::NT / 2; ++np) {
        uint32_t v0, v1, v2, v3;
        ldsm_x4_trans(tile + lswz(vrow, col_chunk0 + np * 2 + (lane >> 4), C::ROW_BYTES), v0, v1, v2, v3);
        mma16816<T>(oacc[2 * np], pf[ks], v0, v1);
        mma16816<T>(oacc[2 * np + 1], pf[ks], v2, v3);
      }
      if constexpr (C::NT % 2 == 1) {  // odd tile count: the last 8 columns alone (lanes 16-31 repeat the address)
        uint32_t v0, v1, v2, v3;
        ldsm_x4_trans(tile + lswz(vrow, col_chunk0 + C::NT - 1, C::ROW_BYTES), v0, v1, v2, v3);
        mma16816<T>(oacc[C::NT - 1], pf[ks], v0, v1);
      }
    }
  }

  // ---- row sums over the CTA, then the partial ----
  cp_async_wait<0>();
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_part[h] += __shfl_xor_sync(0xffffffffu, l_part[h], 1);
    l_part[h] += __shfl_xor_sync(0xffffffffu, l_part[h], 2);
  }
  __syncthreads();  // the maxima in `red` have been read by everyone
  if ((lane & 3) == 0) {
    red[LWARPS * 16 + warp * 16 + row_lo] = l_part[0];
    red[LWARPS * 16 + warp * 16 + row_lo + 8] = l_part[1];
  }
  __syncthreads();
  float lsum[2] = {0.f, 0.f};
#pragma unroll
  for (int w = 0; w < LWARPS; ++w) {
    lsum[0] += red[LWARPS * 16 + w * 16 + row_lo];
    lsum[1] += red[LWARPS * 16 + w * 16 + row_lo + 8];
  }
  const int64_t part = (((int64_t)blockIdx.z * p.Hkv + grp) * p.num_splits + split) * p.rows;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = row_lo + 8 * h;
    if (r >= p.rows) continue;
    const float inv = lsum[h] > 0.f ? 1.f / lsum[h] : 0.f;
#pragma unroll
    for (int n = 0; n < C::NT; ++n) {
      const int col = (warp * C::NT + n) * 8 + (lane & 3) * 2;
      float2 v = make_float2(oacc[n][2 * h] * inv, oacc[n][2 * h + 1] * inv);
      *reinterpret_cast<float2*>(p.o_part + (part + r) * R + col) = v;
    }
    if (warp == 0 && (lane & 3) == 0) p.lse_part[part + r] = lsum[h] > 0.f ? m_run[h] + log2f(lsum[h]) : -INFINITY;
  }
}

template <typename T, int R>
int launch_latent_t(const DecodeParams& p, cudaStream_t stream) {
  using C = LCfg<R>;
  auto kern = decode_latent_kernel<T, R>;
  int rc = check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM),
                      "cudaFuncSetAttribute(latent decode)");
  if (rc) return rc;
  kern<<<dim3(p.num_splits, p.Hkv, p.B), LTHR, C::SMEM, stream>>>(p);
  count_launch();
  return check_cuda(cudaGetLastError(), "latent decode launch");
}

template <typename T>
int launch_latent_r(const DecodeParams& p, cudaStream_t stream) {
  switch (p.D) {
    case 128: return launch_latent_t<T, 128>(p, stream);
    case 256: return launch_latent_t<T, 256>(p, stream);
    case 512: return launch_latent_t<T, 512>(p, stream);
    case 576: return launch_latent_t<T, 576>(p, stream);
  }
  return fail(PJX_ERR_UNSUPPORTED, "latent decode: latent width %d is not built (128, 256, 512, 576)", p.D);
}

}  // namespace

bool decode_latent_supported(int R, int dtype) {
  return (dtype == PJX_BF16 || dtype == PJX_F16) && (R == 128 || R == 256 || R == 512 || R == 576);
}

// Split kernel only; the caller runs the combine of the GQA decode on the same DecodeParams.
int launch_decode_latent_splits(const DecodeParams& p, int dtype, cudaStream_t stream) {
  return dtype == PJX_BF16 ? launch_latent_r<__nv_bfloat16>(p, stream) : launch_latent_r<__half>(p, stream);
}

}  // namespace pjx
