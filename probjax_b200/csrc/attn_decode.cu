// Split-KV decode forward and the exact (o, lse) combine.
//
// The decode step is bandwidth bound: every K and V byte of the valid part of
// the cache is read once, and with GQA the G = Hq/Hkv query heads that share a
// KV head are packed as rows of one small matrix so that the KV tile is read
// once per group (the reference packs the same way,
// probjax/nn/pallas_kernels/kernels/attention_splitkv.py:121-126).
//
// Grid (split, kv head, batch).  A CTA of four warps streams its split of the
// cache through a cp.async ring of 64-key tiles (K and V, 16-byte vector copies,
// XOR-swizzled rows); warp w owns keys 16w..16w+15 of every tile and keeps its
// own running (max, sum, O) so that no CTA-wide exchange happens inside the
// loop.  Scores and P.V use mma.sync m16n8k16 with the packed query rows padded
// to 16 -- the tensor work is far below the memory time, so the padding is free.
// The four warps are merged once at the end and the CTA writes one partial:
// O normalised by its own sum (fp32) and a base-2 LSE, which is what the
// reference kernel emits per split (attention_splitkv.py:97-103).  A second tiny
// kernel combines the valid splits exactly (attention_splitkv.py:236-250).
//
// Unlike the reference kernel this one takes per-sequence valid lengths: keys at
// positions >= kv_lengths[b] are neither read nor counted.
#include "pjx_common.cuh"
#include "mma_sync.cuh"

namespace pjx {
namespace {

using namespace mma_sync;

constexpr int BK = 64;       // keys per tile
constexpr int NWARP = 4;
constexpr int NTHR = NWARP * 32;
constexpr int NSTAGE = 3;

// Byte offset of 16-byte chunk `c` of row `r` inside a swizzled [rows][HD] tile.
template <int HD>
__device__ __forceinline__ uint32_t swz(int r, int c) {
  return static_cast<uint32_t>(r * (HD * 2) + ((c ^ (r & 7)) << 4));
}

__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;\n" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ void st_volatile_v4(uint4* p, uint4 v) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};\n" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 ld_volatile_v4(const uint4* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

// Streams keys [start, end) of (batch b, kv head hk) and writes the partial result -- O normalised by
// its own sum and a base-2 LSE per packed query row -- at row offset `part` of the partial arrays.
// Every thread of the CTA takes part; on return the shared memory is free again.
template <typename T, int HD, bool PAGED>
__device__ __forceinline__ void stream_segment(const DecodeParams& p, unsigned char* smem_raw, int b, int hk, int start,
                                               int end, int64_t part) {
  constexpr int CH = HD / 8;               // 16-byte chunks per row
  constexpr int TILE_BYTES = BK * HD * 2;  // one K or V tile
  constexpr int KS = HD / 16;              // k-steps of the score product
  constexpr int NT_O = HD / 8;             // output n-tiles
  const int n_tiles = max(0, (end - start + BK - 1) / BK);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = p.Hq / p.Hkv;
  // contiguous cache: the sequence's rows; paged cache: the pool (rows are found per tile)
  const int64_t seq_row0 = PAGED ? 0 : (int64_t)b * p.capacity;
  const T* kbase = static_cast<const T*>(p.k) + (seq_row0 * p.Hkv + hk) * HD;
  const T* vbase = static_cast<const T*>(p.v) + (seq_row0 * p.Hkv + hk) * HD;
  const int64_t tok_stride = (int64_t)p.Hkv * HD;
  const uint32_t smem_base = smem_u32(smem_raw);

  auto load_tile = [&](int t) {
    const int stage = t % NSTAGE;
    const uint32_t ks = smem_base + stage * 2 * TILE_BYTES;
    const uint32_t vs = ks + TILE_BYTES;
    const int key0 = start + t * BK;
    // pool row of the tile's first key: a 64-key tile never straddles a page
    int64_t row0 = key0;
    if constexpr (PAGED)
      row0 = (int64_t)p.block_table[(int64_t)b * p.max_pages + key0 / p.page_size] * p.page_size + key0 % p.page_size;
#pragma unroll
    for (int i = 0; i < BK * CH / NTHR; ++i) {
      const int idx = tid + i * NTHR;
      const int r = idx / CH, c = idx % CH;
      const bool ok = key0 + r < end;
      const int64_t off = (row0 + (ok ? r : 0)) * tok_stride + c * 8;
      cp_async16(ks + swz<HD>(r, c), kbase + off, ok ? 16 : 0);
      cp_async16(vs + swz<HD>(r, c), vbase + off, ok ? 16 : 0);
    }
  };

#pragma unroll
  for (int s = 0; s < NSTAGE - 1; ++s) {
    if (s < n_tiles) load_tile(s);
    cp_async_commit();
  }

  // Query fragments (A operand): packed row r = g * Lq + t of this KV head.
  uint32_t qf[KS][4];
  {
    const T* q = static_cast<const T*>(p.q);
    const int r0 = lane >> 2, cq = (lane & 3) * 2;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = r0 + half * 8;
      const bool ok = r < p.rows;
      const int g = ok ? r / p.Lq : 0, t = ok ? r % p.Lq : 0;
      const T* qrow = q + (((int64_t)b * p.Lq + t) * p.Hq + hk * G + g) * HD;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        uint32_t lo = 0, hi = 0;
        if (ok) {
          lo = *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + cq);
          hi = *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + cq + 8);
        }
        qf[ks][half] = lo;
        qf[ks][half + 2] = hi;
      }
    }
  }

  const float c1 = p.sm_scale * kLog2e;
  float m_ref[2] = {-INFINITY, -INFINITY};
  float l_part[2] = {0.f, 0.f};
  float oacc[NT_O][4];
#pragma unroll
  for (int n = 0; n < NT_O; ++n)
#pragma unroll
    for (int e = 0; e < 4; ++e) oacc[n][e] = 0.f;

  for (int t = 0; t < n_tiles; ++t) {
    cp_async_wait<NSTAGE - 2>();
    __syncthreads();
    if (t + NSTAGE - 1 < n_tiles) load_tile(t + NSTAGE - 1);
    cp_async_commit();

    const int stage = t % NSTAGE;
    const uint32_t ks_addr = smem_base + stage * 2 * TILE_BYTES;
    const uint32_t vs_addr = ks_addr + TILE_BYTES;
    const int key_w = start + t * BK + warp * 16;  // first key of this warp's slice
    if (key_w >= end) continue;                    // warp-uniform: slice has no valid key

    // ---- scores: S[16 rows x 16 keys] ----
    float s[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) s[nt][e] = 0.f;
      const int row = warp * 16 + nt * 8 + (lane & 7);
#pragma unroll
      for (int kp = 0; kp < KS / 2; ++kp) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4(ks_addr + swz<HD>(row, kp * 4 + (lane >> 3)), b0, b1, b2, b3);
        mma16816<T>(s[nt], qf[2 * kp], b0, b1);
        mma16816<T>(s[nt], qf[2 * kp + 1], b2, b3);
      }
    }

    // ---- online softmax (exp2 domain) with lazy rescaling ----
    float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = key_w + nt * 8 + (lane & 3) * 2 + (e & 1);
        const float x = key < end ? s[nt][e] * c1 : -INFINITY;
        s[nt][e] = x;
        tmax[e >> 1] = fmaxf(tmax[e >> 1], x);
      }
#pragma unroll
    for (int hrow = 0; hrow < 2; ++hrow) {
      tmax[hrow] = fmaxf(tmax[hrow], __shfl_xor_sync(0xffffffffu, tmax[hrow], 1));
      tmax[hrow] = fmaxf(tmax[hrow], __shfl_xor_sync(0xffffffffu, tmax[hrow], 2));
    }
    const bool need = (tmax[0] > m_ref[0] + 8.f) || (tmax[1] > m_ref[1] + 8.f) ||
                      (m_ref[0] == -INFINITY && tmax[0] > -INFINITY) ||
                      (m_ref[1] == -INFINITY && tmax[1] > -INFINITY);
    if (__any_sync(0xffffffffu, need)) {
      float corr[2];
#pragma unroll
      for (int hrow = 0; hrow < 2; ++hrow) {
        const float m_new = fmaxf(m_ref[hrow], tmax[hrow]);
        corr[hrow] = (m_new == -INFINITY) ? 1.f : exp2f(m_ref[hrow] - m_new);
        m_ref[hrow] = m_new;
        l_part[hrow] *= corr[hrow];
      }
#pragma unroll
      for (int n = 0; n < NT_O; ++n) {
        oacc[n][0] *= corr[0];
        oacc[n][1] *= corr[0];
        oacc[n][2] *= corr[1];
        oacc[n][3] *= corr[1];
      }
    }
    uint32_t pf[4];
    {
      const float mu0 = m_ref[0] == -INFINITY ? 0.f : m_ref[0];
      const float mu1 = m_ref[1] == -INFINITY ? 0.f : m_ref[1];
      float pr[2][4];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        pr[nt][0] = exp2f(s[nt][0] - mu0);
        pr[nt][1] = exp2f(s[nt][1] - mu0);
        pr[nt][2] = exp2f(s[nt][2] - mu1);
        pr[nt][3] = exp2f(s[nt][3] - mu1);
        l_part[0] += pr[nt][0] + pr[nt][1];
        l_part[1] += pr[nt][2] + pr[nt][3];
      }
      pf[0] = pack2<T>(pr[0][0], pr[0][1]);
      pf[1] = pack2<T>(pr[0][2], pr[0][3]);
      pf[2] = pack2<T>(pr[1][0], pr[1][1]);
      pf[3] = pack2<T>(pr[1][2], pr[1][3]);
    }

    // ---- O[16 x HD] += P[16 x 16 keys] . V[16 keys x HD] ----
    {
      const int row = warp * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
#pragma unroll
      for (int np = 0; np < NT_O / 2; ++np) {
        uint32_t v0, v1, v2, v3;
        ldsm_x4_trans(vs_addr + swz<HD>(row, np * 2 + (lane >> 4)), v0, v1, v2, v3);
        mma16816<T>(oacc[2 * np], pf, v0, v1);
        mma16816<T>(oacc[2 * np + 1], pf, v2, v3);
      }
    }
  }

  // ---- merge the four warps ----
  cp_async_wait<0>();
  // Overlapped launch (ex_overlap): this grid may have started while the kernel before it on the stream
  // was still running.  Everything up to here only read this call's inputs; from here on the kernel writes
  // memory the previous kernel may still be reading (partials, counters, exchange records), so it waits
  // for that kernel to have completed.  Without the launch attribute the instruction does nothing.
  if (p.ex_overlap) asm volatile("griddepcontrol.wait;\n" ::: "memory");
  __syncthreads();  // every warp is done with the ring: reuse it as fp32 scratch
  float* sm_o = reinterpret_cast<float*>(smem_raw);          // [NWARP][16][HD]
  float* sm_m = sm_o + NWARP * 16 * HD;                       // [NWARP][16]
  float* sm_l = sm_m + NWARP * 16;                            // [NWARP][16]
#pragma unroll
  for (int hrow = 0; hrow < 2; ++hrow) {
    float lsum = l_part[hrow];
    lsum += __shfl_xor_sync(0xffffffffu, lsum, 1);
    lsum += __shfl_xor_sync(0xffffffffu, lsum, 2);
    if ((lane & 3) == 0) {
      sm_m[warp * 16 + (lane >> 2) + hrow * 8] = m_ref[hrow];
      sm_l[warp * 16 + (lane >> 2) + hrow * 8] = lsum;
    }
  }
#pragma unroll
  for (int n = 0; n < NT_O; ++n) {
    const int col = n * 8 + (lane & 3) * 2;
    float* r0 = sm_o + (warp * 16 + (lane >> 2)) * HD + col;
    float* r1 = r0 + 8 * HD;
    r0[0] = oacc[n][0];
    r0[1] = oacc[n][1];
    r1[0] = oacc[n][2];
    r1[1] = oacc[n][3];
  }
  __syncthreads();

  for (int idx = tid; idx < p.rows * HD; idx += NTHR) {
    const int r = idx / HD, d = idx % HD;
    float mall = -INFINITY;
#pragma unroll
    for (int w = 0; w < NWARP; ++w) mall = fmaxf(mall, sm_m[w * 16 + r]);
    float lall = 0.f, o = 0.f;
#pragma unroll
    for (int w = 0; w < NWARP; ++w) {
      const float mw = sm_m[w * 16 + r];
      const float sc = (mw == -INFINITY) ? 0.f : exp2f(mw - mall);
      lall += sm_l[w * 16 + r] * sc;
      o += sm_o[(w * 16 + r) * HD + d] * sc;
    }
    p.o_part[(part + r) * HD + d] = lall > 0.f ? o / lall : 0.f;
    if (d == 0) p.lse_part[part + r] = lall > 0.f ? mall + log2f(lall) : -INFINITY;
  }

  __syncthreads();  // the merge scratch is shared memory the next segment's tiles will land in
}

// FUSED (sequence-sharded decode, whole grid co-resident): the last CTA of each (batch, kv
// head) to finish combines the head's splits, stores the rank's partial into every rank's
// exchange buffer, raises the head's flag there, waits (bounded) for the same head's flags of
// all ranks and writes the final result -- the whole exchange inside this one launch.
template <typename T, int HD, bool PAGED, bool FUSED>
__global__ void __launch_bounds__(NTHR, 2) decode_splitkv_kernel(const DecodeParams p) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int split = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  int len = p.capacity;
  if (p.kv_lengths) len = max(0, min(len, p.kv_lengths[b]));
  const int start = split * p.split_len;
  // nothing to do; the combine never reads this split (in the fused exchange split 0 always
  // runs, so that a head without keys still publishes its empty partial)
  if (start >= len && !(FUSED && split == 0)) return;
  const int end = min(len, start + p.split_len);
  // Let the next kernel on the stream start as SM slots free up, if it was launched for that: the
  // combine of the splits always is (it waits for this grid before it reads a partial), the next
  // step's kernel of a sharded decode is with ex_overlap.
  if (!FUSED || p.ex_overlap) asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  stream_segment<T, HD, PAGED>(p, smem_raw, b, hk, start, end,
                               (((int64_t)b * p.Hkv + hk) * p.num_splits + split) * p.rows);
  [[maybe_unused]] const int tid = threadIdx.x;
  [[maybe_unused]] const int G = p.Hq / p.Hkv;

  if constexpr (FUSED) {
    // Exchange in "data + flag" words (the low-latency protocol collectives libraries use for small
    // messages): every value crosses NVLink inside a 16-byte store {v0, step, v1, step}, so a value is
    // valid exactly when the step number beside it is this step's -- no fence, no separate flag, one
    // one-way trip.  Only stores go to peers; all polling is on this GPU's own memory.
    const int64_t N = (int64_t)p.B * p.Lq * p.Hq;
    const int unit = b * p.Hkv + hk;
    unsigned char* mine = p.ex_buf[p.ex_rank];
    uint32_t* counters = reinterpret_cast<uint32_t*>(mine + exchange_unit_flags_offset(p.ex_world, N, HD)) + (size_t)p.ex_world * N;
    const size_t ll_off = exchange_ll_offset(p.ex_world, N, HD);
    const int ns = max(1, (len + p.split_len - 1) / p.split_len);  // CTAs of this head that run
    __shared__ int s_last;
    __threadfence();  // this CTA's partial is visible device-wide before it is counted
    __syncthreads();
    if (tid == 0) {
      const uint32_t prev = atomicAdd(counters + unit, 1u);
      s_last = (prev == (uint32_t)(ns - 1));
      if (s_last) counters[unit] = 0;  // ready for the next step (the next launch on this stream)
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();

    const int64_t pbase = ((int64_t)b * p.Hkv + hk) * p.num_splits;
    const uint32_t step = p.ex_step;
    const int par = step & 1;
    // LL region of one rank: [2 parities][world][N] records of (HD / 2 + 1) 16-byte lines:
    // HD / 2 lines of two output values each, then one line holding the natural-log LSE.
    constexpr int LINES = HD / 2 + 1;
    auto line_of = [&](unsigned char* base, int src_rank, int64_t n, int line) {
      return reinterpret_cast<uint4*>(base + ll_off) + ((((size_t)par * p.ex_world + src_rank) * N + n) * LINES + line);
    };
    T* o = static_cast<T*>(p.o);
    bool timed_out = false;
    for (int idx = tid; idx < p.rows * (HD / 4); idx += NTHR) {
      const int r = idx / (HD / 4), d4 = idx % (HD / 4);
      const int g = r / p.Lq, t = r % p.Lq;
      const int64_t n = ((int64_t)b * p.Lq + t) * p.Hq + hk * G + g;
      // ---- this rank's partial of the row: exact combine of its splits (base-2 LSEs) ----
      float m = -INFINITY;
      for (int s = 0; s < ns; ++s) m = fmaxf(m, __ldcg(p.lse_part + (pbase + s) * p.rows + r));
      const float msafe = (m == -INFINITY) ? 0.f : m;
      float denom = 0.f;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int s = 0; s < ns; ++s) {
        const float w = exp2f(__ldcg(p.lse_part + (pbase + s) * p.rows + r) - msafe);
        const float4 x = __ldcg(reinterpret_cast<const float4*>(p.o_part + ((pbase + s) * p.rows + r) * HD) + d4);
        denom += w;
        acc.x = fmaf(w, x.x, acc.x);
        acc.y = fmaf(w, x.y, acc.y);
        acc.z = fmaf(w, x.z, acc.z);
        acc.w = fmaf(w, x.w, acc.w);
      }
      const float inv = denom > 0.f ? 1.f / denom : 0.f;
      acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
      const float my_lse = denom > 0.f ? (msafe + log2f(denom)) * kLn2 : INFINITY;  // natural log, +inf = no keys
      // ---- publish to every peer ----
      const uint4 l0 = make_uint4(__float_as_uint(acc.x), step, __float_as_uint(acc.y), step);
      const uint4 l1 = make_uint4(__float_as_uint(acc.z), step, __float_as_uint(acc.w), step);
      const uint4 ll = make_uint4(__float_as_uint(my_lse), step, 0u, step);
      for (int q = 0; q < p.ex_world; ++q) {
        if (q == p.ex_rank) continue;
        st_volatile_v4(line_of(p.ex_buf[q], p.ex_rank, n, 2 * d4), l0);
        st_volatile_v4(line_of(p.ex_buf[q], p.ex_rank, n, 2 * d4 + 1), l1);
        if (d4 == 0) st_volatile_v4(line_of(p.ex_buf[q], p.ex_rank, n, HD / 2), ll);
      }
      // ---- gather the peers' partials of the same row (bounded wait) and combine ----
      float lse_q[kMaxExchangeRanks];
      float mx = (my_lse == INFINITY) ? -INFINITY : my_lse;
      const long long t0 = clock64();
      for (int q = 0; q < p.ex_world; ++q) {
        if (q == p.ex_rank) {
          lse_q[q] = my_lse;
          continue;
        }
        uint4 v = ld_volatile_v4(line_of(mine, q, n, HD / 2));
        while (!timed_out && (v.y != step || v.w != step)) {
          if (clock64() - t0 > 4000000000LL) timed_out = true;  // about two seconds: a peer never published
          v = ld_volatile_v4(line_of(mine, q, n, HD / 2));
        }
        lse_q[q] = timed_out ? INFINITY : __uint_as_float(v.x);
        if (lse_q[q] != INFINITY) mx = fmaxf(mx, lse_q[q]);
      }
      const float mxs = (mx == -INFINITY) ? 0.f : mx;
      float den = 0.f;
      float4 out4 = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int q = 0; q < p.ex_world; ++q) {
        const float w = (lse_q[q] == INFINITY) ? 0.f : expf(lse_q[q] - mxs);
        den += w;
        float4 x = acc;
        if (q != p.ex_rank) {
          uint4 a = ld_volatile_v4(line_of(mine, q, n, 2 * d4));
          uint4 c = ld_volatile_v4(line_of(mine, q, n, 2 * d4 + 1));
          while (!timed_out && (a.y != step || a.w != step || c.y != step || c.w != step)) {
            if (clock64() - t0 > 4000000000LL) timed_out = true;
            a = ld_volatile_v4(line_of(mine, q, n, 2 * d4));
            c = ld_volatile_v4(line_of(mine, q, n, 2 * d4 + 1));
          }
          x = make_float4(__uint_as_float(a.x), __uint_as_float(a.z), __uint_as_float(c.x), __uint_as_float(c.z));
        }
        if (w != 0.f) {  // a rank without keys contributes nothing (its record may hold anything finite or not)
          out4.x = fmaf(w, x.x, out4.x);
          out4.y = fmaf(w, x.y, out4.y);
          out4.z = fmaf(w, x.z, out4.z);
          out4.w = fmaf(w, x.w, out4.w);
        }
      }
      const float dinv = den > 0.f ? 1.f / den : 0.f;
      uint2 packed;
      packed.x = pack2<T>(out4.x * dinv, out4.y * dinv);
      packed.y = pack2<T>(out4.z * dinv, out4.w * dinv);
      *reinterpret_cast<uint2*>(o + n * HD + d4 * 4) = packed;
      if (p.lse && d4 == 0) p.lse[((int64_t)b * p.Hq + hk * G + g) * p.Lq + t] = den > 0.f ? mxs + logf(den) : INFINITY;
    }
    if (timed_out && p.status) atomicExch(p.status, (int)PJX_ERR_DEVICE_TIMEOUT);
  }
}

// One CTA per packed row (b, kv head, r): exact combine of the valid splits.
template <typename TO>
__global__ void combine_splits_kernel(const DecodeParams p) {
  const int r = blockIdx.x, hk = blockIdx.y;
  // Launched with programmatic stream serialization, the grid may be resident before the split kernel
  // has finished: wait for that grid and its stores.  (Does nothing under a plain launch.)
  asm volatile("griddepcontrol.wait;\n" ::: "memory");
  const DecodeSeq sq = decode_seq(p, blockIdx.z);
  const int len = sq.len;
  const int ns = (len + p.split_len - 1) / p.split_len;
  const int64_t base = ((int64_t)blockIdx.z * p.Hkv + hk) * p.num_splits;
  float m = -INFINITY;
  for (int s = 0; s < ns; ++s) m = fmaxf(m, p.lse_part[(base + s) * p.rows + r]);
  const float msafe = (m == -INFINITY) ? 0.f : m;
  float denom = 0.f;
  for (int s = 0; s < ns; ++s) denom += exp2f(p.lse_part[(base + s) * p.rows + r] - msafe);
  const float inv = denom > 0.f ? 1.f / denom : 0.f;
  const int G = p.Hq / p.Hkv;
  const int g = r / p.Lq, t = r % p.Lq;
  const int h = hk * G + g;
  TO* o = static_cast<TO*>(p.o) + ((sq.q_b * p.Lq + t) * p.Hq + h) * p.Dv;
  for (int d = threadIdx.x; d < p.Dv; d += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < ns; ++s) {
      const float w = exp2f(p.lse_part[(base + s) * p.rows + r] - msafe);
      acc += w * p.o_part[((base + s) * p.rows + r) * p.Dv + d];
    }
    o[d] = Elem<TO>::from_f(acc * inv);
  }
  if (p.lse && threadIdx.x == 0)
    p.lse[decode_lse_index(p, sq, h, t)] = denom > 0.f ? (msafe + log2f(denom)) * kLn2 : INFINITY;
}

// Combine of n_parts partials laid out [n_parts, n_rows, Dv] with natural-log LSEs.
template <typename TO>
__global__ void combine_parts_kernel(const float* __restrict__ o_parts, const float* __restrict__ lse_parts,
                                     int n_parts, int64_t n_rows, int Dv, TO* __restrict__ o,
                                     float* __restrict__ lse) {
  const int64_t row = blockIdx.x;
  float m = -INFINITY;
  for (int s = 0; s < n_parts; ++s) {
    const float x = lse_parts[s * n_rows + row];
    if (x != INFINITY) m = fmaxf(m, x);  // +inf marks a part without keys
  }
  const float msafe = (m == -INFINITY) ? 0.f : m;
  float denom = 0.f;
  for (int s = 0; s < n_parts; ++s) {
    const float x = lse_parts[s * n_rows + row];
    denom += (x == INFINITY) ? 0.f : expf(x - msafe);
  }
  const float inv = denom > 0.f ? 1.f / denom : 0.f;
  for (int d = threadIdx.x; d < Dv; d += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < n_parts; ++s) {
      const float x = lse_parts[s * n_rows + row];
      const float w = (x == INFINITY) ? 0.f : expf(x - msafe);
      acc += w * o_parts[(s * n_rows + row) * Dv + d];
    }
    o[row * Dv + d] = Elem<TO>::from_f(acc * inv);
  }
  if (lse && threadIdx.x == 0) lse[row] = denom > 0.f ? msafe + logf(denom) : INFINITY;
}

// ---------------------------------------------------------------------------
// Sequence-sharded decode: the exchange of per-rank partials is done by the
// kernels themselves with plain stores into the peers' memory over NVLink (no
// library collective): the message is one (Dv + 1)-float record per (sequence,
// query head), a few hundred KB, so its cost is latency, not bandwidth.
//
//   publish_partials_kernel   combines this rank's splits and writes the fp32
//                             partial + natural-log LSE into slot [rank] of every
//                             rank's exchange buffer; the last CTA to finish then
//                             raises this rank's flag on every rank (release, system scope).
//   gather_combine_kernel     waits (bounded) until all ranks' flags show this
//                             step, then combines the partials out of local memory.
//
// Buffers are double buffered by step parity: a rank can run at most one step
// ahead of a peer, because its next combine needs that peer's next flag.
// ---------------------------------------------------------------------------
__global__ void publish_partials_kernel(const DecodeParams p) {
  const int r = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  int len = p.capacity;
  if (p.kv_lengths) len = max(0, min(len, p.kv_lengths[b]));
  const int ns = (len + p.split_len - 1) / p.split_len;
  const int64_t base = ((int64_t)b * p.Hkv + hk) * p.num_splits;
  float m = -INFINITY;
  for (int s = 0; s < ns; ++s) m = fmaxf(m, p.lse_part[(base + s) * p.rows + r]);
  const float msafe = (m == -INFINITY) ? 0.f : m;
  float denom = 0.f;
  for (int s = 0; s < ns; ++s) denom += exp2f(p.lse_part[(base + s) * p.rows + r] - msafe);
  const float inv = denom > 0.f ? 1.f / denom : 0.f;
  const int G = p.Hq / p.Hkv;
  const int g = r / p.Lq, t = r % p.Lq;
  const int h = hk * G + g;
  const int64_t N = (int64_t)p.B * p.Lq * p.Hq;
  const int64_t n = ((int64_t)b * p.Lq + t) * p.Hq + h;
  const size_t half = exchange_record_floats(p.ex_world, N, p.Dv);
  const size_t o_off = (p.ex_step & 1) * half + ((size_t)p.ex_rank * N + n) * p.Dv;
  const size_t l_off = (p.ex_step & 1) * half + (size_t)p.ex_world * N * p.Dv + (size_t)p.ex_rank * N + n;
  for (int d = threadIdx.x; d < p.Dv; d += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < ns; ++s) {
      const float w = exp2f(p.lse_part[(base + s) * p.rows + r] - msafe);
      acc += w * p.o_part[((base + s) * p.rows + r) * p.Dv + d];
    }
    acc *= inv;
    for (int q = 0; q < p.ex_world; ++q) reinterpret_cast<float*>(p.ex_buf[q])[o_off + d] = acc;
  }
  if (threadIdx.x == 0) {
    const float lse = denom > 0.f ? (msafe + log2f(denom)) * kLn2 : INFINITY;
    for (int q = 0; q < p.ex_world; ++q) reinterpret_cast<float*>(p.ex_buf[q])[l_off] = lse;
  }
  __syncthreads();  // the CTA's stores are ordered before thread 0's fence (cumulativity)
  if (threadIdx.x == 0) {
    __threadfence_system();
    uint32_t* flags = reinterpret_cast<uint32_t*>(p.ex_buf[p.ex_rank] + 2 * half * sizeof(float));
    uint32_t* counter = flags + kMaxExchangeRanks;
    const uint32_t total = gridDim.x * gridDim.y * gridDim.z;
    if (atomicAdd(counter, 1u) == total - 1) {
      *counter = 0;
      __threadfence_system();
      for (int q = 0; q < p.ex_world; ++q)
        st_release_sys_u32(reinterpret_cast<uint32_t*>(p.ex_buf[q] + 2 * half * sizeof(float)) + p.ex_rank, p.ex_step);
    }
  }
}

template <typename TO>
__global__ void gather_combine_kernel(const DecodeParams p) {
  const int64_t N = (int64_t)p.B * p.Lq * p.Hq;
  const int64_t n = blockIdx.x;
  const size_t half = exchange_record_floats(p.ex_world, N, p.Dv);
  const unsigned char* mine = p.ex_buf[p.ex_rank];
  if (threadIdx.x < p.ex_world) {  // one thread per peer flag, polled in parallel
    const volatile uint32_t* flag = reinterpret_cast<const volatile uint32_t*>(mine + 2 * half * sizeof(float)) + threadIdx.x;
    const long long t0 = clock64();
    while (static_cast<int32_t>(*flag - p.ex_step) < 0) {
      if (clock64() - t0 > 4000000000LL) {  // about two seconds: a peer never published
        if (p.status) atomicExch(p.status, (int)PJX_ERR_DEVICE_TIMEOUT);
        break;
      }
    }
    __threadfence_system();  // acquire: the peers' records are visible after their flags
  }
  __syncthreads();
  const float* o_parts = reinterpret_cast<const float*>(mine) + (p.ex_step & 1) * half;
  const float* lse_parts = o_parts + (size_t)p.ex_world * N * p.Dv;
  float m = -INFINITY;
  for (int s = 0; s < p.ex_world; ++s) {
    const float x = __ldcg(lse_parts + s * N + n);
    if (x != INFINITY) m = fmaxf(m, x);
  }
  const float msafe = (m == -INFINITY) ? 0.f : m;
  float denom = 0.f;
  for (int s = 0; s < p.ex_world; ++s) {
    const float x = __ldcg(lse_parts + s * N + n);
    denom += (x == INFINITY) ? 0.f : expf(x - msafe);
  }
  const float inv = denom > 0.f ? 1.f / denom : 0.f;
  TO* o = static_cast<TO*>(p.o);
  for (int d = threadIdx.x; d < p.Dv; d += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < p.ex_world; ++s) {
      const float x = __ldcg(lse_parts + s * N + n);
      const float w = (x == INFINITY) ? 0.f : expf(x - msafe);
      acc += w * __ldcg(o_parts + (s * N + n) * p.Dv + d);
    }
    o[n * p.Dv + d] = Elem<TO>::from_f(acc * inv);
  }
  if (p.lse && threadIdx.x == 0) {
    const int h = n % p.Hq, t = (n / p.Hq) % p.Lq, b = n / ((int64_t)p.Hq * p.Lq);
    p.lse[((int64_t)b * p.Hq + h) * p.Lq + t] = denom > 0.f ? msafe + logf(denom) : INFINITY;
  }
}

// The combine of the splits is launched so that it may become resident while the split kernel's last
// CTAs still run (its first instruction waits for that grid): the launch latency of the second kernel,
// a few microseconds of a short decode step, is hidden behind the first.
template <typename TO>
cudaError_t launch_combine_splits(const DecodeParams& p, cudaStream_t stream) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.rows, p.Hkv, p.B);
  cfg.blockDim = dim3(p.Dv >= 128 ? 128 : 64);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, combine_splits_kernel<TO>, p);
}

// CTAs of the split kernel that one device holds at once (2 per SM unless the driver says otherwise).
template <typename T, int HD>
int coresident_ctas_t(int* out) {
  constexpr int smem = NSTAGE * 2 * BK * HD * 2;
  auto kern = decode_splitkv_kernel<T, HD, false, true>;
  int rc = check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem),
                      "cudaFuncSetAttribute(decode)");
  if (rc) return rc;
  int dev = 0, sms = 0, per_sm = 0;
  if ((rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice"))) return rc;
  if ((rc = check_cuda(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev), "SM count"))) return rc;
  if ((rc = check_cuda(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, NTHR, smem), "occupancy query"))) return rc;
  *out = sms * per_sm;
  return PJX_OK;
}

template <typename T, int HD>
int launch_decode_t(const DecodeParams& p, cudaStream_t stream) {
  constexpr int smem = NSTAGE * 2 * BK * HD * 2;
  static_assert(smem >= (NWARP * 16 * HD + 2 * NWARP * 16) * 4, "merge scratch must fit in the ring");
  auto kern = p.block_table
                  ? (p.ex_fused ? decode_splitkv_kernel<T, HD, true, true> : decode_splitkv_kernel<T, HD, true, false>)
                  : (p.ex_fused ? decode_splitkv_kernel<T, HD, false, true> : decode_splitkv_kernel<T, HD, false, false>);
  int rc = check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem),
                      "cudaFuncSetAttribute(decode)");
  if (rc) return rc;
  dim3 grid(p.num_splits, p.Hkv, p.B);
  if (p.ex_fused && p.ex_overlap) {  // programmatic dependent launch: see the kernel's griddepcontrol.wait
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(NTHR);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    rc = check_cuda(cudaLaunchKernelEx(&cfg, kern, p), "decode launch (overlapped)");
    count_launch();
    return rc;
  }
  kern<<<grid, NTHR, smem, stream>>>(p);
  count_launch();
  rc = check_cuda(cudaGetLastError(), "decode launch");
  if (rc || p.ex_fused) return rc;
  dim3 cgrid(p.rows, p.Hkv, p.B);
  const int cthr = p.Dv >= 128 ? 128 : 64;
  if (p.ex_world > 0) {
    publish_partials_kernel<<<cgrid, cthr, 0, stream>>>(p);
    count_launch();
    if ((rc = check_cuda(cudaGetLastError(), "decode publish launch"))) return rc;
    const unsigned rows = (unsigned)((int64_t)p.B * p.Lq * p.Hq);
    if (p.o_is_f32)
      gather_combine_kernel<float><<<rows, cthr, 0, stream>>>(p);
    else
      gather_combine_kernel<T><<<rows, cthr, 0, stream>>>(p);
    count_launch();
    return check_cuda(cudaGetLastError(), "decode gather-combine launch");
  }
  const cudaError_t ce = p.o_is_f32 ? launch_combine_splits<float>(p, stream) : launch_combine_splits<T>(p, stream);
  count_launch();
  return check_cuda(ce, "decode combine launch");
}

}  // namespace

bool decode_fast_supported(const DecodeParams& p, int dtype) {
  if (dtype != PJX_BF16 && dtype != PJX_F16) return false;
  if (p.D != p.Dv || (p.D != 64 && p.D != 128)) return false;
  if (p.rows > 16) return false;
  return true;
}

int decode_coresident_ctas(int dtype, int D, int* out) {
  if (dtype == PJX_BF16) return D == 128 ? coresident_ctas_t<__nv_bfloat16, 128>(out) : coresident_ctas_t<__nv_bfloat16, 64>(out);
  return D == 128 ? coresident_ctas_t<__half, 128>(out) : coresident_ctas_t<__half, 64>(out);
}

int launch_decode(const DecodeParams& p, int dtype, cudaStream_t stream) {
  if (p.B == 0 || p.Hq == 0 || p.Lq == 0) return PJX_OK;
  if (dtype == PJX_BF16) {
    if (p.D == 128) return launch_decode_t<__nv_bfloat16, 128>(p, stream);
    return launch_decode_t<__nv_bfloat16, 64>(p, stream);
  }
  if (p.D == 128) return launch_decode_t<__half, 128>(p, stream);
  return launch_decode_t<__half, 64>(p, stream);
}

// The exact combine of the per-split partials alone (the split kernel of the latent decode writes
// the same partial layout).
int launch_decode_combine(const DecodeParams& p, int dtype, cudaStream_t stream) {
  const cudaError_t ce = p.o_is_f32          ? launch_combine_splits<float>(p, stream)
                         : dtype == PJX_BF16 ? launch_combine_splits<__nv_bfloat16>(p, stream)
                                             : launch_combine_splits<__half>(p, stream);
  count_launch();
  return check_cuda(ce, "decode combine launch");
}

int launch_combine_parts(const float* o_parts, const float* lse_parts, int n_parts, int64_t n_rows,
                         int Dv, void* o, float* lse, int dtype, cudaStream_t stream) {
  if (n_rows == 0) return PJX_OK;
  const int thr = Dv >= 128 ? 128 : 64;
  const unsigned grid = static_cast<unsigned>(n_rows);
  switch (dtype) {
    case PJX_F32:
      combine_parts_kernel<float><<<grid, thr, 0, stream>>>(o_parts, lse_parts, n_parts, n_rows, Dv, static_cast<float*>(o), lse);
      break;
    case PJX_BF16:
      combine_parts_kernel<__nv_bfloat16><<<grid, thr, 0, stream>>>(o_parts, lse_parts, n_parts, n_rows, Dv, static_cast<__nv_bfloat16*>(o), lse);
      break;
    case PJX_F16:
      combine_parts_kernel<__half><<<grid, thr, 0, stream>>>(o_parts, lse_parts, n_parts, n_rows, Dv, static_cast<__half*>(o), lse);
      break;
    default:
      return fail(PJX_ERR_BAD_ARG, "unknown dtype %d", dtype);
  }
  count_launch();
  return check_cuda(cudaGetLastError(), "combine launch");
}


// ---------------------------------------------------------------------------
// Split-KV decode without any allocation by anyone.
//
// Some callers hold no allocator they may use at the moment they need a decode
// step: a serving loop that runs inside a framework's custom-call handler is
// handed its operand and result buffers only (XLA plans every byte ahead of time
// and forbids cudaMalloc inside the handler), and so is code that runs while the
// device allocator is locked or exhausted.  For them the per-split partials live
// in the fixed device array below instead of a workspace argument.
//
// Every device that loads the library reserves the array until the process
// exits, so it is kept modest: 16 MiB holds the partials of the benchmark's
// decode (16 sequences x 8 KV heads x 27 splits x 4 packed rows x 129 floats =
// 7.1 MB) twice over.  Larger calls are rejected, not truncated.
//
// All calls share the one array.  Nothing in it has to start at zero: the combine
// kernel reads exactly the partials that the split kernel of the same call wrote
// (splits past a sequence's length are neither written nor read), so leftovers of
// an earlier call are never looked at.  Two calls whose kernels overlap on the
// GPU (different streams, or different host threads) would overwrite each other's
// partials: callers must order them on one stream.
// ---------------------------------------------------------------------------
namespace {

constexpr size_t kStaticScratchFloats = 4u * 1024u * 1024u;  // 16 MiB
static __device__ __align__(256) float g_decode_scratch[kStaticScratchFloats];

constexpr int kMaxDevices = 64;
float* g_scratch_ptr[kMaxDevices] = {};  // device address of g_decode_scratch, per device

inline size_t round256(size_t x) { return (x + 255) / 256 * 256; }

// The array's name is only a host-side handle; kernels need its device address,
// which differs per device and is looked up once per device with that device
// current.
int static_scratch_address(float** out) {
  int dev = -1;
  int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice");
  if (rc) return rc;
  if (dev < 0 || dev >= kMaxDevices) return fail(PJX_ERR_UNSUPPORTED, "device index %d is beyond the %d supported", dev, kMaxDevices);
  float* p = __atomic_load_n(&g_scratch_ptr[dev], __ATOMIC_ACQUIRE);
  if (!p) {
    void* sym = nullptr;
    rc = check_cuda(cudaGetSymbolAddress(&sym, g_decode_scratch), "cudaGetSymbolAddress(decode scratch)");
    if (rc) return rc;
    if (!sym) return fail(PJX_ERR_CUDA, "cudaGetSymbolAddress returned a null address for the decode scratch");
    p = static_cast<float*>(sym);
    __atomic_store_n(&g_scratch_ptr[dev], p, __ATOMIC_RELEASE);  // every thread computes the same value
  }
  *out = p;
  return PJX_OK;
}

}  // namespace
}  // namespace pjx

extern "C" {

size_t pjx_attn_decode_static_scratch_bytes(void) { return pjx::kStaticScratchFloats * sizeof(float); }

int pjx_attn_decode_splitkv_static(const void* q, const void* k_cache, const void* v_cache,
                                   const int32_t* kv_lengths, void* o, float* lse, int B, int Lq, int Hq,
                                   int Hkv, int D, int Dv, int capacity, int dtype, float sm_scale,
                                   int split_len, void* stream) {
  using namespace pjx;
  if (B < 0 || Lq < 0 || capacity < 0 || Hq < 1 || Hkv < 1 || D < 1 || Dv < 1)
    return fail(PJX_ERR_BAD_ARG, "negative or zero dimension (B=%d Lq=%d capacity=%d Hq=%d Hkv=%d D=%d Dv=%d)", B, Lq, capacity, Hq, Hkv, D, Dv);
  if (Hq % Hkv != 0) return fail(PJX_ERR_BAD_ARG, "query heads %d must be a multiple of kv heads %d", Hq, Hkv);
  if (capacity >= PJX_BAND_NO_UPPER) return fail(PJX_ERR_UNSUPPORTED, "decode: cache capacity must be below 2^30 (got %d)", capacity);
  if (B > 65535 || Hkv > 65535)
    return fail(PJX_ERR_UNSUPPORTED, "decode: at most 65535 sequences and 65535 kv heads per call (got B=%d, Hkv=%d)", B, Hkv);
  if (B == 0 || Lq == 0) return PJX_OK;
  if (!q || !k_cache || !v_cache || !o) return fail(PJX_ERR_BAD_ARG, "q, k_cache, v_cache and o must not be null");
  DecodeParams p;
  p.q = q; p.k = k_cache; p.v = v_cache; p.kv_lengths = kv_lengths; p.o = o; p.lse = lse;
  p.B = B; p.Lq = Lq; p.Hq = Hq; p.Hkv = Hkv; p.D = D; p.Dv = Dv; p.capacity = capacity;
  p.rows = (Hq / Hkv) * Lq;
  p.sm_scale = sm_scale;
  p.o_is_f32 = 0;
  const bool aligned =
      ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache)) & 15) == 0;
  if (!decode_fast_supported(p, dtype) || !aligned || capacity == 0)
    return fail(PJX_ERR_UNSUPPORTED,
                "the allocation-free decode takes bf16/fp16, D = Dv in {64,128}, (Hq/Hkv)*Lq <= 16, capacity > 0 and 16-byte aligned q/k/v");
  if (split_len == 0) split_len = decode_default_split_len(B, Hkv, capacity, kv_lengths != nullptr);
  if (split_len < 64 || split_len % 64 != 0)
    return fail(PJX_ERR_BAD_ARG, "split_len must be a positive multiple of 64 (got %d)", split_len);
  p.split_len = split_len;
  p.num_splits = (capacity + split_len - 1) / split_len;
  const size_t parts = (size_t)B * Hkv * p.num_splits * p.rows;
  const size_t o_bytes = round256(parts * Dv * sizeof(float));
  const size_t need = o_bytes + round256(parts * sizeof(float));
  if (need > kStaticScratchFloats * sizeof(float))
    return fail(PJX_ERR_WORKSPACE,
                "the allocation-free decode holds %zu bytes of partials; this call needs %zu (B=%d Hkv=%d splits=%d rows=%d Dv=%d): "
                "use a larger split_len or pjx_attn_decode_splitkv with a workspace",
                kStaticScratchFloats * sizeof(float), need, B, Hkv, p.num_splits, p.rows, Dv);
  float* scratch = nullptr;
  int rc = static_scratch_address(&scratch);
  if (rc) return rc;
  p.o_part = scratch;
  p.lse_part = reinterpret_cast<float*>(reinterpret_cast<char*>(scratch) + o_bytes);
  return launch_decode(p, dtype, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
