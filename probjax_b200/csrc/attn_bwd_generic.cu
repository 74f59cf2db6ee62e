// Flash-attention backward on CUDA cores (exact fp32 arithmetic), any shape the
// generic forward takes: dQ, dK, dV from Q, K, V, O, dO and the forward's natural-log
// LSE, recomputing the probabilities tile by tile (nothing of size Lq x Lkv is stored).
//
// Math of the reference's backward kernels
// (probjax/nn/pallas_kernels/kernels/attention.py:853-906 `_preprocess_backward_kernel`,
// 1189-1483 the split dK/dV and dQ kernels):
//   delta_i = sum_d dO_id O_id
//   P_ij    = exp(s_ij - lse_i),  s_ij = sm_scale q_i.k_j + bias_ij, masked entries 0
//   dV_j   += sum_i P_ij dO_i
//   dS_ij   = P_ij (dO_i.v_j - delta_i)
//   dQ_i   += sm_scale sum_j dS_ij k_j        dK_j += sm_scale sum_i dS_ij q_i
// With GQA, dK and dV of a KV head are summed over the query heads of its group
// (attention.py:2537-2542 restricts the GQA primitives the same way).
//
// Three launches without atomics: delta; dQ (one CTA per 32-query tile, walking the KV
// tiles); dK/dV (one CTA per 32-key tile of a KV head, walking the group's query heads
// and their query tiles).  Threads form a 16 x 16 grid with 2 x 2 micro-tiles of the
// 32 x 32 score tile.
#include "pjx_common.cuh"

namespace pjx {
namespace {

constexpr int T = 32;     // tile edge (queries and keys)
constexpr int NT = 256;   // threads per CTA


template <typename T_>
__global__ void bwd_delta_kernel(const BwdParams p) {
  // one warp per (b, i, h) with i running over the padded length
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x / 32) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int64_t rows = (int64_t)p.B * p.Lq_pad * p.Hq;
  if (row >= rows) return;
  const int h = row % p.Hq;
  const int64_t bi = row / p.Hq;
  const int i = bi % p.Lq_pad, b = bi / p.Lq_pad;
  const int64_t at = ((int64_t)b * p.Hq + h) * p.Lq_pad + i;
  if (i >= p.Lq) {  // padding: rows that contribute nothing
    if (lane == 0) {
      p.delta[at] = 0.f;
      p.lse2[at] = INFINITY;
    }
    return;
  }
  const int64_t src = ((int64_t)b * p.Lq + i) * p.Hq + h;
  const T_* o = static_cast<const T_*>(p.o) + src * p.Dv;
  const T_* d_o = static_cast<const T_*>(p.d_o) + src * p.Dv;
  float acc = 0.f;
  for (int d = lane; d < p.Dv; d += 32) acc = fmaf(Elem<T_>::to_f(o[d]), Elem<T_>::to_f(d_o[d]), acc);
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) {
    p.delta[at] = acc;
    p.lse2[at] = p.lse[((int64_t)b * p.Hq + h) * p.Lq + i] * kLog2e;  // +inf (row without keys) stays +inf
  }
}

// Shared-memory views of one tile step.
struct Tiles {
  float *Qs, *dOs, *Ks, *Vs, *Ps, *dSs, *lse_s, *delta_s;
  int Dp, Dvp;
};

__device__ __forceinline__ Tiles carve(float* smem, int D, int Dv) {
  Tiles t;
  t.Dp = D | 1;
  t.Dvp = Dv | 1;
  t.Qs = smem;
  t.dOs = t.Qs + T * t.Dp;
  t.Ks = t.dOs + T * t.Dvp;
  t.Vs = t.Ks + T * t.Dp;
  t.Ps = t.Vs + T * t.Dvp;
  t.dSs = t.Ps + T * (T + 1);
  t.lse_s = t.dSs + T * (T + 1);
  t.delta_s = t.lse_s + T;
  return t;
}
inline size_t bwd_smem_bytes(int D, int Dv) {
  return sizeof(float) * ((size_t)2 * T * (D | 1) + (size_t)2 * T * (Dv | 1) + 2 * T * (T + 1) + 2 * T);
}

template <typename T_>
__device__ __forceinline__ void load_rows(float* dst, int pitch, const T_* src, int64_t row_stride, int first, int limit,
                                          int width) {
  for (int idx = threadIdx.x; idx < T * width; idx += NT) {
    const int r = idx / width, d = idx - r * width;
    const int g = first + r;
    dst[r * pitch + d] = g < limit ? Elem<T_>::to_f(src[(int64_t)g * row_stride + d]) : 0.f;
  }
}

// P and dS of the 32 x 32 tile (queries q0.., keys k0..) of head h into shared memory.
// Expects Qs, dOs, Ks, Vs, lse_s, delta_s loaded and a barrier passed.
__device__ __forceinline__ void tile_p_ds(const BwdParams& p, const Tiles& t, int b, int h, int q0, int k0, int kv_len) {
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float s[2][2] = {}, dp[2][2] = {};
  for (int d = 0; d < p.D; ++d) {
    const float q0v = t.Qs[(ty * 2) * t.Dp + d], q1v = t.Qs[(ty * 2 + 1) * t.Dp + d];
    const float k0v = t.Ks[tx * t.Dp + d], k1v = t.Ks[(tx + 16) * t.Dp + d];
    s[0][0] = fmaf(q0v, k0v, s[0][0]);
    s[0][1] = fmaf(q0v, k1v, s[0][1]);
    s[1][0] = fmaf(q1v, k0v, s[1][0]);
    s[1][1] = fmaf(q1v, k1v, s[1][1]);
  }
  for (int d = 0; d < p.Dv; ++d) {
    const float a0 = t.dOs[(ty * 2) * t.Dvp + d], a1 = t.dOs[(ty * 2 + 1) * t.Dvp + d];
    const float v0 = t.Vs[tx * t.Dvp + d], v1 = t.Vs[(tx + 16) * t.Dvp + d];
    dp[0][0] = fmaf(a0, v0, dp[0][0]);
    dp[0][1] = fmaf(a0, v1, dp[0][1]);
    dp[1][0] = fmaf(a1, v0, dp[1][0]);
    dp[1][1] = fmaf(a1, v1, dp[1][1]);
  }
  const float* bias = p.bias ? p.bias + (int64_t)b * p.bias_bs + (int64_t)h * p.bias_hs : nullptr;
  const bool has_mod = p.mod.on != 0;
  ScoreModView mv = {};
  if (has_mod) mv = view_of(p.mod, b, h, p.Lq);
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = ty * 2 + i, qi = q0 + r;
    const float lse = t.lse_s[r], delta = t.delta_s[r];
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const int col = tx + 16 * c, kj = k0 + col;
      float x = s[i][c] * p.sm_scale;
      float dsds = 1.f;  // d(modified score) / d(scaled score)
      bool keep = kj <= qi + p.band_hi && kj >= qi + p.band_lo;
      if (has_mod && qi < p.Lq && kj < kv_len) {
        x = mod_score<true>(mv, x, qi, kj, &dsds);
        keep = mod_keep(mv, keep, qi, kj);
      }
      if (bias && qi < p.Lq && kj < p.Lkv) x += bias[(int64_t)qi * p.Lkv + kj];
      keep = keep && qi < p.Lq && kj < kv_len && lse != INFINITY;
      const float pr = keep ? exp2f((x - lse) * kLog2e) : 0.f;
      // dropout: dV sees the dropped, rescaled probabilities and dP is dropped the same way
      // (kernels/attention.py:1038-1039); delta = rowsum(o * do) already includes it
      const float dm = (has_mod && keep) ? mod_dropout(mv, qi, kj) : 1.f;
      t.Ps[r * (T + 1) + col] = pr * dm;
      t.dSs[r * (T + 1) + col] = pr * (dp[i][c] * dm - delta) * dsds;
    }
  }
}

template <typename T_, int NC>  // NC: per-thread columns = ceil(D / 16)
__global__ void __launch_bounds__(NT) bwd_dq_kernel(const BwdParams p) {
  extern __shared__ float smem[];
  const Tiles t = carve(smem, p.D, p.Dv);
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int q0 = blockIdx.x * T, h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.Hq / p.Hkv);
  int kv_len = p.Lkv;
  if (p.kv_lengths) kv_len = max(0, min(kv_len, p.kv_lengths[b]));
  int kv_end = max(0, min(kv_len, min(q0 + T, p.Lq) + p.band_hi));  // keys past the band of the tile's last row
  const int kv_begin = (max(0, q0 + p.band_lo) / T) * T;             // keys before the band of its first row
  if (p.mod.prefix_len) kv_end = max(kv_end, min(kv_len, p.mod.prefix_len[b]));  // prefix keys: visible to every row
  const int64_t qstride = (int64_t)p.Hq * p.D, ostride = (int64_t)p.Hq * p.Dv;
  const int64_t kstride = (int64_t)p.Hkv * p.D, vstride = (int64_t)p.Hkv * p.Dv;
  const T_* q = static_cast<const T_*>(p.q) + ((int64_t)b * p.Lq * p.Hq + h) * p.D;
  const T_* d_o = static_cast<const T_*>(p.d_o) + ((int64_t)b * p.Lq * p.Hq + h) * p.Dv;
  const T_* k = static_cast<const T_*>(p.k) + ((int64_t)b * p.Lkv * p.Hkv + hk) * p.D;
  const T_* v = static_cast<const T_*>(p.v) + ((int64_t)b * p.Lkv * p.Hkv + hk) * p.Dv;
  load_rows<T_>(t.Qs, t.Dp, q, qstride, q0, p.Lq, p.D);
  load_rows<T_>(t.dOs, t.Dvp, d_o, ostride, q0, p.Lq, p.Dv);
  if (threadIdx.x < T) {
    const int qi = q0 + threadIdx.x;
    const int64_t at = ((int64_t)b * p.Hq + h) * p.Lq + qi;
    t.lse_s[threadIdx.x] = qi < p.Lq ? p.lse[at] : INFINITY;
    t.delta_s[threadIdx.x] = qi < p.Lq ? p.delta[((int64_t)b * p.Hq + h) * p.Lq_pad + qi] : 0.f;
  }
  float acc[2][NC];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int c = 0; c < NC; ++c) acc[i][c] = 0.f;
  for (int k0 = kv_begin; k0 < kv_end; k0 += T) {
    __syncthreads();
    load_rows<T_>(t.Ks, t.Dp, k, kstride, k0, kv_len, p.D);
    load_rows<T_>(t.Vs, t.Dvp, v, vstride, k0, kv_len, p.Dv);
    __syncthreads();
    tile_p_ds(p, t, b, h, q0, k0, kv_len);
    __syncthreads();
    if (p.dbias) {  // d(loss)/d(bias_ij) = dS_ij (the bias enters the score unscaled)
      float* db = p.dbias + (int64_t)b * p.bias_bs + (int64_t)h * p.bias_hs;
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int r = ty * 2 + i, col = tx + 16 * c;
          const int qi = q0 + r, kj = k0 + col;
          if (qi < p.Lq && kj < p.Lkv) {
            const float g = t.dSs[r * (T + 1) + col];
            if (p.dbias_atomic) atomicAdd(&db[(int64_t)qi * p.Lkv + kj], g);
            else db[(int64_t)qi * p.Lkv + kj] = g;
          }
        }
    }
    for (int c = 0; c < T; ++c) {
      const float d0 = t.dSs[(ty * 2) * (T + 1) + c], d1 = t.dSs[(ty * 2 + 1) * (T + 1) + c];
#pragma unroll
      for (int cc = 0; cc < NC; ++cc) {
        const int d = tx + 16 * cc;
        const float kv = d < p.D ? t.Ks[c * t.Dp + d] : 0.f;
        acc[0][cc] = fmaf(d0, kv, acc[0][cc]);
        acc[1][cc] = fmaf(d1, kv, acc[1][cc]);
      }
    }
  }
  T_* dq = static_cast<T_*>(p.dq) + ((int64_t)b * p.Lq * p.Hq + h) * p.D;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int qi = q0 + ty * 2 + i;
    if (qi >= p.Lq) continue;
#pragma unroll
    for (int cc = 0; cc < NC; ++cc) {
      const int d = tx + 16 * cc;
      if (d < p.D) dq[(int64_t)qi * qstride + d] = Elem<T_>::from_f(acc[i][cc] * p.sm_scale);
    }
  }
}

template <typename T_, int NCK, int NCV>  // per-thread columns of dK (D) and dV (Dv)
__global__ void __launch_bounds__(NT) bwd_dkdv_kernel(const BwdParams p) {
  extern __shared__ float smem[];
  const Tiles t = carve(smem, p.D, p.Dv);
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int k0 = blockIdx.x * T, hk = blockIdx.y, b = blockIdx.z;
  const int G = p.Hq / p.Hkv;
  int kv_len = p.Lkv;
  if (p.kv_lengths) kv_len = max(0, min(kv_len, p.kv_lengths[b]));
  const int64_t qstride = (int64_t)p.Hq * p.D, ostride = (int64_t)p.Hq * p.Dv;
  const int64_t kstride = (int64_t)p.Hkv * p.D, vstride = (int64_t)p.Hkv * p.Dv;
  const T_* k = static_cast<const T_*>(p.k) + ((int64_t)b * p.Lkv * p.Hkv + hk) * p.D;
  const T_* v = static_cast<const T_*>(p.v) + ((int64_t)b * p.Lkv * p.Hkv + hk) * p.Dv;
  float acck[2][NCK], accv[2][NCV];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
#pragma unroll
    for (int c = 0; c < NCK; ++c) acck[i][c] = 0.f;
#pragma unroll
    for (int c = 0; c < NCV; ++c) accv[i][c] = 0.f;
  }
  if (k0 < kv_len) {  // keys past the valid length get zero gradients
    load_rows<T_>(t.Ks, t.Dp, k, kstride, k0, kv_len, p.D);
    load_rows<T_>(t.Vs, t.Dvp, v, vstride, k0, kv_len, p.Dv);
    // queries outside [first key - band_hi, last key - band_lo] never see a key of this tile
    int q_first = (max(0, k0 - p.band_hi) / T) * T;
    const int q_end = min(p.Lq, k0 + T - p.band_lo);
    if (p.mod.prefix_len && k0 < p.mod.prefix_len[b]) q_first = 0;  // a prefix key is seen by every row
    for (int g = 0; g < G; ++g) {
      const int h = hk * G + g;
      const T_* q = static_cast<const T_*>(p.q) + ((int64_t)b * p.Lq * p.Hq + h) * p.D;
      const T_* d_o = static_cast<const T_*>(p.d_o) + ((int64_t)b * p.Lq * p.Hq + h) * p.Dv;
      for (int q0 = q_first; q0 < q_end; q0 += T) {
        __syncthreads();
        load_rows<T_>(t.Qs, t.Dp, q, qstride, q0, p.Lq, p.D);
        load_rows<T_>(t.dOs, t.Dvp, d_o, ostride, q0, p.Lq, p.Dv);
        if (threadIdx.x < T) {
          const int qi = q0 + threadIdx.x;
          const int64_t at = ((int64_t)b * p.Hq + h) * p.Lq + qi;
          t.lse_s[threadIdx.x] = qi < p.Lq ? p.lse[at] : INFINITY;
          t.delta_s[threadIdx.x] = qi < p.Lq ? p.delta[((int64_t)b * p.Hq + h) * p.Lq_pad + qi] : 0.f;
        }
        __syncthreads();
        tile_p_ds(p, t, b, h, q0, k0, kv_len);
        __syncthreads();
        for (int r = 0; r < T; ++r) {
          const float p0 = t.Ps[r * (T + 1) + ty * 2], p1 = t.Ps[r * (T + 1) + ty * 2 + 1];
          const float s0 = t.dSs[r * (T + 1) + ty * 2], s1 = t.dSs[r * (T + 1) + ty * 2 + 1];
#pragma unroll
          for (int cc = 0; cc < NCV; ++cc) {
            const int d = tx + 16 * cc;
            const float g_o = d < p.Dv ? t.dOs[r * t.Dvp + d] : 0.f;
            accv[0][cc] = fmaf(p0, g_o, accv[0][cc]);
            accv[1][cc] = fmaf(p1, g_o, accv[1][cc]);
          }
#pragma unroll
          for (int cc = 0; cc < NCK; ++cc) {
            const int d = tx + 16 * cc;
            const float qv = d < p.D ? t.Qs[r * t.Dp + d] : 0.f;
            acck[0][cc] = fmaf(s0, qv, acck[0][cc]);
            acck[1][cc] = fmaf(s1, qv, acck[1][cc]);
          }
        }
      }
    }
  }
  T_* dk = static_cast<T_*>(p.dk) + ((int64_t)b * p.Lkv * p.Hkv + hk) * p.D;
  T_* dv = static_cast<T_*>(p.dv) + ((int64_t)b * p.Lkv * p.Hkv + hk) * p.Dv;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int kj = k0 + ty * 2 + i;
    if (kj >= p.Lkv) continue;
#pragma unroll
    for (int cc = 0; cc < NCK; ++cc) {
      const int d = tx + 16 * cc;
      if (d < p.D) dk[(int64_t)kj * kstride + d] = Elem<T_>::from_f(acck[i][cc] * p.sm_scale);
    }
#pragma unroll
    for (int cc = 0; cc < NCV; ++cc) {
      const int d = tx + 16 * cc;
      if (d < p.Dv) dv[(int64_t)kj * vstride + d] = Elem<T_>::from_f(accv[i][cc]);
    }
  }
}

template <typename K>
int set_smem(K kern, size_t bytes, const char* what) {
  if (bytes <= 48 * 1024) return PJX_OK;
  return check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes), what);
}

template <typename T_, int NCK, int NCV>
int launch_widths(const BwdParams& p, cudaStream_t stream) {
  const size_t smem = bwd_smem_bytes(p.D, p.Dv);
  int rc;
  const int64_t rows = (int64_t)p.B * p.Lq_pad * p.Hq;
  bwd_delta_kernel<T_><<<(unsigned)((rows + 7) / 8), 256, 0, stream>>>(p);
  count_launch();
  if ((rc = check_cuda(cudaGetLastError(), "backward delta launch"))) return rc;
  if (p.use_sm100) return launch_bwd_sm100(p, stream);
  auto kq = bwd_dq_kernel<T_, NCK>;
  if ((rc = set_smem(kq, smem, "cudaFuncSetAttribute(backward dq)"))) return rc;
  kq<<<dim3((p.Lq + T - 1) / T, p.Hq, p.B), NT, smem, stream>>>(p);
  count_launch();
  if ((rc = check_cuda(cudaGetLastError(), "backward dq launch"))) return rc;
  if (p.Lkv == 0) return PJX_OK;
  auto kk = bwd_dkdv_kernel<T_, NCK, NCV>;
  if ((rc = set_smem(kk, smem, "cudaFuncSetAttribute(backward dk/dv)"))) return rc;
  kk<<<dim3((p.Lkv + T - 1) / T, p.Hkv, p.B), NT, smem, stream>>>(p);
  count_launch();
  return check_cuda(cudaGetLastError(), "backward dk/dv launch");
}

template <typename T_>
int launch_dtype(const BwdParams& p, cudaStream_t stream) {
  const int nk = p.D <= 64 ? 4 : (p.D <= 128 ? 8 : 16);
  const int nv = p.Dv <= 64 ? 4 : (p.Dv <= 128 ? 8 : 16);
  switch (nk * 100 + nv) {
    case 404: return launch_widths<T_, 4, 4>(p, stream);
    case 408: return launch_widths<T_, 4, 8>(p, stream);
    case 416: return launch_widths<T_, 4, 16>(p, stream);
    case 804: return launch_widths<T_, 8, 4>(p, stream);
    case 808: return launch_widths<T_, 8, 8>(p, stream);
    case 816: return launch_widths<T_, 8, 16>(p, stream);
    case 1604: return launch_widths<T_, 16, 4>(p, stream);
    case 1608: return launch_widths<T_, 16, 8>(p, stream);
    default: return launch_widths<T_, 16, 16>(p, stream);
  }
}


// ---------------------------------------------------------------------------------------------
// Forward-mode derivative (JVP) from the saved log-sum-exp, the reference's
// `mha_jvp_from_lse_kernel` (kernels/attention.py:536-660): with tangents tq, tk, tv,
//   ds_ij = sm_scale (tq_i.k_j + q_i.tk_j)            (masked entries 0)
//   to_i  = sum_j P_ij ds_ij v_j + sum_j P_ij tv_j - (sum_j P_ij ds_ij) o_i,   o_i = sum_j P_ij v_j
// One CTA per 32-query tile of a (batch, head), walking the KV tiles once; P and P ds are rounded
// to the input dtype before the products with v / tv, as the reference does.
// ---------------------------------------------------------------------------------------------
struct JvpParams {
  const void *q, *k, *v, *tq, *tk, *tv;  // tangents may be null (zero)
  const float* lse;
  void* t_o;
  const int32_t* kv_lengths;
  const float* bias;
  int64_t bias_bs, bias_hs;
  int B, Lq, Lkv, Hq, Hkv, D, Dv;
  int band_lo, band_hi;
  float sm_scale;
  ScoreMod mod;
};

inline size_t jvp_smem_bytes(int D, int Dv) {
  return sizeof(float) * ((size_t)4 * T * (D | 1) + (size_t)2 * T * (Dv | 1) + 2 * T * (T + 1) + T);
}

template <typename T_>
__device__ __forceinline__ void load_rows_or_zero(float* dst, int pitch, const T_* src, int64_t row_stride, int first,
                                                  int limit, int width) {
  if (src) {
    load_rows<T_>(dst, pitch, src, row_stride, first, limit, width);
  } else {
    for (int idx = threadIdx.x; idx < T * width; idx += NT) dst[(idx / width) * pitch + idx % width] = 0.f;
  }
}

template <typename T_, int NC>  // NC: per-thread output columns = ceil(Dv / 16)
__global__ void __launch_bounds__(NT) jvp_kernel(const JvpParams p) {
  extern __shared__ float smem[];
  const int Dp = p.D | 1, Dvp = p.Dv | 1;
  float* Qs = smem;                 // [T][Dp]
  float* tQs = Qs + T * Dp;
  float* Ks = tQs + T * Dp;
  float* tKs = Ks + T * Dp;
  float* Vs = tKs + T * Dp;         // [T][Dvp]
  float* tVs = Vs + T * Dvp;
  float* Ps = tVs + T * Dvp;        // [T][T + 1]  P
  float* PDs = Ps + T * (T + 1);    // [T][T + 1]  P ds
  float* lse_s = PDs + T * (T + 1);
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int q0 = blockIdx.x * T, h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.Hq / p.Hkv);
  int kv_len = p.Lkv;
  if (p.kv_lengths) kv_len = max(0, min(kv_len, p.kv_lengths[b]));
  int kv_end = max(0, min(kv_len, min(q0 + T, p.Lq) + p.band_hi));
  const int kv_begin = (max(0, q0 + p.band_lo) / T) * T;
  const bool has_mod = p.mod.on != 0;
  ScoreModView mv = {};
  if (has_mod) {
    mv = view_of(p.mod, b, h, p.Lq);
    kv_end = max(kv_end, min(kv_len, mv.prefix));
  }
  const int64_t qstride = (int64_t)p.Hq * p.D, ostride = (int64_t)p.Hq * p.Dv;
  const int64_t kstride = (int64_t)p.Hkv * p.D, vstride = (int64_t)p.Hkv * p.Dv;
  const int64_t qoff = ((int64_t)b * p.Lq * p.Hq + h) * p.D;
  const int64_t koff = ((int64_t)b * p.Lkv * p.Hkv + hk) * p.D, voff = ((int64_t)b * p.Lkv * p.Hkv + hk) * p.Dv;
  const T_* q = static_cast<const T_*>(p.q) + qoff;
  const T_* tq = p.tq ? static_cast<const T_*>(p.tq) + qoff : nullptr;
  const T_* k = static_cast<const T_*>(p.k) + koff;
  const T_* tk = p.tk ? static_cast<const T_*>(p.tk) + koff : nullptr;
  const T_* v = static_cast<const T_*>(p.v) + voff;
  const T_* tv = p.tv ? static_cast<const T_*>(p.tv) + voff : nullptr;
  load_rows<T_>(Qs, Dp, q, qstride, q0, p.Lq, p.D);
  load_rows_or_zero<T_>(tQs, Dp, tq, qstride, q0, p.Lq, p.D);
  if (threadIdx.x < T) {
    const int qi = q0 + threadIdx.x;
    lse_s[threadIdx.x] = qi < p.Lq ? p.lse[((int64_t)b * p.Hq + h) * p.Lq + qi] : INFINITY;
  }
  const float* bias = p.bias ? p.bias + (int64_t)b * p.bias_bs + (int64_t)h * p.bias_hs : nullptr;
  float acc[2][NC], out[2][NC], mu[2] = {0.f, 0.f};
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int c = 0; c < NC; ++c) acc[i][c] = out[i][c] = 0.f;

  for (int k0 = kv_begin; k0 < kv_end; k0 += T) {
    __syncthreads();
    load_rows<T_>(Ks, Dp, k, kstride, k0, kv_len, p.D);
    load_rows_or_zero<T_>(tKs, Dp, tk, kstride, k0, kv_len, p.D);
    load_rows<T_>(Vs, Dvp, v, vstride, k0, kv_len, p.Dv);
    load_rows_or_zero<T_>(tVs, Dvp, tv, vstride, k0, kv_len, p.Dv);
    __syncthreads();
    float s[2][2] = {}, ds[2][2] = {};
    for (int d = 0; d < p.D; ++d) {
      const float qa = Qs[(ty * 2) * Dp + d], qb = Qs[(ty * 2 + 1) * Dp + d];
      const float ta = tQs[(ty * 2) * Dp + d], tb = tQs[(ty * 2 + 1) * Dp + d];
      const float ka = Ks[tx * Dp + d], kb = Ks[(tx + 16) * Dp + d];
      const float ua = tKs[tx * Dp + d], ub = tKs[(tx + 16) * Dp + d];
      s[0][0] = fmaf(qa, ka, s[0][0]);
      s[0][1] = fmaf(qa, kb, s[0][1]);
      s[1][0] = fmaf(qb, ka, s[1][0]);
      s[1][1] = fmaf(qb, kb, s[1][1]);
      ds[0][0] = fmaf(ta, ka, fmaf(qa, ua, ds[0][0]));
      ds[0][1] = fmaf(ta, kb, fmaf(qa, ub, ds[0][1]));
      ds[1][0] = fmaf(tb, ka, fmaf(qb, ua, ds[1][0]));
      ds[1][1] = fmaf(tb, kb, fmaf(qb, ub, ds[1][1]));
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int r = ty * 2 + i, qi = q0 + r;
      const float lse = lse_s[r];
      float part = 0.f;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int col = tx + 16 * c, kj = k0 + col;
        float x = s[i][c] * p.sm_scale;
        float dsds = 1.f;
        bool keep = kj <= qi + p.band_hi && kj >= qi + p.band_lo;
        if (has_mod && qi < p.Lq && kj < kv_len) {
          x = mod_score<true>(mv, x, qi, kj, &dsds);
          keep = mod_keep(mv, keep, qi, kj);
        }
        if (bias && qi < p.Lq && kj < p.Lkv) x += bias[(int64_t)qi * p.Lkv + kj];
        keep = keep && qi < p.Lq && kj < kv_len && lse != INFINITY;
        const float pr = keep ? exp2f((x - lse) * kLog2e) : 0.f;
        const float pd = keep ? pr * ds[i][c] * p.sm_scale * dsds : 0.f;
        part += pd;  // sum of p ds without dropout: the derivative of the normaliser
        const float dm = (has_mod && keep) ? mod_dropout(mv, qi, kj) : 1.f;
        Ps[r * (T + 1) + col] = Elem<T_>::round(pr * dm);
        PDs[r * (T + 1) + col] = Elem<T_>::round(pd * dm);
      }
#pragma unroll
      for (int off = 8; off >= 1; off >>= 1) part += __shfl_xor_sync(0xffffffffu, part, off);
      mu[i] += part;  // the 16 threads of a row hold the same sum
    }
    __syncthreads();
    for (int c = 0; c < T; ++c) {
      const float p0 = Ps[(ty * 2) * (T + 1) + c], p1 = Ps[(ty * 2 + 1) * (T + 1) + c];
      const float e0 = PDs[(ty * 2) * (T + 1) + c], e1 = PDs[(ty * 2 + 1) * (T + 1) + c];
#pragma unroll
      for (int cc = 0; cc < NC; ++cc) {
        const int d = tx + 16 * cc;
        const float vv = d < p.Dv ? Vs[c * Dvp + d] : 0.f;
        const float tvv = d < p.Dv ? tVs[c * Dvp + d] : 0.f;
        acc[0][cc] = fmaf(e0, vv, fmaf(p0, tvv, acc[0][cc]));
        acc[1][cc] = fmaf(e1, vv, fmaf(p1, tvv, acc[1][cc]));
        out[0][cc] = fmaf(p0, vv, out[0][cc]);
        out[1][cc] = fmaf(p1, vv, out[1][cc]);
      }
    }
  }
  T_* t_o = static_cast<T_*>(p.t_o) + ((int64_t)b * p.Lq * p.Hq + h) * p.Dv;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int qi = q0 + ty * 2 + i;
    if (qi >= p.Lq) continue;
#pragma unroll
    for (int cc = 0; cc < NC; ++cc) {
      const int d = tx + 16 * cc;
      if (d < p.Dv) t_o[(int64_t)qi * ostride + d] = Elem<T_>::from_f(acc[i][cc] - mu[i] * out[i][cc]);
    }
  }
}

template <typename T_, int NC>
int launch_jvp_width(const JvpParams& p, cudaStream_t stream) {
  const size_t smem = jvp_smem_bytes(p.D, p.Dv);
  auto kern = jvp_kernel<T_, NC>;
  int rc;
  if ((rc = set_smem(kern, smem, "cudaFuncSetAttribute(jvp)"))) return rc;
  kern<<<dim3((p.Lq + T - 1) / T, p.Hq, p.B), NT, smem, stream>>>(p);
  count_launch();
  return check_cuda(cudaGetLastError(), "jvp launch");
}

template <typename T_>
int launch_jvp(const JvpParams& p, cudaStream_t stream) {
  if (p.Dv <= 64) return launch_jvp_width<T_, 4>(p, stream);
  if (p.Dv <= 128) return launch_jvp_width<T_, 8>(p, stream);
  return launch_jvp_width<T_, 16>(p, stream);
}

}  // namespace
}  // namespace pjx

using namespace pjx;

extern "C" {

size_t pjx_attn_bwd_workspace_bytes(int B, int Lq, int Hq) {
  if (B < 0 || Lq < 0 || Hq < 1) return 0;
  const size_t lq_pad = ((size_t)Lq + 127) / 128 * 128;  // two float arrays [B, Hq, lq_pad]
  return 2 * (size_t)B * Hq * lq_pad * sizeof(float);
}

int pjx_attn_bwd_band(const void* q, const void* k, const void* v, const void* o, const float* lse, const void* d_o,
                      void* dq, void* dk, void* dv, const int32_t* kv_lengths, const float* bias,
                      int64_t bias_batch_stride, int64_t bias_head_stride, float* dbias, int B, int Lq, int Lkv, int Hq,
                      int Hkv, int D, int Dv, int dtype, int band_lo, int band_hi, float sm_scale, int impl,
                      void* workspace, size_t workspace_bytes, int32_t* status, void* stream) {
  return pjx_attn_bwd_mod(q, k, v, o, lse, d_o, dq, dk, dv, kv_lengths, bias, bias_batch_stride, bias_head_stride, dbias,
                          B, Lq, Lkv, Hq, Hkv, D, Dv, dtype, band_lo, band_hi, sm_scale, nullptr, impl, workspace,
                          workspace_bytes, status, stream);
}

int pjx_attn_bwd_mod(const void* q, const void* k, const void* v, const void* o, const float* lse, const void* d_o,
                     void* dq, void* dk, void* dv, const int32_t* kv_lengths, const float* bias,
                     int64_t bias_batch_stride, int64_t bias_head_stride, float* dbias, int B, int Lq, int Lkv, int Hq,
                     int Hkv, int D, int Dv, int dtype, int band_lo, int band_hi, float sm_scale,
                     const pjx_score_mod* mod, int impl, void* workspace, size_t workspace_bytes, int32_t* status,
                     void* stream) {
  ScoreMod smod;
  {
    int rcm = convert_score_mod(mod, &smod);
    if (rcm) return rcm;
  }
  if (dbias && smod.nonlinear())
    return fail(PJX_ERR_UNSUPPORTED, "backward: the bias gradient is not computed together with head_scale / softcap");
  if (impl != PJX_IMPL_AUTO && impl != PJX_IMPL_GENERIC && impl != PJX_IMPL_SM100)
    return fail(PJX_ERR_BAD_ARG, "impl must be 0 (auto), 1 (generic) or 2 (tcgen05), got %d", impl);
  if (dtype != PJX_F32 && dtype != PJX_BF16 && dtype != PJX_F16)
    return fail(PJX_ERR_BAD_ARG, "dtype must be float32, bfloat16 or float16 (got code %d)", dtype);
  if (B < 0 || Lq < 0 || Lkv < 0 || Hq < 1 || Hkv < 1 || D < 1 || Dv < 1)
    return fail(PJX_ERR_BAD_ARG, "negative or zero dimension");
  if (Hq % Hkv != 0) return fail(PJX_ERR_BAD_ARG, "query heads %d must be a multiple of kv heads %d", Hq, Hkv);
  if (D > 256 || Dv > 256) return fail(PJX_ERR_UNSUPPORTED, "head dims above 256 are not supported (D=%d, Dv=%d)", D, Dv);
  if (Lq >= PJX_BAND_NO_UPPER || Lkv >= PJX_BAND_NO_UPPER)
    return fail(PJX_ERR_BAD_ARG, "sequence lengths must be below 2^30");
  if (B == 0 || Hq == 0) return PJX_OK;
  if (Lq > 0 && (!q || !o || !d_o || !lse || !dq)) return fail(PJX_ERR_BAD_ARG, "backward: null query-side buffer");
  if (Lkv > 0 && (!k || !v || !dk || !dv)) return fail(PJX_ERR_BAD_ARG, "backward: null key-side buffer");
  const size_t need = pjx_attn_bwd_workspace_bytes(B, Lq, Hq);
  if (Lq > 0 && (!workspace || workspace_bytes < need))
    return fail(PJX_ERR_WORKSPACE, "backward workspace: need %zu bytes, got %zu", need, workspace ? workspace_bytes : (size_t)0);
  if (Lq == 0 && Lkv == 0) return PJX_OK;
  BwdParams p;
  p.q = q; p.k = k; p.v = v; p.o = o; p.d_o = d_o; p.lse = lse;
  p.Lq_pad = (Lq + 127) / 128 * 128;
  p.delta = static_cast<float*>(workspace);
  p.lse2 = p.delta + (size_t)B * Hq * p.Lq_pad;
  p.dq = dq; p.dk = dk; p.dv = dv;
  p.kv_lengths = kv_lengths; p.bias = bias; p.bias_bs = bias_batch_stride; p.bias_hs = bias_head_stride;
  p.B = B; p.Lq = Lq; p.Lkv = Lkv; p.Hq = Hq; p.Hkv = Hkv; p.D = D; p.Dv = Dv;
  p.band_lo = band_lo < PJX_BAND_NO_LOWER ? PJX_BAND_NO_LOWER : (band_lo > PJX_BAND_NO_UPPER ? PJX_BAND_NO_UPPER : band_lo);
  p.band_hi = band_hi > PJX_BAND_NO_UPPER ? PJX_BAND_NO_UPPER : (band_hi < PJX_BAND_NO_LOWER ? PJX_BAND_NO_LOWER : band_hi);
  p.sm_scale = sm_scale;
  p.dtype = dtype;
  p.status = status;
  p.mod = smod;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dbias) {
    if (!bias) return fail(PJX_ERR_BAD_ARG, "backward: dbias given without a bias");
    if (bias_batch_stride < 0 || bias_head_stride < 0) return fail(PJX_ERR_BAD_ARG, "bias strides must be non-negative");
    // the bias is [Bb, Hb, Lq, Lkv] with Bb in {1, B}, Hb in {1, Hq}: its extent follows from the strides
    const int64_t hb = bias_head_stride ? Hq : 1, bbn = bias_batch_stride ? B : 1;
    int rc0 = check_cuda(cudaMemsetAsync(dbias, 0, (size_t)bbn * hb * Lq * Lkv * sizeof(float), st), "clear dbias");
    if (rc0) return rc0;
    p.dbias = dbias;
    p.dbias_atomic = (bias_batch_stride == 0 && B > 1) || (bias_head_stride == 0 && Hq > 1);
  }
  if (Lq == 0) {  // no queries: the key-side gradients are zero
    int rc = check_cuda(cudaMemsetAsync(dk, 0, (size_t)B * Lkv * Hkv * D * dtype_size(dtype), st), "clear dk");
    if (rc) return rc;
    return check_cuda(cudaMemsetAsync(dv, 0, (size_t)B * Lkv * Hkv * Dv * dtype_size(dtype), st), "clear dv");
  }
  const char* why = nullptr;
  bool tc_ok = bwd_sm100_supported(p, &why);
  if (tc_ok && smod.on) {
    tc_ok = false;
    why = "score modifiers are evaluated by the CUDA-core backward only";
  }
  if (impl == PJX_IMPL_SM100 && !tc_ok) return fail(PJX_ERR_UNSUPPORTED, "tcgen05 backward: %s", why);
  p.use_sm100 = impl != PJX_IMPL_GENERIC && tc_ok;
  switch (dtype) {
    case PJX_F32: return launch_dtype<float>(p, st);
    case PJX_BF16: return launch_dtype<__nv_bfloat16>(p, st);
    default: return launch_dtype<__half>(p, st);
  }
}

int pjx_attn_bwd(const void* q, const void* k, const void* v, const void* o, const float* lse, const void* d_o,
                 void* dq, void* dk, void* dv, const int32_t* kv_lengths, const float* bias,
                 int64_t bias_batch_stride, int64_t bias_head_stride, int B, int Lq, int Lkv, int Hq, int Hkv, int D,
                 int Dv, int dtype, int causal, float sm_scale, void* workspace, size_t workspace_bytes, void* stream) {
  return pjx_attn_bwd_band(q, k, v, o, lse, d_o, dq, dk, dv, kv_lengths, bias, bias_batch_stride, bias_head_stride,
                           nullptr, B, Lq, Lkv, Hq, Hkv, D, Dv, dtype, PJX_BAND_NO_LOWER, causal ? 0 : PJX_BAND_NO_UPPER, sm_scale,
                           PJX_IMPL_AUTO, workspace, workspace_bytes, nullptr, stream);
}

int pjx_attn_jvp_band(const void* q, const void* k, const void* v, const void* tq, const void* tk, const void* tv,
                      const float* lse, void* t_o, const int32_t* kv_lengths, const float* bias,
                      int64_t bias_batch_stride, int64_t bias_head_stride, int B, int Lq, int Lkv, int Hq, int Hkv,
                      int D, int Dv, int dtype, int band_lo, int band_hi, float sm_scale, void* stream) {
  return pjx_attn_jvp_mod(q, k, v, tq, tk, tv, lse, t_o, kv_lengths, bias, bias_batch_stride, bias_head_stride, B, Lq, Lkv,
                          Hq, Hkv, D, Dv, dtype, band_lo, band_hi, sm_scale, nullptr, stream);
}

int pjx_attn_jvp_mod(const void* q, const void* k, const void* v, const void* tq, const void* tk, const void* tv,
                     const float* lse, void* t_o, const int32_t* kv_lengths, const float* bias,
                     int64_t bias_batch_stride, int64_t bias_head_stride, int B, int Lq, int Lkv, int Hq, int Hkv,
                     int D, int Dv, int dtype, int band_lo, int band_hi, float sm_scale, const pjx_score_mod* mod,
                     void* stream) {
  ScoreMod smod;
  {
    int rcm = convert_score_mod(mod, &smod);
    if (rcm) return rcm;
  }
  if (dtype != PJX_F32 && dtype != PJX_BF16 && dtype != PJX_F16)
    return fail(PJX_ERR_BAD_ARG, "dtype must be float32, bfloat16 or float16 (got code %d)", dtype);
  if (B < 0 || Lq < 0 || Lkv < 0 || Hq < 1 || Hkv < 1 || D < 1 || Dv < 1)
    return fail(PJX_ERR_BAD_ARG, "negative or zero dimension");
  if (Hq % Hkv != 0) return fail(PJX_ERR_BAD_ARG, "query heads %d must be a multiple of kv heads %d", Hq, Hkv);
  if (D > 256 || Dv > 256) return fail(PJX_ERR_UNSUPPORTED, "head dims above 256 are not supported (D=%d, Dv=%d)", D, Dv);
  if (Lq >= PJX_BAND_NO_UPPER || Lkv >= PJX_BAND_NO_UPPER)
    return fail(PJX_ERR_BAD_ARG, "sequence lengths must be below 2^30");
  if (B == 0 || Lq == 0) return PJX_OK;
  if (!q || !lse || !t_o || (Lkv > 0 && (!k || !v))) return fail(PJX_ERR_BAD_ARG, "jvp: null buffer");
  JvpParams p;
  p.q = q; p.k = k; p.v = v; p.tq = tq; p.tk = tk; p.tv = tv; p.lse = lse; p.t_o = t_o;
  p.kv_lengths = kv_lengths; p.bias = bias; p.bias_bs = bias_batch_stride; p.bias_hs = bias_head_stride;
  p.B = B; p.Lq = Lq; p.Lkv = Lkv; p.Hq = Hq; p.Hkv = Hkv; p.D = D; p.Dv = Dv;
  p.band_lo = band_lo < PJX_BAND_NO_LOWER ? PJX_BAND_NO_LOWER : (band_lo > PJX_BAND_NO_UPPER ? PJX_BAND_NO_UPPER : band_lo);
  p.band_hi = band_hi > PJX_BAND_NO_UPPER ? PJX_BAND_NO_UPPER : (band_hi < PJX_BAND_NO_LOWER ? PJX_BAND_NO_LOWER : band_hi);
  p.sm_scale = sm_scale;
  p.mod = smod;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case PJX_F32: return launch_jvp<float>(p, st);
    case PJX_BF16: return launch_jvp<__nv_bfloat16>(p, st);
    default: return launch_jvp<__half>(p, st);
  }
}

}  // extern "C"
