// Generic flash-attention forward: exact fp32 FMA arithmetic on CUDA cores.
//
// Computes any call the C ABI accepts (fp32 / bf16 / fp16, any head width up to
// 256, ragged lengths, causal + key-length masks, dense bias).  It is the kernel
// for fp32 inputs -- tensor cores would round them to TF32, which misses the
// 1e-4 parity bound -- and for shapes the tcgen05 kernel does not take.
//
// Math follows the reference's forward kernel
// (probjax/nn/pallas_kernels/kernels/attention.py:456-529): scores in fp32,
// times sm_scale, plus bias, masked, exp2-domain online softmax, P rounded to the
// input dtype before P.V, final division by the row sum.
//
// One CTA owns a 64-query tile of one (batch, query head) and walks the KV
// sequence in 64-key tiles staged in shared memory as fp32.  Threads form a
// 16 x 16 grid; thread (ty, tx) owns score rows 4*ty..4*ty+3 and columns
// tx + 16*c, and the same rows of the output with columns tx + 16*c.
#include "pjx_common.cuh"

namespace pjx {
namespace {

constexpr int BM = 64;
constexpr int BN = 64;
constexpr int NT = 256;

template <typename T, int NCOL>
__global__ void __launch_bounds__(NT) attn_fwd_generic_kernel(const FwdParams p) {
  extern __shared__ float smem[];
  const int D = p.D, Dv = p.Dv;
  const int Dp = D | 1;    // odd row pitch: conflict-free column walks
  const int Dvp = Dv;      // V rows are read along the row: any pitch works
  float* Qs = smem;                 // [BM][Dp]
  float* Ks = Qs + BM * Dp;         // [BN][Dp]
  float* Vs = Ks + BN * Dp;         // [BN][Dvp]
  float* Ps = Vs + BN * Dvp;        // [BM][BN + 1]

  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int q0 = blockIdx.x * BM, h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.Hq / p.Hkv);
  const T* q = static_cast<const T*>(p.q);
  const T* k = static_cast<const T*>(p.k);
  const T* v = static_cast<const T*>(p.v);

  int kv_len = p.Lkv;
  if (p.kv_lengths) kv_len = max(0, min(kv_len, p.kv_lengths[b]));
  // keys outside [first query + band_lo, last query + band_hi] of the tile are masked for all its rows
  int kv_end = max(0, min(kv_len, min(q0 + BM, p.Lq) + p.band_hi));
  const int kv_begin = (max(0, q0 + p.band_lo) / BN) * BN;
  const bool has_mod = p.mod.on != 0;
  ScoreModView mv = {};
  if (has_mod) {
    mv = view_of(p.mod, b, h, p.Lq);
    kv_end = max(kv_end, min(kv_len, mv.prefix));  // prefix keys are visible to every row
  }

  for (int idx = tid; idx < BM * D; idx += NT) {
    int r = idx / D, d = idx - r * D;
    int qi = q0 + r;
    float x = 0.f;
    if (qi < p.Lq) x = Elem<T>::to_f(q[(((int64_t)b * p.Lq + qi) * p.Hq + h) * D + d]);
    Qs[r * Dp + d] = x;
  }

  float m[4], l[4], acc[4][NCOL];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    m[i] = -INFINITY;
    l[i] = 0.f;
#pragma unroll
    for (int c = 0; c < NCOL; ++c) acc[i][c] = 0.f;
  }
  const float c1 = p.sm_scale * kLog2e;
  const float* bias = nullptr;
  if (p.bias) bias = p.bias + (int64_t)b * p.bias_bs + (int64_t)h * p.bias_hs;

  for (int k0 = kv_begin; k0 < kv_end; k0 += BN) {
    __syncthreads();  // previous tile fully consumed (also orders the Q staging)
    for (int idx = tid; idx < BN * D; idx += NT) {
      int r = idx / D, d = idx - r * D;
      int kj = k0 + r;
      float x = 0.f;
      if (kj < kv_len) x = Elem<T>::to_f(k[(((int64_t)b * p.Lkv + kj) * p.Hkv + hk) * D + d]);
      Ks[r * Dp + d] = x;
    }
    for (int idx = tid; idx < BN * Dv; idx += NT) {
      int r = idx / Dv, d = idx - r * Dv;
      int kj = k0 + r;
      float x = 0.f;
      if (kj < kv_len) x = Elem<T>::to_f(v[(((int64_t)b * p.Lkv + kj) * p.Hkv + hk) * Dv + d]);
      Vs[r * Dvp + d] = x;
    }
    __syncthreads();

    float s[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int c = 0; c < 4; ++c) s[i][c] = 0.f;
    for (int d = 0; d < D; ++d) {
      float qv[4], kv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) qv[i] = Qs[(ty * 4 + i) * Dp + d];
#pragma unroll
      for (int c = 0; c < 4; ++c) kv[c] = Ks[(tx + 16 * c) * Dp + d];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) s[i][c] = fmaf(qv[i], kv[c], s[i][c]);
    }

    // scale -> bias -> mask, in the exp2 domain
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int qi = q0 + ty * 4 + i;
      float tmax = -INFINITY;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int kj = k0 + tx + 16 * c;
        float x = s[i][c] * c1;
        bool keep = kj <= qi + p.band_hi && kj >= qi + p.band_lo;
        if (has_mod && qi < p.Lq && kj < kv_len) {
          x = mod_score<true>(mv, s[i][c] * p.sm_scale, qi, kj, nullptr) * kLog2e;
          keep = mod_keep(mv, keep, qi, kj);
        }
        if (bias && qi < p.Lq && kj < p.Lkv) x = fmaf(bias[(int64_t)qi * p.Lkv + kj], kLog2e, x);
        keep = keep && (kj < kv_len);
        x = keep ? x : -INFINITY;
        s[i][c] = x;
        tmax = fmaxf(tmax, x);
      }
#pragma unroll
      for (int off = 8; off >= 1; off >>= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, off));
      const float m_new = fmaxf(m[i], tmax);
      const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
      const float corr = exp2f(m[i] - m_safe);
      float rsum = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float pv = exp2f(s[i][c] - m_safe);
        rsum += pv;  // the row sum is taken before dropout (kernels/attention.py:497-505)
        const float dm = has_mod ? mod_dropout(mv, qi, k0 + tx + 16 * c) : 1.f;
        Ps[(ty * 4 + i) * (BN + 1) + tx + 16 * c] = Elem<T>::round(pv * dm);
      }
#pragma unroll
      for (int off = 8; off >= 1; off >>= 1) rsum += __shfl_xor_sync(0xffffffffu, rsum, off);
      l[i] = l[i] * corr + rsum;
      m[i] = m_new;
#pragma unroll
      for (int c = 0; c < NCOL; ++c) acc[i][c] *= corr;
    }
    __syncthreads();

    for (int kk = 0; kk < BN; ++kk) {
      float pv[4], vv[NCOL];
#pragma unroll
      for (int i = 0; i < 4; ++i) pv[i] = Ps[(ty * 4 + i) * (BN + 1) + kk];
#pragma unroll
      for (int c = 0; c < NCOL; ++c) {
        const int d = tx + 16 * c;
        vv[c] = d < Dv ? Vs[kk * Dvp + d] : 0.f;
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int c = 0; c < NCOL; ++c) acc[i][c] = fmaf(pv[i], vv[c], acc[i][c]);
    }
  }

  T* o = static_cast<T*>(p.o);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int qi = q0 + ty * 4 + i;
    if (qi >= p.Lq) continue;
    const bool nonempty = l[i] > 0.f;
    const float inv = nonempty ? 1.f / l[i] : 0.f;
#pragma unroll
    for (int c = 0; c < NCOL; ++c) {
      const int d = tx + 16 * c;
      if (d < Dv) o[(((int64_t)b * p.Lq + qi) * p.Hq + h) * Dv + d] = Elem<T>::from_f(acc[i][c] * inv);
    }
    if (p.lse && tx == 0)
      p.lse[((int64_t)b * p.Hq + h) * p.Lq + qi] = nonempty ? (m[i] + log2f(l[i])) * kLn2 : INFINITY;
  }
}

template <typename T, int NCOL>
int launch_t(const FwdParams& p, cudaStream_t stream) {
  const int Dp = p.D | 1;
  size_t smem = sizeof(float) * ((size_t)BM * Dp + (size_t)BN * Dp + (size_t)BN * p.Dv + (size_t)BM * (BN + 1));
  auto kern = attn_fwd_generic_kernel<T, NCOL>;
  if (smem > 48 * 1024) {
    int rc = check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                        "cudaFuncSetAttribute(generic fwd)");
    if (rc) return rc;
  }
  dim3 grid((p.Lq + BM - 1) / BM, p.Hq, p.B);
  kern<<<grid, NT, smem, stream>>>(p);
  count_launch();
  return check_cuda(cudaGetLastError(), "generic forward launch");
}

template <typename T>
int launch_d(const FwdParams& p, cudaStream_t stream) {
  if (p.Dv <= 64) return launch_t<T, 4>(p, stream);
  if (p.Dv <= 128) return launch_t<T, 8>(p, stream);
  return launch_t<T, 16>(p, stream);
}

}  // namespace

int launch_fwd_generic(const FwdParams& p, int dtype, cudaStream_t stream) {
  if (p.D > 256 || p.Dv > 256) return fail(PJX_ERR_UNSUPPORTED, "head dims above 256 are not supported (D=%d, Dv=%d)", p.D, p.Dv);
  if (p.B == 0 || p.Lq == 0 || p.Hq == 0) return PJX_OK;
  switch (dtype) {
    case PJX_F32: return launch_d<float>(p, stream);
    case PJX_BF16: return launch_d<__nv_bfloat16>(p, stream);
    case PJX_F16: return launch_d<__half>(p, stream);
  }
  return fail(PJX_ERR_BAD_ARG, "unknown dtype %d", dtype);
}

}  // namespace pjx
