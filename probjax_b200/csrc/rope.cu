// Interleaved rotary position embedding: pairs (x[2i], x[2i+1]) of the first `rotary_dim`
// elements of every head vector are rotated by the angle pos * base^(-2i / rotary_dim); the rest
// of the vector is copied.  One pass over the tensor, 16-byte accesses: HBM-bound.
//
// Mirrors the reference's rotary layer (probjax/nn/layers/encoding.py:171-211: inverse
// frequencies 1 / base^(2i / rotary_dim), cos / sin of positions x frequencies, even / odd pair
// rotation), which the latent-attention layer applies to the decoupled rotary key
// (probjax/nn/layers/latent_attention.py:424-481).
#include "pjx_common.cuh"

namespace pjx {
namespace {

template <typename T>
struct Vec16;  // 16 bytes of T as floats
template <>
struct Vec16<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const void* p, float (&f)[8]) {
    const float4 v = *static_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
  }
  static __device__ __forceinline__ void store(void* p, const float (&f)[8]) {
    *static_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
  }
};
template <typename T2, typename T1>
struct Vec16Half {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const void* p, float (&f)[8]) {
    const uint4 v = *static_cast<const uint4*>(p);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const T2 h = *reinterpret_cast<const T2*>(&w[i]);
      f[2 * i] = Elem<T1>::to_f(h.x);
      f[2 * i + 1] = Elem<T1>::to_f(h.y);
    }
  }
  static __device__ __forceinline__ void store(void* p, const float (&f)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      T2 h;
      h.x = Elem<T1>::from_f(f[2 * i]);
      h.y = Elem<T1>::from_f(f[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    *static_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  }
};
template <>
struct Vec16<__nv_bfloat16> : Vec16Half<__nv_bfloat162, __nv_bfloat16> {};
template <>
struct Vec16<__half> : Vec16Half<__half2, __half> {};

// x, y: [outer, T, H, D].  A thread owns one 16-byte unit position (t, d0) and walks up to
// kVecsPerThread of the outer * H head vectors that share its angles, so cos / sin are computed
// once per (position, pair) and not once per element.
constexpr int kVecsPerThread = 8;

// x and y may be the same buffer (in-place rotation), so neither is declared restrict.
template <typename T>
__global__ void rope_kernel(const T* x, T* y, const float* __restrict__ positions, float offset,
                            int64_t outer, int T_len, int H, int D, int rotary_dim, float neg_log2_base_2_over_rot) {
  constexpr int N = Vec16<T>::N;
  const int units_per_vec = D / N;
  const int64_t spots = (int64_t)T_len * units_per_vec;
  const int64_t spot = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (spot >= spots) return;
  const int t = (int)(spot / units_per_vec);
  const int d0 = (int)(spot - (int64_t)t * units_per_vec) * N;
  float c[N / 2], sn[N / 2];
  const bool rotates = d0 < rotary_dim;
  if (rotates) {
    const float pos = positions ? positions[t] : (float)t + offset;
#pragma unroll
    for (int i = 0; i < N / 2; ++i) {
      const int pair = d0 / 2 + i;
      c[i] = 1.f;
      sn[i] = 0.f;
      if (2 * pair + 1 < rotary_dim) sincosf(pos * exp2f(neg_log2_base_2_over_rot * (float)pair), &sn[i], &c[i]);
    }
  }
  const int64_t n_vec = outer * H;  // vectors (o, h) that share this thread's (t, d0)
  const int64_t v0 = (int64_t)blockIdx.y * kVecsPerThread;
#pragma unroll 4
  for (int k = 0; k < kVecsPerThread; ++k) {
    const int64_t v = v0 + k;
    if (v >= n_vec) break;
    const int64_t o = v / H, h = v - o * H;
    const int64_t at = (((o * T_len + t) * H + h) * D) + d0;
    float f[8];
    Vec16<T>::load(x + at, f);
    if (rotates) {
#pragma unroll
      for (int i = 0; i < N / 2; ++i) {
        const float e = f[2 * i], od = f[2 * i + 1];
        f[2 * i] = e * c[i] - od * sn[i];
        f[2 * i + 1] = od * c[i] + e * sn[i];
      }
    }
    Vec16<T>::store(y + at, f);
  }
}

template <typename T>
int launch_rope(const void* x, void* y, const float* positions, float offset, int64_t outer, int T_len, int H, int D,
                int rotary_dim, float base, cudaStream_t stream) {
  const int64_t spots = (int64_t)T_len * (D / Vec16<T>::N);
  const int64_t n_vec = outer * H;
  const int threads = 128;
  const int64_t bx = (spots + threads - 1) / threads, by = (n_vec + kVecsPerThread - 1) / kVecsPerThread;
  if (bx > 0x7fffffffLL || by > 65535) return fail(PJX_ERR_UNSUPPORTED, "rope: tensor too large for one launch");
  rope_kernel<T><<<dim3((unsigned)bx, (unsigned)by), threads, 0, stream>>>(
      static_cast<const T*>(x), static_cast<T*>(y), positions, offset, outer, T_len, H, D, rotary_dim,
      -log2f(base) * 2.f / (float)rotary_dim);
  count_launch();
  return check_cuda(cudaGetLastError(), "rope launch");
}

}  // namespace
}  // namespace pjx

extern "C" int pjx_rope_interleaved(const void* x, void* y, const float* positions, float offset, int64_t outer, int T,
                                    int H, int D, int rotary_dim, float base, int dtype, void* stream) {
  using namespace pjx;
  if (dtype != PJX_F32 && dtype != PJX_BF16 && dtype != PJX_F16)
    return fail(PJX_ERR_BAD_ARG, "dtype must be float32, bfloat16 or float16 (got code %d)", dtype);
  if (outer < 0 || T < 0 || H < 1 || D < 1) return fail(PJX_ERR_BAD_ARG, "negative or zero dimension");
  if (rotary_dim < 0 || rotary_dim > D || rotary_dim % 2)
    return fail(PJX_ERR_BAD_ARG, "rotary_dim must be even and at most the head width (got %d for D=%d)", rotary_dim, D);
  if (!(base > 0.f)) return fail(PJX_ERR_BAD_ARG, "base must be positive");
  if (outer == 0 || T == 0) return PJX_OK;
  if (!x || !y) return fail(PJX_ERR_BAD_ARG, "rope: null buffer");
  const int n = dtype == PJX_F32 ? 4 : 8;
  if (D % n || ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15))
    return fail(PJX_ERR_UNSUPPORTED, "rope: head width must be a multiple of %d elements and buffers 16-byte aligned", n);
  if (rotary_dim == 0) rotary_dim = 2;  // nothing rotates; keeps the frequency step finite
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int rot = rotary_dim;
  switch (dtype) {
    case PJX_F32: return launch_rope<float>(x, y, positions, offset, outer, T, H, D, rot, base, st);
    case PJX_BF16: return launch_rope<__nv_bfloat16>(x, y, positions, offset, outer, T, H, D, rot, base, st);
    default: return launch_rope<__half>(x, y, positions, offset, outer, T, H, D, rot, base, st);
  }
}
