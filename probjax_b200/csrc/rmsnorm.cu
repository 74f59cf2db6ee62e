// Root-mean-square normalisation of the rows of x [rows, width]:
//   y = x * rsqrt(mean(x^2) + eps) * scale
// in fp32, stored in the input dtype.  It is the normalisation the latent-attention layer applies
// to the encoded latent before it enters the cache (probjax/nn/layers/latent_attention.py:313-319,
// 435-438: `nnx.RMSNorm(kv_lora_rank)` after `wkv_a`).
//
// HBM bound: one warp per row, 16-byte accesses; the row is read twice (the second read hits
// L1 / L2), so the algorithmic traffic is 2 x rows x width x element size.
#include "pjx_common.cuh"

namespace pjx {
namespace {

template <typename T>
__global__ void __launch_bounds__(128) rms_norm_kernel(const T* x, const float* __restrict__ scale, T* y, int64_t rows,
                                                       int width, float eps) {
  constexpr int VEC = 16 / sizeof(T);
  const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const T* xr = x + row * width;
  T* yr = y + row * width;
  const bool vec_ok = (width % VEC == 0) && ((reinterpret_cast<uintptr_t>(xr) | reinterpret_cast<uintptr_t>(yr)) & 15) == 0;
  float ss = 0.f;
  if (vec_ok) {
    for (int c = lane * VEC; c < width; c += 32 * VEC) {
      const uint4 raw = *reinterpret_cast<const uint4*>(xr + c);
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        const float f = Elem<T>::to_f(e[i]);
        ss = fmaf(f, f, ss);
      }
    }
  } else {
    for (int c = lane; c < width; c += 32) {
      const float f = Elem<T>::to_f(xr[c]);
      ss = fmaf(f, f, ss);
    }
  }
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
  const float r = rsqrtf(ss / (float)width + eps);
  if (vec_ok) {
    for (int c = lane * VEC; c < width; c += 32 * VEC) {
      const uint4 raw = *reinterpret_cast<const uint4*>(xr + c);
      const T* e = reinterpret_cast<const T*>(&raw);
      uint4 out;
      T* o = reinterpret_cast<T*>(&out);
#pragma unroll
      for (int i = 0; i < VEC; ++i) o[i] = Elem<T>::from_f(Elem<T>::to_f(e[i]) * r * (scale ? scale[c + i] : 1.f));
      *reinterpret_cast<uint4*>(yr + c) = out;
    }
  } else {
    for (int c = lane; c < width; c += 32) yr[c] = Elem<T>::from_f(Elem<T>::to_f(xr[c]) * r * (scale ? scale[c] : 1.f));
  }
}

}  // namespace
}  // namespace pjx

using namespace pjx;

extern "C" int pjx_rms_norm(const void* x, const float* scale, void* y, int64_t rows, int width, float eps, int dtype,
                            void* stream) {
  if (dtype != PJX_F32 && dtype != PJX_BF16 && dtype != PJX_F16)
    return fail(PJX_ERR_BAD_ARG, "dtype must be float32, bfloat16 or float16 (got code %d)", dtype);
  if (rows < 0 || width < 1 || !(eps >= 0.f)) return fail(PJX_ERR_BAD_ARG, "rms_norm: rows=%lld width=%d eps=%g", (long long)rows, width, (double)eps);
  if (rows == 0) return PJX_OK;
  if (!x || !y) return fail(PJX_ERR_BAD_ARG, "rms_norm: null buffer");
  if ((rows + 3) / 4 > 2147483647LL) return fail(PJX_ERR_UNSUPPORTED, "rms_norm: too many rows");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)((rows + 3) / 4);
  switch (dtype) {
    case PJX_F32:
      rms_norm_kernel<float><<<grid, 128, 0, st>>>(static_cast<const float*>(x), scale, static_cast<float*>(y), rows, width, eps);
      break;
    case PJX_BF16:
      rms_norm_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>(static_cast<const __nv_bfloat16*>(x), scale,
                                                          static_cast<__nv_bfloat16*>(y), rows, width, eps);
      break;
    default:
      rms_norm_kernel<__half><<<grid, 128, 0, st>>>(static_cast<const __half*>(x), scale, static_cast<__half*>(y), rows, width, eps);
  }
  count_launch();
  return check_cuda(cudaGetLastError(), "rms_norm launch");
}
