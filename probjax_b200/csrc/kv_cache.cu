// Decode KV-cache update: the new tokens' keys and values are written at each sequence's
// current position and the positions advance, in one launch and without a host round trip,
// so a decode step (append, then split-KV attention over `positions`) can be captured in a
// CUDA graph.
//
// Mirrors the cache update of the reference's attention layer
// (probjax/nn/layers/attention.py:631-643: `lax.dynamic_update_slice` of `cached_key` /
// `cached_value` at `cache_index`, then `cache_index += 1`), with one position per sequence
// instead of one shared index, which is what a ragged batch needs.
#include "pjx_common.cuh"

namespace pjx {
namespace {

// One thread per 16-byte unit of the new rows: [B, n_new, Hkv * Dim] -> cache row positions[b] + t.
__global__ void kv_append_kernel(uint4* __restrict__ k_cache, uint4* __restrict__ v_cache, const uint4* __restrict__ k_new,
                                 const uint4* __restrict__ v_new, int32_t* __restrict__ positions, int B, int capacity,
                                 int n_new, int k_units, int v_units, int advance, int32_t* __restrict__ overflow) {
  const int b = blockIdx.y;
  const int pos = positions[b];
  const int64_t per_b = (int64_t)n_new * (k_units + v_units);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < per_b; i += (int64_t)gridDim.x * blockDim.x) {
    const int t = (int)(i / (k_units + v_units));
    const int u = (int)(i - (int64_t)t * (k_units + v_units));
    const int row = pos + t;
    if (row < 0 || row >= capacity) continue;  // rows past the capacity are dropped and reported
    if (u < k_units)
      k_cache[((int64_t)b * capacity + row) * k_units + u] = k_new[((int64_t)b * n_new + t) * k_units + u];
    else
      v_cache[((int64_t)b * capacity + row) * v_units + (u - k_units)] = v_new[((int64_t)b * n_new + t) * v_units + (u - k_units)];
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    if (overflow && (pos < 0 || pos + n_new > capacity)) atomicExch(overflow, 1);
  }
  // positions advance after every block of this sequence has read them: the last block to finish does it
  if (advance) {
    __shared__ int last;
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      // the counter lives in the top bits' neighbour word: positions[B + b]
      last = atomicAdd(&positions[B + b], 1) == (int)gridDim.x - 1;
    }
    __syncthreads();
    if (last && threadIdx.x == 0) {
      positions[B + b] = 0;
      positions[b] = min(pos + n_new, capacity);
    }
  }
}

}  // namespace
}  // namespace pjx

extern "C" int pjx_kv_cache_append(void* k_cache, void* v_cache, const void* k_new, const void* v_new, int32_t* positions,
                                   int B, int capacity, int n_new, int Hkv, int D, int Dv, int dtype, int advance,
                                   int32_t* overflow, void* stream) {
  using namespace pjx;
  if (dtype != PJX_F32 && dtype != PJX_BF16 && dtype != PJX_F16)
    return fail(PJX_ERR_BAD_ARG, "dtype must be float32, bfloat16 or float16 (got code %d)", dtype);
  if (B < 0 || capacity < 0 || n_new < 0 || Hkv < 1 || D < 1 || Dv < 1) return fail(PJX_ERR_BAD_ARG, "negative or zero dimension");
  if (B == 0 || n_new == 0) return PJX_OK;
  if (!k_cache || !v_cache || !k_new || !v_new || !positions) return fail(PJX_ERR_BAD_ARG, "kv cache append: null buffer");
  const size_t es = dtype_size(dtype);
  if ((Hkv * D * es) % 16 || (Hkv * Dv * es) % 16)
    return fail(PJX_ERR_UNSUPPORTED, "kv cache append: a token's keys and values must be multiples of 16 bytes");
  if ((reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache) | reinterpret_cast<uintptr_t>(k_new) |
       reinterpret_cast<uintptr_t>(v_new)) & 15)
    return fail(PJX_ERR_UNSUPPORTED, "kv cache append: buffers must be 16-byte aligned");
  if (B > 65535) return fail(PJX_ERR_UNSUPPORTED, "kv cache append: batch above 65535");
  const int k_units = (int)(Hkv * D * es / 16), v_units = (int)(Hkv * Dv * es / 16);
  const int64_t per_b = (int64_t)n_new * (k_units + v_units);
  const int threads = 256;
  int blocks = (int)((per_b + threads - 1) / threads);
  if (blocks > 64) blocks = 64;
  kv_append_kernel<<<dim3(blocks, B), threads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<uint4*>(k_cache), static_cast<uint4*>(v_cache), static_cast<const uint4*>(k_new),
      static_cast<const uint4*>(v_new), positions, B, capacity, n_new, k_units, v_units, advance != 0, overflow);
  count_launch();
  return check_cuda(cudaGetLastError(), "kv cache append launch");
}
