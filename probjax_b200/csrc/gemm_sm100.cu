// C[M, N] = A[M, K] . B[N, K]^T with fp32 accumulation, C in the input dtype.
//
// This is the up-projection of latent attention: the shared latent cache
// C [B*S, R] times the stacked per-head projections W [H*Dh, R]^T gives the
// per-head keys (or values) [B*S, H*Dh] in one product -- what the reference
// computes with einsum("...sr,hdr->...shd") in `_materialize_kv`
// (probjax/nn/pallas_kernels/kernels/latent_attention.py:396-410), and what its
// fused kernel recomputes per query tile (:143-145, :177).
//
// tcgen05 kernel: one 128 x 128 output tile per CTA; a TMA producer lane fills a
// 4-stage ring of 128 x 64 A and B tiles (both K-major, 128-byte swizzle), an MMA
// lane accumulates in tensor memory, four epilogue warps read the accumulator
// (one 32-lane quarter each), convert and store.  A plain CUDA-core kernel covers
// fp32 inputs and shapes the tensor-map rules exclude.
#include "pjx_common.cuh"
#include "sm100_ptx.cuh"

namespace pjx {

int make_tmap_2d(CUtensorMap* m, const void* base, int dtype, int64_t rows, int64_t cols, int box_rows);

namespace {

using namespace sm100;

constexpr int TM = 128, TN = 128, TK = 64, ST = 4;
constexpr int A_BYTES = TM * TK * 2, B_BYTES = TN * TK * 2;
constexpr int G_OFF_BAR = ST * (A_BYTES + B_BYTES);
constexpr int G_NBAR = 2 * ST + 1;
constexpr int G_SMEM = G_OFF_BAR + G_NBAR * 8 + 16 + 1024;
constexpr int G_THREADS = 192;

template <bool BF16>
__device__ __forceinline__ uint32_t gpack(float lo, float hi) {
  if constexpr (BF16) {
    __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&t);
  } else {
    __half2 t = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&t);
  }
}

template <bool BF16>
__global__ void __launch_bounds__(G_THREADS, 1)
gemm_tn_sm100_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                     void* __restrict__ Cout, int64_t M, int N, int K, int32_t* status) {
  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  auto BAR = [&](int i) { return sbase + G_OFF_BAR + 8u * i; };
  const int FULL = 0, EMPTY = ST, ACC = 2 * ST;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + G_OFF_BAR + G_NBAR * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * TN;
  const int64_t m0 = (int64_t)blockIdx.y * TM;
  const int nk = (K + TK - 1) / TK;

  if (threadIdx.x == 0) {
    for (int i = 0; i < G_NBAR; ++i) mbar_init(BAR(i), 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(tmem_slot), 128);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      prefetch_tmap(&tm_a);
      prefetch_tmap(&tm_b);
      for (int k = 0; k < nk; ++k) {
        const int s = k % ST;
        if (!mbar_wait(BAR(EMPTY + s), ((k / ST) & 1) ^ 1, abort_flag)) break;
        mbar_arrive_expect_tx(BAR(FULL + s), A_BYTES + B_BYTES);
        tma_load_2d(sbase + s * (A_BYTES + B_BYTES), &tm_a, BAR(FULL + s), k * TK, (int)m0);
        tma_load_2d(sbase + s * (A_BYTES + B_BYTES) + A_BYTES, &tm_b, BAR(FULL + s), k * TK, n0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(TM, TN, BF16, false, false);
      bool ok = true;
      for (int k = 0; k < nk; ++k) {
        const int s = k % ST;
        ok = mbar_wait(BAR(FULL + s), (k / ST) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a = sbase + s * (A_BYTES + B_BYTES), bb = a + A_BYTES;
#pragma unroll
        for (int kk = 0; kk < TK / 16; ++kk)
          mma_ss(tmem, make_smem_desc(a + kk * 32, 16, 1024), make_smem_desc(bb + kk * 32, 16, 1024), idesc,
                 (k | kk) != 0);
        mma_commit(BAR(EMPTY + s));
      }
      if (ok) mma_commit(BAR(ACC));
    }
  } else {
    const int quarter = warp & 3;
    bool ok = mbar_wait(BAR(ACC), 0, abort_flag);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      tc_fence_after();
      const int64_t row = m0 + quarter * 32 + lane;
      const uint32_t taddr = tmem + (static_cast<uint32_t>(quarter * 32) << 16);
      const bool vec_ok = (N % 8 == 0) && ((reinterpret_cast<uintptr_t>(Cout) & 15) == 0);
#pragma unroll
      for (int c = 0; c < TN / 32; ++c) {
        float acc[32];
        tmem_ld32f(taddr + c * 32, acc);
        tmem_wait_ld();
        const int col0 = n0 + c * 32;
        if (row < M && col0 < N) {
          unsigned char* dst = static_cast<unsigned char*>(Cout) + (row * N + col0) * 2;
          if (vec_ok && col0 + 32 <= N) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint4 w;
              w.x = gpack<BF16>(acc[8 * i + 0], acc[8 * i + 1]);
              w.y = gpack<BF16>(acc[8 * i + 2], acc[8 * i + 3]);
              w.z = gpack<BF16>(acc[8 * i + 4], acc[8 * i + 5]);
              w.w = gpack<BF16>(acc[8 * i + 6], acc[8 * i + 7]);
              reinterpret_cast<uint4*>(dst)[i] = w;
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (col0 + i < N) {
                if constexpr (BF16) reinterpret_cast<__nv_bfloat16*>(dst)[i] = __float2bfloat16_rn(acc[i]);
                else reinterpret_cast<__half*>(dst)[i] = __float2half_rn(acc[i]);
              }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    __syncwarp();
    tmem_dealloc(tmem, 128);
    if (lane == 0 && *abort_flag && status) atomicExch(status, (int)PJX_ERR_DEVICE_TIMEOUT);
  }
}

// CUDA-core fallback: 64 x 64 tile, 16-wide K slices, 4 x 4 outputs per thread.
template <typename T>
__global__ void __launch_bounds__(256) gemm_tn_simt_kernel(const T* __restrict__ A, const T* __restrict__ Bm,
                                                          T* __restrict__ Cout, int64_t M, int N, int K) {
  __shared__ float As[16][65], Bs[16][65];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int64_t m0 = (int64_t)blockIdx.y * 64;
  const int n0 = blockIdx.x * 64;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += 16) {
    for (int idx = tid; idx < 64 * 16; idx += 256) {
      const int r = idx >> 4, kk = idx & 15;
      const int64_t gm = m0 + r;
      const int gn = n0 + r;
      As[kk][r] = (gm < M && k0 + kk < K) ? Elem<T>::to_f(A[gm * K + k0 + kk]) : 0.f;
      Bs[kk][r] = (gn < N && k0 + kk < K) ? Elem<T>::to_f(Bm[(int64_t)gn * K + k0 + kk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx + 16 * j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx + 16 * j;
      if (gn < N) Cout[gm * N + gn] = Elem<T>::from_f(acc[i][j]);
    }
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn2() {
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

template <typename T>
int launch_simt(const void* A, const void* Bm, void* C, int64_t M, int N, int K, cudaStream_t stream) {
  dim3 grid((N + 63) / 64, (unsigned)((M + 63) / 64));
  gemm_tn_simt_kernel<T><<<grid, 256, 0, stream>>>(static_cast<const T*>(A), static_cast<const T*>(Bm),
                                                   static_cast<T*>(C), M, N, K);
  count_launch();
  return check_cuda(cudaGetLastError(), "projection (CUDA-core) launch");
}

}  // namespace

// Row-major [rows, cols] 16-bit matrix, box = 64 columns x box_rows rows.
int make_tmap_2d(CUtensorMap* m, const void* base, int dtype, int64_t rows, int64_t cols, int box_rows) {
  EncodeTiledFn fn = encode_fn2();
  if (!fn) return fail(PJX_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, dtype == PJX_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                  const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(PJX_ERR_CUDA, "cuTensorMapEncodeTiled (2-D) failed with CUresult %d", (int)r);
  return PJX_OK;
}

int launch_gemm_tn(const void* A, const void* Bm, void* C, int64_t M, int N, int K, int dtype, int impl,
                   cudaStream_t stream) {
  if (M == 0 || N == 0) return PJX_OK;
  const bool tc_ok = (dtype == PJX_BF16 || dtype == PJX_F16) && K % 8 == 0 && K >= 64 &&
                     ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(Bm)) & 15) == 0 &&
                     (M + TM - 1) / TM <= 65535;
  if (impl == PJX_IMPL_SM100 && !tc_ok)
    return fail(PJX_ERR_UNSUPPORTED, "tcgen05 projection needs 16-bit inputs, K %% 8 == 0, K >= 64 and 16-byte aligned operands");
  if (impl != PJX_IMPL_GENERIC && tc_ok) {
    CUtensorMap ta, tb;
    int rc;
    if ((rc = make_tmap_2d(&ta, A, dtype, M, K, TM))) return rc;
    if ((rc = make_tmap_2d(&tb, Bm, dtype, N, K, TN))) return rc;
    dim3 grid((N + TN - 1) / TN, (unsigned)((M + TM - 1) / TM));
    if (dtype == PJX_BF16) {
      auto kern = gemm_tn_sm100_kernel<true>;
      if ((rc = check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, G_SMEM), "cudaFuncSetAttribute(projection)"))) return rc;
      kern<<<grid, G_THREADS, G_SMEM, stream>>>(ta, tb, C, M, N, K, nullptr);
    } else {
      auto kern = gemm_tn_sm100_kernel<false>;
      if ((rc = check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, G_SMEM), "cudaFuncSetAttribute(projection)"))) return rc;
      kern<<<grid, G_THREADS, G_SMEM, stream>>>(ta, tb, C, M, N, K, nullptr);
    }
    count_launch();
    return check_cuda(cudaGetLastError(), "projection (tcgen05) launch");
  }
  switch (dtype) {
    case PJX_F32: return launch_simt<float>(A, Bm, C, M, N, K, stream);
    case PJX_BF16: return launch_simt<__nv_bfloat16>(A, Bm, C, M, N, K, stream);
    case PJX_F16: return launch_simt<__half>(A, Bm, C, M, N, K, stream);
  }
  return fail(PJX_ERR_BAD_ARG, "unknown dtype %d", dtype);
}

}  // namespace pjx
