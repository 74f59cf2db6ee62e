// C[M, N] = A[M, K] . B[N, K]^T with fp32 accumulation, C in the input dtype.
//
// This is the up-projection of latent attention: the shared latent cache
// C [B*S, R] times the stacked per-head projections W [H*Dh, R]^T gives the
// per-head keys (or values) [B*S, H*Dh] in one product -- what the reference
// computes with einsum("...sr,hdr->...shd") in `_materialize_kv`
// (probjax/nn/pallas_kernels/kernels/latent_attention.py:396-410), and what its
// fused kernel recomputes per query tile (:143-145, :177).
//
// tcgen05 kernel: persistent CTAs walk 128 x 256 output tiles; a TMA producer lane fills a
// 3-stage ring of 128 x 64 A and 256 x 64 B tiles (both K-major, 128-byte swizzle), an MMA
// lane accumulates in tensor memory (double buffered), four epilogue warps read the
// accumulator (one 32-lane quarter each), convert and write the tile through a shared-memory
// staging buffer and TMA stores.  A plain CUDA-core kernel covers
// fp32 inputs and shapes the tensor-map rules exclude.
#include "pjx_common.cuh"
#include "sm100_ptx.cuh"

namespace pjx {

int make_tmap_2d(CUtensorMap* m, const void* base, int dtype, int64_t rows, int64_t cols, int box_rows,
                 int64_t pitch = 0);

namespace {

using namespace sm100;

constexpr int TM = 128, TN = 256, TK = 64;
constexpr int A_BYTES = TM * TK * 2, B_BYTES = TN * TK * 2;
constexpr int STAGE_BYTES = TM * TN * 2;
constexpr int G_THREADS = 192;

// Two shapes of the kernel. STAGED: a 3-stage operand ring plus a staging tile, outputs leave by
// TMA stores - for short K, where the epilogue of a tile is as long as its main loop. Otherwise a
// 4-stage ring and stores straight from the registers, which a long main loop hides.
template <bool STAGED>
struct GCfg {
  static constexpr int ST = STAGED ? 3 : 4;
  static constexpr int OFF_STAGE = ST * (A_BYTES + B_BYTES);  // 4 blocks of 128 rows x 64 columns
  static constexpr int OFF_BAR = OFF_STAGE + (STAGED ? STAGE_BYTES : 0);
  static constexpr int NBAR = 2 * ST + 4 + 2;
  static constexpr int SMEM = OFF_BAR + NBAR * 8 + 16 + 1024;
  static_assert(SMEM <= 227 * 1024, "shared memory budget");
};

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

// Up to two products that share A run in one launch: C0 = A.B0^T [M, N0] and
// C1 = A.B1^T [M, N1] (keys and values of latent attention).  Persistent CTAs walk
// the 128 x 256 output tiles of both; the accumulator is double buffered in tensor
// memory (2 x 256 columns) so the epilogue of one tile overlaps the MMAs of the next.
struct GemmArgs {
  void* c0;
  void* c1;
  int64_t M;
  int n0, n1, K;
  int32_t* status;
  int group_m;   // row tiles per group of the tile walk
};

template <bool BF16, bool STAGED>
__global__ void __launch_bounds__(G_THREADS, 1)
gemm_tn_sm100_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b0,
                     const __grid_constant__ CUtensorMap tm_b1, const __grid_constant__ CUtensorMap tm_c0,
                     const __grid_constant__ CUtensorMap tm_c1, const GemmArgs g) {
  using GC = GCfg<STAGED>;
  constexpr int ST = GC::ST, G_OFF_BAR = GC::OFF_BAR, G_NBAR = GC::NBAR, G_OFF_STAGE = GC::OFF_STAGE;
  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  auto BAR = [&](int i) { return sbase + G_OFF_BAR + 8u * i; };
  const int FULL = 0, EMPTY = ST, ACC_FULL = 2 * ST, ACC_EMPTY = 2 * ST + 2, OUT_STAGED = 2 * ST + 4, OUT_FREE = 2 * ST + 5;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + G_OFF_BAR + G_NBAR * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nk = (g.K + TK - 1) / TK;
  const int mt = (int)((g.M + TM - 1) / TM);
  const int nt0 = (g.n0 + TN - 1) / TN, nt1 = (g.n1 + TN - 1) / TN;
  const int ntiles = mt * (nt0 + nt1);
  // tile id -> (which product, m tile, n tile).  Tiles are walked in groups of kGroupM row tiles:
  // inside a group the row tile is the fast axis and the column tile the slow one, so the CTAs in
  // flight share a few B column tiles and at most kGroupM A row tiles, which stay in L2 while the
  // group sweeps all columns (a plain column-major walk streams all of A once per column tile,
  // out of HBM as soon as A is larger than L2).
  const int kGroupM = g.group_m;
  const int ncols = nt0 + nt1;
  auto decode = [&](int tile, int& which, int& m_idx, int& n_idx) {
    const int grp = tile / (kGroupM * ncols);
    const int first_m = grp * kGroupM;
    const int gm = min(kGroupM, mt - first_m);
    const int r = tile - grp * (kGroupM * ncols);
    const int col = r / gm;
    m_idx = first_m + (r - col * gm);
    which = col >= nt0;
    n_idx = which ? col - nt0 : col;
  };

  if (threadIdx.x == 0) {
    for (int i = 0; i < G_NBAR; ++i) mbar_init(BAR(i), (i >= ACC_EMPTY && i <= OUT_STAGED) ? 128u : 1u);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      prefetch_tmap(&tm_a);
      prefetch_tmap(&tm_b0);
      if (nt1) prefetch_tmap(&tm_b1);
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < ntiles; tile += gridDim.x) {
        int which, m_idx, n_idx;
        decode(tile, which, m_idx, n_idx);
        const CUtensorMap* tb = which ? &tm_b1 : &tm_b0;
        for (int k = 0; k < nk; ++k, ++it) {
          const int s = it % ST;
          ok = mbar_wait(BAR(EMPTY + s), ((it / ST) & 1) ^ 1, abort_flag);
          if (!ok) break;
          mbar_arrive_expect_tx(BAR(FULL + s), A_BYTES + B_BYTES);
          const uint32_t a = sbase + s * (A_BYTES + B_BYTES);
          tma_load_2d(a, &tm_a, BAR(FULL + s), k * TK, m_idx * TM);
          // the B tile is 256 rows: two 128-row boxes
          tma_load_2d(a + A_BYTES, tb, BAR(FULL + s), k * TK, n_idx * TN);
          tma_load_2d(a + A_BYTES + B_BYTES / 2, tb, BAR(FULL + s), k * TK, n_idx * TN + 128);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(TM, TN, BF16, false, false);
      int it = 0, local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < ntiles; tile += gridDim.x, ++local) {
        const int acc = local & 1;
        ok = mbar_wait(BAR(ACC_EMPTY + acc), ((local >> 1) & 1) ^ 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        for (int k = 0; k < nk; ++k, ++it) {
          const int s = it % ST;
          ok = mbar_wait(BAR(FULL + s), (it / ST) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a = sbase + s * (A_BYTES + B_BYTES), bb = a + A_BYTES;
#pragma unroll
          for (int kk = 0; kk < TK / 16; ++kk)
            mma_ss(tmem + acc * TN, make_smem_desc(a + kk * 32, 16, 1024), make_smem_desc(bb + kk * 32, 16, 1024),
                   idesc, (k | kk) != 0);
          mma_commit(BAR(EMPTY + s));
        }
        if (ok) mma_commit(BAR(ACC_FULL + acc));
      }
    }
  } else {
    const int quarter = warp & 3;
    int local = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < ntiles; tile += gridDim.x, ++local) {
      const int acc = local & 1;
      int which, m_idx, n_idx;
      decode(tile, which, m_idx, n_idx);
      const int N = which ? g.n1 : g.n0;
      void* Cout = which ? g.c1 : g.c0;
      ok = mbar_wait(BAR(ACC_FULL + acc), (local >> 1) & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int64_t row = (int64_t)m_idx * TM + quarter * 32 + lane;
      const uint32_t taddr = tmem + (static_cast<uint32_t>(quarter * 32) << 16) + acc * TN;
      if constexpr (STAGED) {
        // Output through shared memory: every thread converts its row and writes it into the staging
        // tile in the tensor map's 128-byte-swizzled layout; one thread hands the tile to TMA stores,
        // which clip rows past M and columns past N. Stores straight from the registers touch 32
        // separate rows per instruction and made short-K products epilogue-bound.
        if (local > 0) {  // the previous tile's stores have read the staging tile
          ok = mbar_wait(BAR(OUT_FREE), (local - 1) & 1, abort_flag);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
        }
        const int r_in = quarter * 32 + lane;
        const uint32_t stage = sbase + G_OFF_STAGE;
#pragma unroll 2
        for (int c = 0; c < TN / 32; ++c) {
          float accv[32];
          tmem_ld32f(taddr + c * 32, accv);
          tmem_wait_ld();
          const uint32_t rbase = stage + (c >> 1) * (TM * 128) + r_in * 128;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t unit = static_cast<uint32_t>((c & 1) * 4 + i) ^ static_cast<uint32_t>(r_in & 7);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};\n" ::"r"(rbase + unit * 16),
                         "r"(gpack<BF16>(accv[8 * i + 0], accv[8 * i + 1])), "r"(gpack<BF16>(accv[8 * i + 2], accv[8 * i + 3])),
                         "r"(gpack<BF16>(accv[8 * i + 4], accv[8 * i + 5])), "r"(gpack<BF16>(accv[8 * i + 6], accv[8 * i + 7]))
                         : "memory");
          }
        }
        tc_fence_before();
        mbar_arrive(BAR(ACC_EMPTY + acc));  // the accumulator is free for the tile after next
        fence_proxy_async();
        mbar_arrive(BAR(OUT_STAGED));
        if (threadIdx.x == 64) {
          if (mbar_wait(BAR(OUT_STAGED), local & 1, abort_flag)) {
            const CUtensorMap* tc = which ? &tm_c1 : &tm_c0;
#pragma unroll
            for (int blk = 0; blk < TN / 64; ++blk)
              if (n_idx * TN + blk * 64 < N) tma_store_2d(tc, stage + blk * (TM * 128), n_idx * TN + blk * 64, m_idx * TM);
            tma_store_commit();
            tma_store_wait_read();
          }
          mbar_arrive(BAR(OUT_FREE));
        }
        continue;
      }
      const bool vec_ok = (N % 8 == 0) && ((reinterpret_cast<uintptr_t>(Cout) & 15) == 0);
#pragma unroll 2
      for (int c = 0; c < TN / 32; ++c) {
        float accv[32];
        tmem_ld32f(taddr + c * 32, accv);
        tmem_wait_ld();
        const int col0 = n_idx * TN + c * 32;
        if (row < g.M && col0 < N) {
          unsigned char* dst = static_cast<unsigned char*>(Cout) + (row * N + col0) * 2;
          if (vec_ok && col0 + 32 <= N) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint4 w;
              w.x = gpack<BF16>(accv[8 * i + 0], accv[8 * i + 1]);
              w.y = gpack<BF16>(accv[8 * i + 2], accv[8 * i + 3]);
              w.z = gpack<BF16>(accv[8 * i + 4], accv[8 * i + 5]);
              w.w = gpack<BF16>(accv[8 * i + 6], accv[8 * i + 7]);
              reinterpret_cast<uint4*>(dst)[i] = w;
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (col0 + i < N) {
                if constexpr (BF16) reinterpret_cast<__nv_bfloat16*>(dst)[i] = __float2bfloat16_rn(accv[i]);
                else reinterpret_cast<__half*>(dst)[i] = __float2half_rn(accv[i]);
              }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(BAR(ACC_EMPTY + acc));
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    __syncwarp();
    tmem_dealloc(tmem, 512);
    if (lane == 0 && *abort_flag && g.status) atomicExch(g.status, (int)PJX_ERR_DEVICE_TIMEOUT);
  }
}

// CUDA-core fallback: 64 x 64 tile, 16-wide K slices, 4 x 4 outputs per thread.
template <typename T>
__global__ void __launch_bounds__(256) gemm_tn_simt_kernel(const T* __restrict__ A, const T* __restrict__ Bm,
                                                          T* __restrict__ Cout, int64_t M, int N, int K, int64_t lda,
                                                          int64_t ldc) {
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
      As[kk][r] = (gm < M && k0 + kk < K) ? Elem<T>::to_f(A[gm * lda + k0 + kk]) : 0.f;
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
      if (gn < N) Cout[gm * ldc + gn] = Elem<T>::from_f(acc[i][j]);
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
int launch_simt(const void* A, const void* Bm, void* C, int64_t M, int N, int K, int64_t lda, int64_t ldc,
                cudaStream_t stream) {
  dim3 grid((N + 63) / 64, (unsigned)((M + 63) / 64));
  gemm_tn_simt_kernel<T><<<grid, 256, 0, stream>>>(static_cast<const T*>(A), static_cast<const T*>(Bm),
                                                   static_cast<T*>(C), M, N, K, lda, ldc);
  count_launch();
  return check_cuda(cudaGetLastError(), "projection (CUDA-core) launch");
}

}  // namespace

// Row-major [rows, cols] 16-bit matrix with a row pitch of `pitch` elements (0 = cols),
// box = 64 columns x box_rows rows.
int make_tmap_2d(CUtensorMap* m, const void* base, int dtype, int64_t rows, int64_t cols, int box_rows, int64_t pitch) {
  EncodeTiledFn fn = encode_fn2();
  if (!fn) return fail(PJX_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)(pitch ? pitch : cols) * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, dtype == PJX_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                  const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(PJX_ERR_CUDA, "cuTensorMapEncodeTiled (2-D) failed with CUresult %d", (int)r);
  return PJX_OK;
}

namespace {

int simt_by_dtype(const void* A, const void* Bm, void* C, int64_t M, int N, int K, int64_t lda, int64_t ldc, int dtype,
                  cudaStream_t stream) {
  switch (dtype) {
    case PJX_F32: return launch_simt<float>(A, Bm, C, M, N, K, lda, ldc, stream);
    case PJX_BF16: return launch_simt<__nv_bfloat16>(A, Bm, C, M, N, K, lda, ldc, stream);
    case PJX_F16: return launch_simt<__half>(A, Bm, C, M, N, K, lda, ldc, stream);
  }
  return fail(PJX_ERR_BAD_ARG, "unknown dtype %d", dtype);
}

}  // namespace

int launch_gemm_tn2(const void* A, const void* B0, void* C0, int N0, const void* B1, void* C1, int N1, int64_t M,
                    int K, int dtype, int impl, int32_t* status, cudaStream_t stream, int64_t lda, int64_t ldc) {
  if (M == 0 || (N0 == 0 && N1 == 0)) return PJX_OK;
  if (lda == 0) lda = K;
  const bool c_strided = ldc != 0 && ldc != N0;
  if (c_strided && N1) return fail(PJX_ERR_BAD_ARG, "a row pitch for C is taken for one product only");
  if (ldc == 0) ldc = N0;
  uintptr_t al = reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B0);
  if (N1) al |= reinterpret_cast<uintptr_t>(B1);
  bool tc_ok = (dtype == PJX_BF16 || dtype == PJX_F16) && K % 8 == 0 && K >= 64 && (al & 15) == 0 &&
               M <= 2147483647LL - TM && lda % 8 == 0;
  // a pitched C leaves through TMA stores only (the direct stores assume dense rows)
  if (c_strided && !(ldc % 8 == 0 && N0 % 8 == 0 && (reinterpret_cast<uintptr_t>(C0) & 15) == 0)) tc_ok = false;
  if (impl == PJX_IMPL_SM100 && !tc_ok)
    return fail(PJX_ERR_UNSUPPORTED, "tcgen05 projection needs 16-bit inputs, K %% 8 == 0, K >= 64 and 16-byte aligned operands");
  if (impl != PJX_IMPL_GENERIC && tc_ok) {
    CUtensorMap ta, tb0, tb1;
    int rc;
    if ((rc = make_tmap_2d(&ta, A, dtype, M, K, TM, lda))) return rc;
    if ((rc = make_tmap_2d(&tb0, B0, dtype, N0, K, 128))) return rc;
    if (N1) {
      if ((rc = make_tmap_2d(&tb1, B1, dtype, N1, K, 128))) return rc;
    } else {
      tb1 = tb0;
    }
    GemmArgs g;
    g.c0 = C0; g.c1 = C1; g.M = M; g.n0 = N0; g.n1 = N1; g.K = K; g.status = status;
    uintptr_t cal = reinterpret_cast<uintptr_t>(C0);
    if (N1) cal |= reinterpret_cast<uintptr_t>(C1);
    // Short K: a tile's epilogue is as long as its main loop, so the outputs go through shared memory
    // and TMA stores (needs row pitches that are multiples of 16 bytes). Long K hides the direct stores
    // and prefers the fourth operand stage.
    const bool staged = (K < 1536 || c_strided) && (N0 % 8 == 0) && (N1 % 8 == 0) && (cal & 15) == 0;
    CUtensorMap tc0 = ta, tc1 = ta;
    if (staged) {
      if ((rc = make_tmap_2d(&tc0, C0, dtype, M, N0, TM, ldc))) return rc;
      tc1 = tc0;
      if (N1 && (rc = make_tmap_2d(&tc1, C1, dtype, M, N1, TM))) return rc;
    }
    g.group_m = 16;  // 16 to 32 measure alike on B200; 4 and 64 lose 3-6 %
    const int64_t tiles = ((M + TM - 1) / TM) * ((N0 + TN - 1) / TN + (N1 + TN - 1) / TN);
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const unsigned grid = (unsigned)(tiles < sms ? tiles : sms);
    auto launch = [&](auto kern, int smem) -> int {
      int r = check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem), "cudaFuncSetAttribute(projection)");
      if (r) return r;
      kern<<<grid, G_THREADS, smem, stream>>>(ta, tb0, tb1, tc0, tc1, g);
      return PJX_OK;
    };
    if (dtype == PJX_BF16)
      rc = staged ? launch(gemm_tn_sm100_kernel<true, true>, GCfg<true>::SMEM) : launch(gemm_tn_sm100_kernel<true, false>, GCfg<false>::SMEM);
    else
      rc = staged ? launch(gemm_tn_sm100_kernel<false, true>, GCfg<true>::SMEM) : launch(gemm_tn_sm100_kernel<false, false>, GCfg<false>::SMEM);
    if (rc) return rc;
    count_launch();
    return check_cuda(cudaGetLastError(), "projection (tcgen05) launch");
  }
  int rc = simt_by_dtype(A, B0, C0, M, N0, K, lda, ldc, dtype, stream);
  if (rc || !N1) return rc;
  return simt_by_dtype(A, B1, C1, M, N1, K, lda, N1, dtype, stream);
}

int launch_gemm_tn(const void* A, const void* Bm, void* C, int64_t M, int N, int K, int dtype, int impl,
                   cudaStream_t stream) {
  return launch_gemm_tn2(A, Bm, C, N, nullptr, nullptr, 0, M, K, dtype, impl, nullptr, stream);
}

}  // namespace pjx
