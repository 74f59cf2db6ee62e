// Stand-alone probe: the rate at which one thread can issue tcgen05.mma sequences of the shapes the
// attention kernels use (S = Q.K^T from shared memory or with A in tensor memory, O += P.V), one CTA on
// one SM and one CTA on every SM.  Not part of the library; build and run with
//   python -m probjax_b200.build --probe && probjax_b200/build/probe_mma_rate
// The operands are constants; only the timing means anything.
#include <cstdio>
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include "sm100_ptx.cuh"
using namespace pjx::sm100;

// mode 0: SS K-major A,B  (S = Q K^T): M=128, N, 8 k-steps of 16 per "tile" (D=128)
// mode 1: TS, B K-major  (A from tensor memory)
// mode 2: TS, B MN-major (O += P V): N=128 fixed, ksteps per tile = NK/16
// mode 3: interleaved like the kernel: SS(N) tile then TS-MN tile
template <int MODE, int N>
__global__ void __launch_bounds__(128, 1) rate_kernel(long long* out, int tiles, int* status) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t base = smem_u32(smem);
  const uint32_t a_addr = base, b_addr = base + 32768, v_addr = base + 32768 + 65536;  // B up to 256 rows x 128 d
  const uint32_t bar = base + 32768 + 65536 + 32768, slot = bar + 16;
  for (int i = threadIdx.x; i < (32768 + 65536 + 32768) / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0x3c003c00u;
  if (threadIdx.x == 0) { mbar_init(bar, 1); fence_barrier_init(); }
  __syncthreads();
  if (threadIdx.x < 32) { tmem_alloc(slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  fence_proxy_async();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(smem + (slot - base));
  volatile int abort_flag = 0;
  if (threadIdx.x == 0) {
    constexpr uint32_t idesc_s = make_idesc(128, N, true, false, false);
    constexpr uint32_t idesc_o = make_idesc(128, 128, true, false, true);
    const long long t0 = clock64();
    for (int t = 0; t < tiles; ++t) {
      const uint32_t d = tmem + (t & 1) * 128;  // two accumulators, alternating
      if (MODE == 0 || MODE == 3) {
#pragma unroll
        for (int s = 0; s < 2; ++s)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            mma_ss(d, make_smem_desc(a_addr + s * 128 * 128 + kk * 32, 16, 1024),
                   make_smem_desc(b_addr + s * N * 128 + kk * 32, 16, 1024), idesc_s, (s | kk) != 0);
      }
      if (MODE == 1) {
#pragma unroll
        for (int s = 0; s < 2; ++s)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            mma_ts(d, tmem + 256 + (s * 4 + kk) * 8, make_smem_desc(b_addr + s * N * 128 + kk * 32, 16, 1024), idesc_s, (s | kk) != 0);
      }
      if (MODE == 2 || MODE == 3) {
#pragma unroll
        for (int kk = 0; kk < N / 16; ++kk)
          mma_ts(tmem + 384 + (t & 1) * 0, tmem + 256 + kk * 8, make_smem_desc(v_addr + kk * 2048, 128 * 128, 1024), idesc_o, kk != 0);
      }
    }
    mma_commit(bar);
    const bool ok = mbar_wait(bar, 0, &abort_flag);
    const long long t1 = clock64();
    if (!ok) atomicExch(status, 1);
    out[blockIdx.x] = t1 - t0;
  }
  __syncthreads();
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) tmem_dealloc(tmem, 512);
}

template <int MODE, int N>
void run(const char* name, long long* d_out, int* d_status, int tiles, double flops_per_tile) {
  const int smem = 32768 + 65536 + 32768 + 64 + 1024;
  cudaFuncSetAttribute(rate_kernel<MODE, N>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  for (int grid : {1, 148}) {
    rate_kernel<MODE, N><<<grid, 128, smem>>>(d_out, tiles, d_status);
    rate_kernel<MODE, N><<<grid, 128, smem>>>(d_out, tiles, d_status);
    cudaError_t e = cudaDeviceSynchronize();
    long long h[148]; int st = 0;
    cudaMemcpy(h, d_out, sizeof(long long) * grid, cudaMemcpyDeviceToHost);
    cudaMemcpy(&st, d_status, 4, cudaMemcpyDeviceToHost);
    double avg = 0; for (int i = 0; i < grid; ++i) avg += h[i]; avg /= grid;
    printf("%-28s grid %3d: %8.1f cycles/tile  (ideal %6.1f)  err=%s status=%d\n", name, grid, avg / tiles,
           flops_per_tile / 8192.0, cudaGetErrorString(e), st);
  }
}

int main() {
  long long* d_out; int* d_status;
  cudaMalloc(&d_out, 148 * 8); cudaMalloc(&d_status, 4); cudaMemset(d_status, 0, 4);
  const int tiles = 2000;
  run<0, 128>("SS  N=128 K=128", d_out, d_status, tiles, 2.0 * 128 * 128 * 128);
  run<0, 64>("SS  N=64  K=128", d_out, d_status, tiles, 2.0 * 128 * 64 * 128);
  run<0, 256>("SS  N=256 K=128", d_out, d_status, tiles, 2.0 * 128 * 256 * 128);
  run<1, 128>("TS  N=128 K=128 (A in tmem)", d_out, d_status, tiles, 2.0 * 128 * 128 * 128);
  run<1, 64>("TS  N=64  K=128 (A in tmem)", d_out, d_status, tiles, 2.0 * 128 * 64 * 128);
  run<2, 128>("TS-MN N=128 K=128 (P.V)", d_out, d_status, tiles, 2.0 * 128 * 128 * 128);
  run<2, 64>("TS-MN N=128 K=64  (P.V half)", d_out, d_status, tiles, 2.0 * 128 * 128 * 64);
  run<3, 128>("SS128 + PV128 alternating", d_out, d_status, tiles, 4.0 * 128 * 128 * 128);
  run<3, 64>("SS64 + PV64 alternating", d_out, d_status, tiles, 4.0 * 128 * 64 * 128);
  return 0;
}
