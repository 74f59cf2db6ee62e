// Shared declarations of the attention library: element traits, the launch
// parameter blocks, error plumbing and the internal launcher prototypes.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/pjx_attention.h"
#include "score_mod.cuh"

namespace pjx {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// ---------------------------------------------------------------------------
// Element traits
// ---------------------------------------------------------------------------
template <typename T>
struct Elem;
template <>
struct Elem<float> {
  static __device__ __forceinline__ float to_f(float x) { return x; }
  static __device__ __forceinline__ float from_f(float x) { return x; }
  static __device__ __forceinline__ float round(float x) { return x; }
};
template <>
struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f(__nv_bfloat16 x) { return __bfloat162float(x); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float x) { return __float2bfloat16_rn(x); }
  static __device__ __forceinline__ float round(float x) {
    return __bfloat162float(__float2bfloat16_rn(x));
  }
};
template <>
struct Elem<__half> {
  static __device__ __forceinline__ float to_f(__half x) { return __half2float(x); }
  static __device__ __forceinline__ __half from_f(float x) { return __float2half_rn(x); }
  static __device__ __forceinline__ float round(float x) {
    return __half2float(__float2half_rn(x));
  }
};

inline size_t dtype_size(int dtype) { return dtype == PJX_F32 ? 4 : 2; }

// ---------------------------------------------------------------------------
// Parameter block of the forward kernels
// ---------------------------------------------------------------------------
// The part every forward kernel takes as its parameter block.  The score modifiers travel beside it
// (FwdParams below, a second kernel parameter in the tcgen05 forward): with the modifiers inside this
// block the compiler's register allocation of the tcgen05 variants that never touch them got worse
// (staged-bias variant: 132 -> 868 bytes of spills, 0.097 -> 0.15 ms).
struct FwdParamsCore {
  const void* q;
  const void* k;
  const void* v;
  void* o;
  float* lse;                 // [B, Hq, Lq] or null
  const int32_t* kv_lengths;  // [B] or null
  const float* bias;          // [Bb, Hb, Lq, Lkv] or null
  int64_t bias_bs, bias_hs;   // element strides of the bias batch / head axes (0 = broadcast)
  int B, Lq, Lkv, Hq, Hkv, D, Dv;
  int causal;   // shorthand for band_hi == 0 with no lower bound (the kernels' fast path)
  // Band of visible keys around each query row: row + band_lo <= key <= row + band_hi.
  // PJX_BAND_NO_LOWER / PJX_BAND_NO_UPPER leave a side open.
  int band_lo = PJX_BAND_NO_LOWER, band_hi = PJX_BAND_NO_UPPER;
  float sm_scale;
  int32_t* status;  // device status word or null

  bool banded() const { return !causal && (band_lo > PJX_BAND_NO_LOWER || band_hi < PJX_BAND_NO_UPPER); }
};

struct FwdParams : FwdParamsCore {
  ScoreMod mod;  // structured masks / score modifiers (mod.on == 0: none)
};

struct DecodeParams {
  const void* q;
  const void* k;
  const void* v;
  const int32_t* kv_lengths;
  void* o;
  float* lse;
  float* o_part;    // [B, Hkv, S, R, Dv] fp32
  float* lse_part;  // [B, Hkv, S, R] fp32, base 2, -inf for a split without keys
  int B, Lq, Hq, Hkv, D, Dv, capacity;
  int split_len, num_splits, rows;  // rows = (Hq / Hkv) * Lq
  float sm_scale;
  int o_is_f32;
  // Sequence-sharded decode (ex_world > 0): instead of the local combine, every
  // rank publishes its partial into all ranks' exchange buffers and then combines
  // the partials of all ranks. Buffer layout (identical on every rank), N = B*Lq*Hq:
  //   2 x { float o[world][N][Dv]; float lse[world][N]; }   (double buffered by step parity)
  //   uint32 flags[16]; uint32 counter;          (per-rank flags of the three-kernel exchange)
  //   uint32 unit_flags[world][N];               (reserved)
  //   uint32 unit_counters[N];                   (split CTAs of a (batch, kv head) that have finished)
  //   uint4 ll[2][world][N][Dv / 2 + 1];         (one-kernel exchange: values travelling with their step number)
  int ex_world = 0, ex_rank = 0;
  int ex_fused = 0;  // 1: the split kernel's last CTA of each (batch, kv head) exchanges and combines
  int ex_overlap = 0;  // 1 (with ex_fused): may start before the previous kernel on the stream has finished
  uint32_t ex_step = 0;
  unsigned char* ex_buf[16] = {};
  int32_t* status = nullptr;
  // Paged cache (block_table != null): k and v are page pools [num_pages, page_size, Hkv, D];
  // logical key j of sequence b lives in page block_table[b * max_pages + j / page_size] at row
  // j % page_size. page_size is a multiple of the 64-key tile, capacity = max_pages * page_size.
  const int32_t* block_table = nullptr;
  int page_size = 0, max_pages = 0;
  // Prefill rows through the latent decode kernels (seq_tokens > 0): grid z walks B x seq_tokens
  // one-token sequences.  Sequence z reads cache row z / seq_tokens, is query token
  // t = seq_first + z % seq_tokens of seq_total, and sees the keys below t + seq_visible (and below
  // the cache row's valid length); its partials are indexed by z, its output by (cache row, t).
  int seq_tokens = 0, seq_first = 0, seq_total = 0, seq_visible = 0;
};

// What grid index z of a decode launch stands for (see DecodeParams::seq_tokens).
struct DecodeSeq {
  int cache_b;   // batch row of the cache and of kv_lengths
  int64_t q_b;   // row of q / o counted in blocks of Lq tokens
  int len;       // valid keys
};

// Batch rows the cache of a decode launch holds.
inline int64_t decode_cache_rows(const DecodeParams& p) { return p.seq_tokens > 0 ? p.B / p.seq_tokens : p.B; }

#ifdef __CUDACC__
__device__ __forceinline__ DecodeSeq decode_seq(const DecodeParams& p, int z) {
  DecodeSeq s;
  s.cache_b = z;
  s.q_b = z;
  int lim = p.capacity;
  if (p.seq_tokens > 0) {
    s.cache_b = z / p.seq_tokens;
    const int t = p.seq_first + z % p.seq_tokens;
    s.q_b = (int64_t)s.cache_b * p.seq_total + t;
    lim = max(0, min(p.capacity, t + p.seq_visible));
  }
  s.len = p.kv_lengths ? max(0, min(lim, p.kv_lengths[s.cache_b])) : lim;
  return s;
}

// Index of the LSE of (sequence, head, token of the launch) in the caller's [B, Hq, Lq] array.
__device__ __forceinline__ int64_t decode_lse_index(const DecodeParams& p, const DecodeSeq& s, int h, int t) {
  if (p.seq_tokens > 0)
    return ((int64_t)s.cache_b * p.Hq + h) * p.seq_total + (s.q_b - (int64_t)s.cache_b * p.seq_total);
  return ((int64_t)s.cache_b * p.Hq + h) * p.Lq + t;
}
#endif

// Parameter block of the backward kernels
struct BwdParams {
  const void* q;
  const void* k;
  const void* v;
  const void* o;
  const void* d_o;
  const float* lse;     // [B, Hq, Lq] natural log, +inf for rows without keys
  float* delta;         // [B, Hq, Lq_pad] workspace: rowsum(o * d_o), 0 in the padding
  float* lse2;          // [B, Hq, Lq_pad] workspace: lse * log2(e), +inf in the padding
  int Lq_pad;           // Lq rounded up to a multiple of 128 (row pitch of the two arrays)
  void* dq;
  void* dk;
  void* dv;
  const int32_t* kv_lengths;
  const float* bias;
  int64_t bias_bs, bias_hs;
  float* dbias = nullptr;     // gradient of the bias, same shape and strides, zeroed by the caller; or null
  bool dbias_atomic = false;  // a broadcast axis: several (batch, head) pairs add into one entry
  int B, Lq, Lkv, Hq, Hkv, D, Dv;
  int band_lo, band_hi;  // key j is visible to query i iff i + band_lo <= j <= i + band_hi
  float sm_scale;
  int dtype = PJX_F32;
  int32_t* status = nullptr;  // device status word or null
  bool use_sm100 = false;     // dQ and dK/dV by the tcgen05 kernels instead of the CUDA-core ones
  ScoreMod mod;               // structured masks / score modifiers (CUDA-core kernels only)
};

constexpr int kMaxExchangeRanks = 16;
__host__ __device__ inline size_t exchange_record_floats(int world, int64_t n_rows, int Dv) { return (size_t)world * n_rows * (Dv + 1); }
// byte offset of unit_flags inside an exchange buffer (16-byte aligned)
__host__ __device__ inline size_t exchange_unit_flags_offset(int world, int64_t n_rows, int Dv) {
  const size_t head = 2 * exchange_record_floats(world, n_rows, Dv) * sizeof(float) + (kMaxExchangeRanks + 1) * sizeof(uint32_t);
  return (head + 15) / 16 * 16;
}
// byte offset of the data+flag region of the one-kernel exchange (16-byte aligned):
// [2 parities][world][n_rows] records of (Dv / 2 + 1) 16-byte lines {v0, step, v1, step}
__host__ __device__ inline size_t exchange_ll_offset(int world, int64_t n_rows, int Dv) {
  const size_t off = exchange_unit_flags_offset(world, n_rows, Dv) + (size_t)(world + 1) * n_rows * sizeof(uint32_t);
  return (off + 15) / 16 * 16;
}
inline size_t exchange_buffer_bytes(int world, int64_t n_rows, int Dv) {
  return exchange_ll_offset(world, n_rows, Dv) + (size_t)2 * world * n_rows * (Dv / 2 + 1) * 16;
}

// ---------------------------------------------------------------------------
// Error plumbing (host)
// ---------------------------------------------------------------------------
int fail(int status, const char* fmt, ...);
int convert_score_mod(const pjx_score_mod* m, ScoreMod* out);
int check_cuda(cudaError_t e, const char* what);
void count_launch(int n = 1);

// ---------------------------------------------------------------------------
// Launchers implemented in the kernel translation units. Each returns a
// pjx_status and enqueues on `stream` only.
// ---------------------------------------------------------------------------
int launch_fwd_generic(const FwdParams& p, int dtype, cudaStream_t stream);
bool fwd_sm100_supported(const FwdParams& p, int dtype, const char** why);
int launch_fwd_sm100(const FwdParams& p, int dtype, cudaStream_t stream);
// tcgen05 backward (dQ kernel and dK/dV kernel); expects p.delta filled.
bool bwd_sm100_supported(const BwdParams& p, const char** why);
int launch_bwd_sm100(const BwdParams& p, cudaStream_t stream);
bool decode_fast_supported(const DecodeParams& p, int dtype);
int launch_decode(const DecodeParams& p, int dtype, cudaStream_t stream);
// Split length chosen for split_len = 0; `ragged`: per-sequence lengths are given (see pjx_api.cu).
int decode_default_split_len(int B, int Hkv, int capacity, bool ragged);
// CTAs of the split-KV kernel (dtype, head width D) that the current device holds at once.
int decode_coresident_ctas(int dtype, int D, int* out);
int launch_decode_combine(const DecodeParams& p, int dtype, cudaStream_t stream);
// Absorbed latent decode (K = V = cache [B, S, R]): split kernel writing the decode partial layout.
bool decode_latent_supported(int R, int dtype);
int launch_decode_latent_splits(const DecodeParams& p, int dtype, cudaStream_t stream);
// The same on the tcgen05 tensor cores (attn_decode_latent_sm100.cu); needs p.status.
bool decode_latent_tc_supported(const DecodeParams& p, int dtype);
int launch_decode_latent_tc_splits(const DecodeParams& p, int dtype, cudaStream_t stream);
int launch_combine_parts(const float* o_parts, const float* lse_parts, int n_parts, int64_t n_rows,
                         int Dv, void* o, float* lse, int dtype, cudaStream_t stream);
// C[M, N] = A[M, K] . B[N, K]^T, all row-major, fp32 accumulation, C in `dtype`.
int launch_gemm_tn(const void* A, const void* Bm, void* C, int64_t M, int N, int K, int dtype,
                   int impl, cudaStream_t stream);
// Two products sharing A in one launch: C0 = A . B0^T [M, N0], C1 = A . B1^T [M, N1] (N1 may be 0).
// `lda` / `ldc` are row pitches of A and C0 in elements (0 = dense rows); a pitched C0 excludes C1.
int launch_gemm_tn2(const void* A, const void* B0, void* C0, int N0, const void* B1, void* C1, int N1,
                    int64_t M, int K, int dtype, int impl, int32_t* status, cudaStream_t stream,
                    int64_t lda = 0, int64_t ldc = 0);

}  // namespace pjx
