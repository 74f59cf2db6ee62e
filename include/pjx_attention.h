/*
 * pjx_attention.h -- C ABI of the sm_100a attention library.
 *
 * Everything probjax.nn's attention hot path lowers to on a GPU, as plain
 * `extern "C"` entry points: caller-owned device buffers, sizes, a CUDA stream.
 * No entry point allocates or frees device memory, synchronises the device
 * (except the *_host and pjx_read_status helpers, which say so) or throws.
 * All tensors are row-major and dense, laid out exactly as the reference
 * passes them to its kernels (no transposes):
 *
 *   q   [B, Lq,  Hq,  D ]      k [B, Lkv, Hkv, D]      v [B, Lkv, Hkv, Dv]
 *   o   [B, Lq,  Hq,  Dv]      lse [B, Hq, Lq] float32, natural log
 *
 * Query head h reads KV head h / (Hq / Hkv).  Rows without any valid key give
 * o = 0 and lse = +inf.  Scores are (q.k) * sm_scale, then + bias, then the
 * mask; the softmax is taken in fp32 and the probabilities are rounded to the
 * input dtype before the product with V, as the reference does.
 *
 * Every function returns a pjx_status (0 = ok).  A message for the last failure
 * on the calling thread is available from pjx_last_error().
 *
 * Citations give the reference interface each entry point replaces, as paths
 * inside the probjax project.
 */
#ifndef PJX_ATTENTION_H_
#define PJX_ATTENTION_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum pjx_status {
  PJX_OK = 0,
  PJX_ERR_BAD_ARG = 1,        /* shapes / pointers / dtypes the reference rejects with ValueError */
  PJX_ERR_UNSUPPORTED = 2,    /* valid call that no kernel here computes */
  PJX_ERR_WORKSPACE = 3,      /* workspace missing or too small */
  PJX_ERR_DEVICE_TIMEOUT = 4, /* a bounded in-kernel wait expired (reported through the status word) */
  PJX_ERR_CUDA = 5            /* a CUDA runtime / driver call failed */
} pjx_status;

typedef enum pjx_dtype { PJX_F32 = 0, PJX_BF16 = 1, PJX_F16 = 2 } pjx_dtype;

/* Which forward kernel to run. AUTO picks the tcgen05 kernel whenever the call
 * is one it computes and the generic one otherwise. */
typedef enum pjx_impl { PJX_IMPL_AUTO = 0, PJX_IMPL_GENERIC = 1, PJX_IMPL_SM100 = 2 } pjx_impl;

int pjx_version(void);
const char* pjx_status_string(int status);
const char* pjx_last_error(void);

/*
 * Flash-attention forward (MHA / GQA; optional causal mask, per-batch key
 * lengths and dense additive bias).
 *
 * Replaces the `mha_fwd`, `mha_fwd_res` and their `_gqa` kernel primitives
 * (probjax/nn/pallas_kernels/kernels/attention.py:2456-2490, 2537-2565; body
 * `_mha_impl_raw` 2130-2278 launching `mha_forward_kernel` 377-533) for masks
 * in {none, CausalMask, KVLenMask, their AND} and bias in {none, DenseBias}.
 *
 *   lse          may be NULL (the non-`_res` primitive).
 *   kv_lengths   int32[B] or NULL: key j of batch b is valid iff j < kv_lengths[b].
 *   bias         float32 [Bb, Hb, Lq, Lkv] with Bb in {1,B}, Hb in {1,Hq}, or NULL;
 *                bias_batch_stride / bias_head_stride are element strides
 *                (0 broadcasts that axis).
 *   causal       nonzero: key j is valid for query i iff j <= i.
 *   status       int32 device word or NULL; a kernel writes a nonzero pjx_status
 *                there if a bounded wait expires. Read it with pjx_read_status.
 */
int pjx_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse,
                 const int32_t* kv_lengths, const float* bias, int64_t bias_batch_stride,
                 int64_t bias_head_stride, int B, int Lq, int Lkv, int Hq, int Hkv, int D, int Dv,
                 int dtype, int causal, float sm_scale, int impl, int32_t* status, void* stream);

/*
 * pjx_attn_fwd with a band of visible keys instead of the causal flag: key j is
 * valid for query i iff i + band_lo <= j <= i + band_hi.  PJX_BAND_NO_LOWER /
 * PJX_BAND_NO_UPPER leave a side open; (NO_LOWER, 0) is the causal mask.
 *
 * Covers the index masks the reference's default dispatch sends to its fused kernel
 * (probjax/nn/layers/attention.py:1167-1202): `LocalWindowMask(l, r)` -> (-l, r),
 * `CausalLocalWindowMask(l)` -> (-l, 0), `CausalFromBottomRightMask` -> (NO_LOWER,
 * Lkv - Lq) (probjax/nn/pallas_kernels/attention_mask_bias.py:651-782), and their AND
 * with each other and with key lengths.  KV tiles wholly outside the band of a query
 * tile are skipped, as the reference's block-sparse iteration does
 * (`fast_blockmask_local_window`).
 */
#define PJX_BAND_NO_LOWER (-(1 << 30))
#define PJX_BAND_NO_UPPER (1 << 30)
int pjx_attn_fwd_band(const void* q, const void* k, const void* v, void* o, float* lse,
                      const int32_t* kv_lengths, const float* bias, int64_t bias_batch_stride,
                      int64_t bias_head_stride, int B, int Lq, int Lkv, int Hq, int Hkv, int D, int Dv,
                      int dtype, int band_lo, int band_hi, float sm_scale, int impl, int32_t* status,
                      void* stream);

/*
 * Structured masks and score modifiers, evaluated element by element inside the kernels from
 * O(B T) / O(H T) data: no [Lq, Lkv] tensor is ever built.  A NULL pointer / zero switches a
 * field off; an all-zero struct (or a NULL struct pointer) is "no modifiers".
 *
 * Replaces the per-tile evaluation of the reference's mask / bias classes inside its kernels
 * (probjax/nn/pallas_kernels/attention_mask_bias.py; applied at kernels/attention.py:456-481):
 *
 *   seg_q, seg_k     int32 [Bs, Lq] / [Bs, Lkv] (Bs in {1, B}; *_batch_stride in elements, 0 =
 *                    shared): key j is visible to query i iff seg_q[b,i] == seg_k[b,j].
 *                    SameSegmentMask 1537-1565, BlockDiagonalMask 871-893 (AND the causal band:
 *                    BlockDiagonalCausalMask 984-1008).  SeqLenMask 1239-1323 and
 *                    MarginalizationMask 1671-1699, both of the form (a_i & a_j) | i == j for a
 *                    per-token keep vector a, are the ids "0 where a, else -(t+1)".
 *   row_kv_limit     int32 [Bs, Lq]: visible iff j < row_kv_limit[b,i] (KeyPaddingMask 1132-1234,
 *                    whose lengths are per query row).
 *   prefix_len       int32 [B]: keys j < prefix_len[b] are visible to every row, OR-ed with the
 *                    band (PrefixLMMask 785-809 with the causal band).
 *   rel_bias         float32 [Hr, Lq + Lkv - 1] (Hr in {1, Hq}; head stride in elements, 0 =
 *                    shared): score += rel_bias[h, (j - i) + Lq - 1].  Any bias of the head and the
 *                    relative position: T5RelativePositionBias 2453, LearnedRelativePositionBias
 *                    2521 (bucket look-up done per distance by the caller), ConstantBias 1781.
 *   alibi_slopes     float32 [Hq] with alibi_mode 1: score -= slope[h] * max(i - j, 0)
 *                    (CausalAlibiBias 2230-2247); mode 2: score -= slope[h] * |i - j|
 *                    (SymmetricAlibiBias 2355-2372, DistanceDecayBias 2387-2406).
 *   head_scale       float32 [Hq]: score *= head_scale[h] (PerHeadScaleBias 2606).
 *   softcap          > 0: score = softcap * tanh(score / softcap) (SoftCappingBias 2564-2582).
 *   dropout_rate,    attention dropout with the reference's counter hash (`_dropout_mask_counter`,
 *   dropout_seed     probjax/nn/pallas_kernels/kernels/attention.py:116-148): probability (b, h, i, j) is
 *                    dropped iff hash(seed, b, h, i, j) * 2^-32 < rate, survivors are scaled by
 *                    1 / (1 - rate), after the row sum has been taken (497-505); the backward and the
 *                    forward-mode entry points regenerate the same mask from the same seed.  The seed is
 *                    the folded key of `_rng_seed_from_key` (151-159).
 *
 * "score" is sm_scale * q.k; every term is a delta on that same value and the deltas add up, as
 * SumBias 553-579 defines the sum of modifiers; the dense `bias` argument adds on top.  The
 * backward and forward-mode entry points multiply dS by d(modified score)/d(score), the `grad`
 * methods of the two non-additive classes (2590-2601, 2637-2650).
 */
typedef struct pjx_score_mod {
  const int32_t* seg_q;
  const int32_t* seg_k;
  int64_t seg_q_batch_stride, seg_k_batch_stride;
  const int32_t* row_kv_limit;
  int64_t row_kv_limit_batch_stride;
  const int32_t* prefix_len;
  const float* rel_bias;
  int64_t rel_bias_head_stride;
  const float* alibi_slopes;
  int32_t alibi_mode;
  const float* head_scale;
  float softcap;
  float dropout_rate;
  uint32_t dropout_seed;
} pjx_score_mod;

/* pjx_attn_fwd_band with score modifiers (mod may be NULL).  16-bit inputs with head shapes the
 * tcgen05 kernel takes run on it with the modifiers evaluated in its softmax warps; other calls
 * run the exact-fp32 kernel. */
int pjx_attn_fwd_mod(const void* q, const void* k, const void* v, void* o, float* lse,
                     const int32_t* kv_lengths, const float* bias, int64_t bias_batch_stride,
                     int64_t bias_head_stride, int B, int Lq, int Lkv, int Hq, int Hkv, int D, int Dv,
                     int dtype, int band_lo, int band_hi, float sm_scale, const pjx_score_mod* mod,
                     int impl, int32_t* status, void* stream);

/*
 * Backward of pjx_attn_fwd: dq, dk, dv from q, k, v, o, d_o and the forward's
 * natural-log lse, for the same masks and bias (the bias itself gets no gradient
 * here).  First correct path: exact fp32 arithmetic on CUDA cores for every dtype.
 *
 * Replaces the `mha_bwd` primitive (probjax/nn/pallas_kernels/kernels/
 * attention.py:2509-2534; kernels `_preprocess_backward_kernel` 853-906,
 * `mha_backward_kernel_split_dkdv` 1189 and `_split_dq` 1364).  With GQA, dk and dv
 * of a KV head are summed over its group's query heads.
 *
 *   d_o        [B, Lq, Hq, Dv] gradient of o, in `dtype`
 *   dq, dk, dv like q, k, v, in `dtype`
 *   workspace  pjx_attn_bwd_workspace_bytes(B, Lq, Hq) bytes
 */
int pjx_attn_bwd(const void* q, const void* k, const void* v, const void* o, const float* lse,
                 const void* d_o, void* dq, void* dk, void* dv, const int32_t* kv_lengths,
                 const float* bias, int64_t bias_batch_stride, int64_t bias_head_stride, int B, int Lq,
                 int Lkv, int Hq, int Hkv, int D, int Dv, int dtype, int causal, float sm_scale,
                 void* workspace, size_t workspace_bytes, void* stream);
/* The same for the band form of the mask (see pjx_attn_fwd_band).  `impl` picks the
 * kernels as in the forward: AUTO runs the tcgen05 dQ and dK/dV kernels for 16-bit
 * inputs with D = Dv in {64, 128} and no bias, the CUDA-core kernels otherwise;
 * `status` as in pjx_attn_fwd.  `dbias` (float32, shape and strides of `bias`, or NULL) receives
 * the gradient of a learnable dense bias, summed over the axes the bias broadcasts (with
 * atomic adds there, so that sum is not bit-repeatable). */
int pjx_attn_bwd_band(const void* q, const void* k, const void* v, const void* o, const float* lse,
                      const void* d_o, void* dq, void* dk, void* dv, const int32_t* kv_lengths,
                      const float* bias, int64_t bias_batch_stride, int64_t bias_head_stride,
                      float* dbias, int B, int Lq, int Lkv, int Hq, int Hkv, int D, int Dv, int dtype,
                      int band_lo, int band_hi, float sm_scale, int impl, void* workspace,
                      size_t workspace_bytes, int32_t* status, void* stream);
size_t pjx_attn_bwd_workspace_bytes(int B, int Lq, int Hq);
/* pjx_attn_bwd_band with score modifiers (mod may be NULL).  With modifiers the CUDA-core kernels
 * run; `dbias` cannot be combined with head_scale / softcap. */
int pjx_attn_bwd_mod(const void* q, const void* k, const void* v, const void* o, const float* lse,
                     const void* d_o, void* dq, void* dk, void* dv, const int32_t* kv_lengths,
                     const float* bias, int64_t bias_batch_stride, int64_t bias_head_stride,
                     float* dbias, int B, int Lq, int Lkv, int Hq, int Hkv, int D, int Dv, int dtype,
                     int band_lo, int band_hi, float sm_scale, const pjx_score_mod* mod, int impl,
                     void* workspace, size_t workspace_bytes, int32_t* status, void* stream);

/*
 * Forward-mode derivative of pjx_attn_fwd_band: the tangent t_o of o for tangents tq, tk, tv of
 * q, k, v (each may be NULL = zero), from the forward's natural-log lse.  Exact fp32 arithmetic
 * on CUDA cores, one pass over the keys.
 *
 * Replaces `mha_jvp_from_lse_kernel` (probjax/nn/pallas_kernels/kernels/attention.py:536-660),
 * the forward-mode path behind `diff_mode="forward"` (`jax.custom_jvp` wiring at 3303-3330).
 */
int pjx_attn_jvp_band(const void* q, const void* k, const void* v, const void* tq, const void* tk,
                      const void* tv, const float* lse, void* t_o, const int32_t* kv_lengths,
                      const float* bias, int64_t bias_batch_stride, int64_t bias_head_stride, int B,
                      int Lq, int Lkv, int Hq, int Hkv, int D, int Dv, int dtype, int band_lo,
                      int band_hi, float sm_scale, void* stream);
/* The same with score modifiers (mod may be NULL). */
int pjx_attn_jvp_mod(const void* q, const void* k, const void* v, const void* tq, const void* tk,
                     const void* tv, const float* lse, void* t_o, const int32_t* kv_lengths,
                     const float* bias, int64_t bias_batch_stride, int64_t bias_head_stride, int B,
                     int Lq, int Lkv, int Hq, int Hkv, int D, int Dv, int dtype, int band_lo,
                     int band_hi, float sm_scale, const pjx_score_mod* mod, void* stream);

/*
 * Split-KV decode forward over a KV cache with per-sequence valid lengths,
 * followed by the exact log-sum-exp combine of the per-split partials.
 *
 * Replaces `splitkv_forward` (probjax/nn/pallas_kernels/kernels/
 * attention_splitkv.py:137-250: kernel 43-103, GQA row packing 121-134,
 * combine 236-250) and, through kv_lengths, what `flex_attention(...,
 * mask=KVLenMask(lengths))` computes for a decode step
 * (probjax/nn/layers/attention.py:1426-1759).
 *
 *   k_cache, v_cache  [B, capacity, Hkv, D|Dv]; rows >= kv_lengths[b] are never read.
 *   kv_lengths        int32[B] or NULL (= capacity everywhere).
 *   o                 [B, Lq, Hq, Dv] in `dtype`, or float32 when o_is_f32 != 0
 *                     (the per-rank partial of a sequence-sharded decode).
 *   lse               [B, Hq, Lq] float32 natural log, or NULL.
 *   split_len         keys per split (multiple of 64), 0 = choose.
 *   workspace         pjx_attn_decode_workspace_bytes(...) bytes of device memory.
 */
int pjx_attn_decode_splitkv(const void* q, const void* k_cache, const void* v_cache,
                            const int32_t* kv_lengths, void* o, float* lse, int B, int Lq, int Hq,
                            int Hkv, int D, int Dv, int capacity, int dtype, float sm_scale,
                            int split_len, int o_is_f32, void* workspace, size_t workspace_bytes,
                            void* stream);
size_t pjx_attn_decode_workspace_bytes(int B, int Lq, int Hq, int Hkv, int Dv, int capacity,
                                       int split_len);
/* The split length pjx_attn_decode_splitkv uses when given split_len = 0. */
int pjx_attn_decode_default_split_len(int B, int Hkv, int capacity);

/*
 * The same decode for callers that cannot allocate device memory and are given
 * none to pass on: a serving loop inside a compiler-planned custom call (the
 * runtime hands it its operand and result buffers only and forbids cudaMalloc
 * there), or code running while the device allocator is locked or exhausted.
 * The per-split partials live in a fixed 16 MiB array inside the library
 * (pjx_attn_decode_static_scratch_bytes(); every GPU that loads the library
 * holds it until the process exits) instead of a workspace argument.  This entry
 * point has no counterpart in the reference.
 *
 *   - Takes what the streaming kernel takes: bf16/fp16, D = Dv in {64, 128},
 *     (Hq/Hkv)*Lq <= 16, 16-byte aligned q/k/v; anything else is
 *     PJX_ERR_UNSUPPORTED.  A call whose partials exceed the array is refused
 *     with PJX_ERR_WORKSPACE (choose a larger split_len, or use
 *     pjx_attn_decode_splitkv).  o is written in `dtype`.
 *   - It calls no cudaMalloc / cudaFree and no allocating library routine.
 *   - The first call on each device looks up the array's device address; make
 *     that first call before starting any stream capture.  The address is kept
 *     for the life of the process: it does not survive a cudaDeviceReset.
 *   - All calls share the array.  Nothing in it needs clearing between calls,
 *     but two calls whose kernels overlap on the GPU (different streams or
 *     threads) corrupt each other: order them on one stream.
 */
int pjx_attn_decode_splitkv_static(const void* q, const void* k_cache, const void* v_cache,
                                   const int32_t* kv_lengths, void* o, float* lse, int B, int Lq,
                                   int Hq, int Hkv, int D, int Dv, int capacity, int dtype,
                                   float sm_scale, int split_len, void* stream);
size_t pjx_attn_decode_static_scratch_bytes(void);

/*
 * Decode step with the KV sequence sharded over `world` GPUs (one process per
 * GPU).  Each rank passes its own shard (`k_local`, `v_local`, `local_lengths` =
 * valid tokens this rank holds per sequence) and the replicated q; every rank
 * gets the full result.  The exchange is fused into the kernels.  When the split
 * kernel's grid fits on the GPU at once (the default split length makes it so for
 * up to 296 (sequence, kv head) pairs) the whole step is ONE launch: the last CTA of
 * each (sequence, kv head) to finish combines the head's splits, writes the rank's
 * (o, lse) partial straight into every rank's exchange buffer with peer stores over
 * NVLink, raises that head's flag there, waits (bounded, about two seconds, then
 * PJX_ERR_DEVICE_TIMEOUT in `status`) for the same head's flag of every rank and
 * combines the partials out of local memory.  Larger grids use three launches
 * (split kernel, publish with one flag per rank, gather + combine) with the same
 * bounded wait.  Only stores cross NVLink; every load is local.
 *
 * Exchange buffer of one rank, N = B * Lq * Hq (identical on every rank):
 *   2 x { float o[world][N][Dv]; float lse[world][N]; }   halves alternate with step parity
 *   uint32 rank_flags[16]; uint32 counter;                (three-launch form)
 *   (padding to 16 bytes) uint32 unit_flags[world][N]; uint32 unit_counters[N];  (one-launch form)
 * Flags hold the step number of the last partial published.
 * It generalises the split combine of attention_splitkv.py:236-250 across GPUs;
 * the reference itself never shards the sequence axis (probjax/nn/sharding.py:70, 97).
 *
 *   exchange_buffers  host array of `world` device pointers: entry r is rank r's
 *                     exchange buffer (pjx_attn_decode_sharded_buffer_bytes bytes,
 *                     zero-filled before the first step, mapped into this process,
 *                     e.g. a torch symmetric-memory allocation).  All ranks pass the
 *                     same list.
 *   step              1, 2, 3, ... : every rank must make the same sequence of calls
 *                     with the same step numbers.
 *   flags             0, or PJX_DECODE_OVERLAP_PREVIOUS: the one-launch form is started as a
 *                     programmatic dependent launch and streams its cache while the kernel
 *                     launched just before it on `stream` is still finishing (it waits for that
 *                     kernel before it writes anything).  Set it only when that previous kernel
 *                     does not write this call's q, caches, lengths or block table -- e.g. it is
 *                     the previous step's call of this function, whose exchange then overlaps the
 *                     next step's streaming.
 *   o, lse            as pjx_attn_decode_splitkv (o in `dtype`).
 */
#define PJX_DECODE_OVERLAP_PREVIOUS 1
int pjx_attn_decode_sharded(const void* q, const void* k_local, const void* v_local,
                            const int32_t* local_lengths, void* o, float* lse, int B, int Lq, int Hq,
                            int Hkv, int D, int Dv, int capacity_local, int dtype, float sm_scale,
                            int split_len, void* workspace, size_t workspace_bytes, int rank,
                            int world, void* const* exchange_buffers, uint32_t step, int flags,
                            int32_t* status, void* stream);
size_t pjx_attn_decode_sharded_buffer_bytes(int B, int Lq, int Hq, int Dv, int world);
/* The same with this rank's share of the cache held in pages (the format of
 * pjx_attn_decode_paged): k_pool / v_pool [num_pages, page_size, Hkv, D|Dv], block_table int32
 * [B, max_pages] naming the local pages of every sequence in order, local_lengths the valid tokens
 * this rank holds.  The workspace is sized with capacity = max_pages * page_size.  No counterpart
 * in the reference (contiguous caches, no sequence sharding). */
int pjx_attn_decode_sharded_paged(const void* q, const void* k_pool, const void* v_pool,
                                  const int32_t* block_table, const int32_t* local_lengths, void* o,
                                  float* lse, int B, int Lq, int Hq, int Hkv, int D, int Dv,
                                  int page_size, int max_pages, int dtype, float sm_scale,
                                  int split_len, void* workspace, size_t workspace_bytes, int rank,
                                  int world, void* const* exchange_buffers, uint32_t step, int flags,
                                  int32_t* status, void* stream);

/*
 * Exact combine of n_parts normalised partial results, each with its natural-
 * log LSE: m = max_p lse_p, w_p = exp(lse_p - m), o = sum w_p o_p / sum w_p,
 * lse = m + log sum w_p (attention_splitkv.py:236-250, in natural log).  Used
 * after the all-gather of a sequence-sharded decode.
 *
 *   o_parts   float32 [n_parts, n_rows, Dv]     lse_parts float32 [n_parts, n_rows]
 *   o         [n_rows, Dv] in `dtype`           lse float32 [n_rows] or NULL
 */
int pjx_attn_combine(const float* o_parts, const float* lse_parts, int n_parts, int64_t n_rows,
                     int Dv, void* o, float* lse, int dtype, void* stream);

/*
 * pjx_attn_decode_splitkv over a paged cache: k_pool / v_pool are [num_pages, page_size, Hkv, D|Dv]
 * and logical key j of sequence b lives in page block_table[b * max_pages + j / page_size]
 * (int32 device array [B, max_pages]) at row j % page_size.  page_size is a multiple of 64 (the
 * kernel's key tile, so a tile never straddles a page); kv_lengths is required.  The workspace is
 * pjx_attn_decode_workspace_bytes(..., capacity = max_pages * page_size, split_len) bytes.
 *
 * No counterpart in the reference, whose caches are contiguous per sequence
 * (probjax/nn/layers/attention.py:727-757); it is the cache format a serving stack hands over.
 */
int pjx_attn_decode_paged(const void* q, const void* k_pool, const void* v_pool,
                          const int32_t* block_table, const int32_t* kv_lengths, void* o, float* lse,
                          int B, int Lq, int Hq, int Hkv, int D, int Dv, int page_size, int max_pages,
                          int dtype, float sm_scale, int split_len, void* workspace,
                          size_t workspace_bytes, void* stream);

/*
 * Decode KV-cache update: writes k_new [B, n_new, Hkv, D] and v_new [B, n_new, Hkv, Dv] into
 * the caches [B, capacity, Hkv, D|Dv] at rows positions[b] .. positions[b] + n_new - 1 and, if
 * `advance` is nonzero, adds n_new to positions[b] in the same launch (no host round trip:
 * append + pjx_attn_decode_splitkv with kv_lengths = positions is one graph-capturable step).
 *
 * Replaces the cache update of the attention layer's decode branch (probjax/nn/layers/
 * attention.py:631-643: dynamic_update_slice of cached_key / cached_value at cache_index, then
 * cache_index += 1), with one position per sequence instead of one shared index.
 *
 *   positions  int32 device array of 2 * B entries: [0, B) the positions, [B, 2B) scratch
 *              counters that must be zero on entry and are zero again on exit.
 *   overflow   optional int32 device word set to 1 if a sequence ran past `capacity` (its
 *              excess rows are dropped and its position saturates).
 */
int pjx_kv_cache_append(void* k_cache, void* v_cache, const void* k_new, const void* v_new,
                        int32_t* positions, int B, int capacity, int n_new, int Hkv, int D, int Dv,
                        int dtype, int advance, int32_t* overflow, void* stream);

/*
 * y [M, N] = x [M, K] . w [N, K]^T, fp32 accumulation, y in `dtype`: a bias-free linear layer
 * with the weight stored [out, in].  16-bit inputs with K >= 64, K % 8 == 0 and 16-byte aligned
 * operands run the persistent tcgen05 kernel (the one behind pjx_mla_fwd's up-projections),
 * anything else a CUDA-core kernel.
 *
 * Replaces the query / key / value / output projections around the attention call
 * (probjax/nn/layers/attention.py:591-594 and the output projection at the end of `__call__`).
 */
int pjx_linear(const void* x, const void* w, void* y, int64_t M, int N, int K, int dtype, int impl,
               int32_t* status, void* stream);

/* pjx_linear on a column block of wider matrices: row i of x starts at x + i * x_row_pitch and row i
 * of y at y + i * y_row_pitch (pitches in elements).  One call per head applies a per-head weight
 * to a [.., H, K] activation without gathering it, e.g. the value up-projection folded onto the
 * output of absorbed latent attention, einsum("...qhr,hdr->...qhd")
 * (probjax/nn/layers/latent_attention.py:468-474). */
int pjx_linear_strided(const void* x, int64_t x_row_pitch, const void* w, void* y, int64_t y_row_pitch,
                       int64_t M, int N, int K, int dtype, int impl, int32_t* status, void* stream);

/*
 * Root-mean-square normalisation of the rows of x [rows, width]: y = x * rsqrt(mean(x^2) + eps) *
 * scale (float32 [width] or NULL = ones), arithmetic in float32, y in `dtype` (may alias x).
 *
 * Replaces the `nnx.RMSNorm(kv_lora_rank)` the latent-attention layer applies to the encoded latent
 * before it is cached (probjax/nn/layers/latent_attention.py:313-319, 435-438).
 */
int pjx_rms_norm(const void* x, const float* scale, void* y, int64_t rows, int width, float eps,
                 int dtype, void* stream);

/*
 * Interleaved rotary position embedding of x [outer, T, H, D] into y (may alias x): pairs
 * (x[2i], x[2i+1]) with 2i < rotary_dim are rotated by pos * base^(-2i / rotary_dim); pos is
 * positions[t] (float32 [T]) or t + offset when positions is NULL.
 *
 * Replaces the rotary layer applied to queries / keys and to the latent layer's decoupled
 * rotary key (probjax/nn/layers/encoding.py:171-211, probjax/nn/layers/latent_attention.py:
 * 424-481).
 */
int pjx_rope_interleaved(const void* x, void* y, const float* positions, float offset, int64_t outer,
                         int T, int H, int D, int rotary_dim, float base, int dtype, void* stream);

/*
 * Latent attention forward: q over a shared latent cache with per-head
 * up-projections (wk, wv both given) or with K = V = cache (both NULL).
 *
 * Replaces the `mla_fwd` / `mla_fwd_absorbed` primitives
 * (probjax/nn/pallas_kernels/kernels/latent_attention.py:204-244, built by
 * `_mla_build` 247-377 around `_mla_forward_kernel` 79-197).
 *
 *   q [B, Lq, H, Dqk]  cache [B, S, R]  wk [H, Dqk, R]  wv [H, Dv, R]  o [B, Lq, H, Dv]
 *   workspace: pjx_mla_workspace_bytes(...) bytes; holds K = C.wk^T and V = C.wv^T.
 *
 * Without projections the call is multi-query attention of head width R.  Up to R = 256 the
 * regular forward kernels take it.  At R = 512 and 576 (bf16 / fp16, no bias, no score modifiers,
 * a mask without a lower band edge: none, causal, bottom-right causal, key lengths) every query
 * token runs as a one-token sequence of the absorbed latent decode kernels, whose partials live in
 * the workspace (pjx_mla_workspace_bytes with has_projections = 0); other calls at those widths
 * return PJX_ERR_UNSUPPORTED.
 */
int pjx_mla_fwd(const void* q, const void* cache, const void* wk, const void* wv, void* o,
                float* lse, const int32_t* kv_lengths, const float* bias,
                int64_t bias_batch_stride, int64_t bias_head_stride, int B, int Lq, int S, int H,
                int Dqk, int Dv, int R, int dtype, int causal, float sm_scale, int impl,
                void* workspace, size_t workspace_bytes, int32_t* status, void* stream);
size_t pjx_mla_workspace_bytes(int B, int S, int H, int Dqk, int Dv, int R, int dtype,
                               int has_projections);
/* pjx_mla_fwd with the band form of the mask and score modifiers (mod may be NULL): the masks and
 * biases `mla` shares with `mha` (latent_attention.py:636-766 takes the same mask / bias objects). */
int pjx_mla_fwd_mod(const void* q, const void* cache, const void* wk, const void* wv, void* o,
                    float* lse, const int32_t* kv_lengths, const float* bias,
                    int64_t bias_batch_stride, int64_t bias_head_stride, int B, int Lq, int S, int H,
                    int Dqk, int Dv, int R, int dtype, int band_lo, int band_hi, float sm_scale,
                    const pjx_score_mod* mod, int impl, void* workspace, size_t workspace_bytes,
                    int32_t* status, void* stream);

/*
 * Decode step of absorbed latent attention: q [B, Lq, H, R] over the latent cache [B, capacity, R]
 * with K = V = cache, per-sequence valid lengths, split along the keys and combined exactly.  Every
 * latent tile is read once and used for both products (half the bytes of a decode that streams K
 * and V), and the latent may be 128, 256, 512 or 576 wide (512 + 64 rotary columns); Lq <= 16.
 * o [B, Lq, H, R] in `dtype`; lse [B, H, Lq] natural log or NULL.
 *
 * Replaces the `mla_fwd_absorbed` primitive (probjax/nn/pallas_kernels/kernels/
 * latent_attention.py:204-244, 604-607) at decode time, where the reference's own split-KV rule
 * (kernels/attention.py:2653-2689) does not reach the latent kernel.
 */
int pjx_mla_decode_absorbed(const void* q, const void* cache, const int32_t* kv_lengths, void* o,
                            float* lse, int B, int Lq, int H, int R, int capacity, int dtype,
                            float sm_scale, int split_len, void* workspace, size_t workspace_bytes,
                            void* stream);
/* The same with a choice of kernel and a status word.  impl: PJX_IMPL_AUTO, PJX_IMPL_GENERIC (the
 * mma.sync kernel) or PJX_IMPL_SM100 (TMA + tcgen05: both products with the keys on the M axis of the
 * MMA, the latent tile loaded once into a ring of sub-tiles; chosen by AUTO when `status` is given).
 * `status` (device int32, may be NULL for the mma.sync kernel) receives PJX_ERR_DEVICE_TIMEOUT if
 * a bounded wait of the tcgen05 kernel expires.  No counterpart in the reference. */
int pjx_mla_decode_absorbed_impl(const void* q, const void* cache, const int32_t* kv_lengths, void* o,
                                 float* lse, int B, int Lq, int H, int R, int capacity, int dtype,
                                 float sm_scale, int split_len, int impl, void* workspace,
                                 size_t workspace_bytes, int32_t* status, void* stream);
size_t pjx_mla_decode_workspace_bytes(int B, int Lq, int H, int R, int capacity, int split_len);

/*
 * The forward with HOST buffers: copies q, k, v (and kv_lengths, bias) to the
 * device staging area, runs pjx_attn_fwd, copies o (and lse) back, and
 * synchronises the stream before returning.  The batch is processed in chunks so
 * that uploads, kernels and downloads overlap (two internal copy streams per
 * device, created on first use).  `staging` is device memory of
 * pjx_attn_fwd_host_staging_bytes(...) bytes owned by the caller.  Same
 * reference interface as pjx_attn_fwd; this is the call a host-side plugin
 * makes when its arrays live in host memory.
 */
int pjx_attn_fwd_host(const void* q, const void* k, const void* v, void* o, float* lse,
                      const int32_t* kv_lengths, const float* bias, int bias_batch, int bias_heads,
                      int B, int Lq, int Lkv, int Hq, int Hkv, int D, int Dv, int dtype,
                      int causal, float sm_scale, int impl, void* staging, size_t staging_bytes,
                      void* stream);
size_t pjx_attn_fwd_host_staging_bytes(int bias_batch, int bias_heads, int has_lse, int B, int Lq,
                                       int Lkv, int Hq, int Hkv, int D, int Dv, int dtype);

/* Synchronises `stream`, reads the device status word and returns it (0 = ok). */
int pjx_read_status(const int32_t* status, void* stream);

/* Number of this library's kernels launched by the calling process so far. */
int64_t pjx_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* PJX_ATTENTION_H_ */
