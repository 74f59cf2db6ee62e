// Structured masks and score modifiers evaluated inside the kernels, element by element, from
// O(B T) / O(H T) data -- never a [Q, K] tensor.  One descriptor covers the reference's classes
// (probjax/nn/pallas_kernels/attention_mask_bias.py):
//
//   seg_q / seg_k      keep iff seg_q[b, i] == seg_k[b, j]: SameSegmentMask 1537, BlockDiagonalMask
//                      871 (with the causal band: BlockDiagonalCausalMask 984); SeqLenMask 1239 and
//                      MarginalizationMask 1671 through ids that give every dropped token a segment
//                      of its own ((a_i & a_j) | i == j for a per-token keep vector a).
//   row_kv_limit       keep iff j < row_kv_limit[b, i]: KeyPaddingMask 1132 (per query row).
//   prefix_len         key j < prefix_len[b] is visible to every row, OR-ed with the band:
//                      PrefixLMMask 785 (band = causal).
//   rel_bias           s += rel_bias[h, (j - i) + Lq - 1]: any bias that depends on the head and the
//                      relative position only -- T5RelativePositionBias 2453 and
//                      LearnedRelativePositionBias 2521 (their bucket look-up done once per
//                      distance on the host), ConstantBias 1781.
//   alibi_slopes       s -= slope[h] * max(i - j, 0)  (mode 1, CausalAlibiBias 2230) or
//                      s -= slope[h] * |i - j|        (mode 2, SymmetricAlibiBias 2355,
//                      DistanceDecayBias 2387 with one slope for all heads).
//   head_scale         s += s * (head_scale[h] - 1): PerHeadScaleBias 2606.
//   softcap            s += softcap * tanh(s / softcap) - s: SoftCappingBias 2564.
//   dropout_rate,      counter-hash dropout (probjax/nn/pallas_kernels/kernels/attention.py:116-148,
//   dropout_seed       497-505): probability (b, h, i, j) is dropped when a 32-bit hash of
//                      (seed, b, h, i, j) falls below the rate, survivors are scaled by 1 / (1 - rate);
//                      applied to the probabilities after the row sum is accumulated.
//
// All score terms are deltas on the scaled score s = sm_scale q.k, summed the way SumBias 553
// sums them (every term sees the same s); a dense bias adds on top as before.  The derivative
// d s' / d s = 1 + (head_scale - 1) + (1 - tanh^2(s / softcap) - 1) is what the backward and
// the forward-mode kernels multiply dS with (the classes' `grad` methods, 2590-2601, 2637-2650).
#pragma once

#include <stdint.h>

namespace pjx {

struct ScoreMod {
  const int32_t* seg_q = nullptr;  // [Bs, Lq]
  const int32_t* seg_k = nullptr;  // [Bs, Lkv]
  int64_t seg_q_bs = 0, seg_k_bs = 0;  // element strides of the batch axis (0 = shared by the batch)
  const int32_t* row_kv_limit = nullptr;  // [Bs, Lq]
  int64_t row_limit_bs = 0;
  const int32_t* prefix_len = nullptr;  // [B]
  const float* rel_bias = nullptr;      // [Hr, Lq + Lkv - 1]
  int64_t rel_hs = 0;                   // element stride of the head axis (0 = shared by the heads)
  const float* alibi_slopes = nullptr;  // [Hq]
  int alibi_mode = 0;
  const float* head_scale = nullptr;  // [Hq]
  float softcap = 0.f;                // > 0: on
  float dropout_rate = 0.f;           // > 0: on
  uint32_t dropout_seed = 0;
  int on = 0;                         // any field set
  // Filled by the tcgen05 forward's launcher, not by callers: for every tile of 128 query rows the
  // range [first, last + 1) of keys whose segment id lies between the smallest and the largest id
  // of the tile's rows -- no key outside it can match a row of the tile, so the KV loop skips the
  // tiles outside (what the reference's block-sparse `index_offset` lists do for its kernels,
  // kernels/attention.py:1485-1566).  [Bs, tiles, 2]; batch stride in tiles (0 = shared).
  const int32_t* q_tile_range = nullptr;
  int64_t q_tile_range_bs = 0;

  __host__ __device__ bool has_mask() const { return seg_q || row_kv_limit || prefix_len; }
  __host__ __device__ bool nonlinear() const { return head_scale || softcap > 0.f; }
};

// Per-(batch, head) view: pointers advanced to the batch element, per-head scalars loaded.
struct ScoreModView {
  const int32_t* seg_q;
  const int32_t* seg_k;
  const int32_t* row_limit;
  const float* rel;  // already offset so that rel[j - i] is the entry of (i, j)
  int prefix;        // 0 when off
  float slope, hscale_m1, softcap;
  int alibi_mode;
  float drop_rate, drop_keep;  // rate (0 = off) and 1 / (1 - rate)
  uint32_t drop_base;          // seed mixed with the batch and head indices
};

__device__ __forceinline__ ScoreModView view_of(const ScoreMod& m, int b, int h, int Lq) {
  ScoreModView v;
  v.seg_q = m.seg_q ? m.seg_q + (int64_t)b * m.seg_q_bs : nullptr;
  v.seg_k = m.seg_k ? m.seg_k + (int64_t)b * m.seg_k_bs : nullptr;
  v.row_limit = m.row_kv_limit ? m.row_kv_limit + (int64_t)b * m.row_limit_bs : nullptr;
  v.rel = m.rel_bias ? m.rel_bias + (int64_t)h * m.rel_hs + (Lq - 1) : nullptr;
  v.prefix = m.prefix_len ? m.prefix_len[b] : 0;
  v.alibi_mode = m.alibi_slopes ? m.alibi_mode : 0;
  v.slope = m.alibi_slopes ? m.alibi_slopes[h] : 0.f;
  v.hscale_m1 = m.head_scale ? m.head_scale[h] - 1.f : 0.f;
  v.softcap = m.softcap;
  v.drop_rate = m.dropout_rate;
  v.drop_keep = m.dropout_rate > 0.f ? 1.f / (1.f - m.dropout_rate) : 1.f;
  v.drop_base = m.dropout_seed ^ (static_cast<uint32_t>(b) * 0x85EBCA6Bu) ^ (static_cast<uint32_t>(h) * 0xC2B2AE35u);
  return v;
}

// Multiplier of probability (i, j): 0 if the counter hash drops it, 1 / (1 - rate) otherwise
// (`_dropout_mask_counter`, kernels/attention.py:116-148: the same constants, shifts and the
// uint32 -> float32 conversion before the comparison).
__device__ __forceinline__ float mod_dropout(const ScoreModView& v, int i, int j) {
  if (v.drop_rate <= 0.f) return 1.f;
  uint32_t x = v.drop_base ^ (static_cast<uint32_t>(i) * 0x27D4EB2Fu) ^ (static_cast<uint32_t>(j) * 0x165667B1u);
  x ^= x >> 16;
  x *= 0x7FEB352Du;
  x ^= x >> 15;
  x *= 0x846CA68Bu;
  x ^= x >> 16;
  const float u = __uint2float_rn(x) * (1.0f / 4294967296.0f);
  return u < v.drop_rate ? 0.f : v.drop_keep;
}

// Mask part.  `band_keep` is the band test of (i, j); the key-length test is the caller's.
__device__ __forceinline__ bool mod_keep(const ScoreModView& v, bool band_keep, int i, int j) {
  bool keep = band_keep || j < v.prefix;
  if (v.seg_q) keep = keep && (v.seg_q[i] == v.seg_k[j]);
  if (v.row_limit) keep = keep && (j < v.row_limit[i]);
  return keep;
}

// Score part, natural-log domain: s is the scaled score; returns s' and, through `dsds`, d s'/d s.
template <bool EXACT>
__device__ __forceinline__ float mod_score(const ScoreModView& v, float s, int i, int j, float* dsds) {
  float out = s, g = 1.f;
  if (v.hscale_m1 != 0.f) {
    out = fmaf(s, v.hscale_m1, out);
    g += v.hscale_m1;
  }
  if (v.softcap > 0.f) {
    float t;
    if constexpr (EXACT) {
      t = tanhf(s / v.softcap);
    } else {
      asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(s / v.softcap));
    }
    out += v.softcap * t - s;
    g -= t * t;
  }
  if (v.rel) out += v.rel[j - i];
  if (v.alibi_mode == 1) out -= v.slope * (float)max(i - j, 0);
  else if (v.alibi_mode == 2) out -= v.slope * (float)abs(i - j);
  if (dsds) *dsds = g;
  return out;
}

}  // namespace pjx
