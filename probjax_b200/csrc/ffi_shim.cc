// XLA FFI handlers over the C ABI of libpjx_attention.so: what a jax.ffi custom call binds.
//
// One handler per entry point of include/pjx_attention.h that probjax's kernel primitives
// replace (probjax/core/custom_primitives/sharded_primitive.py:382-483 builds a primitive from
// a KernelSpec and an `impl`; the impl of the B200 path is `jax.ffi.ffi_call(<target>)`).
// Each handler only unpacks buffers, shapes and attributes and forwards to the C function, so
// everything the handlers can get wrong is argument order; the arithmetic is the tested library.
//
// Conventions shared by all handlers:
//   * The stream is XLA's (PlatformStream<cudaStream_t>); nothing synchronises.
//   * An optional operand that is absent is passed as a zero-element array (e.g. kv_lengths of
//     shape [0]); the handler turns it into NULL.
//   * Scratch memory is an extra result buffer (uint8) sized on the Python side by the matching
//     pjx_*_workspace_bytes function, so XLA plans it like any other buffer and the handler never
//     allocates.
//   * dims are read off the buffers: q [B, Lq, Hq, D], k [B, Lkv, Hkv, D], v [B, Lkv, Hkv, Dv].
//   * A pjx_status other than PJX_OK becomes an ffi::Error carrying pjx_last_error().
//
// Build (only where jaxlib's headers exist; `python -m probjax_b200.build --ffi` does this):
//   g++ -std=c++17 -shared -fPIC -I$(python -c "import jax.ffi; print(jax.ffi.include_dir())") \
//       -I include -I /usr/local/cuda/include probjax_b200/csrc/ffi_shim.cc \
//       -L probjax_b200 -lpjx_attention -Wl,-rpath,'$ORIGIN' -o probjax_b200/libpjx_ffi.so
#if __has_include("xla/ffi/api/ffi.h")

#include <cuda_runtime_api.h>

#include <cstdint>

#include "pjx_attention.h"
#include "xla/ffi/api/ffi.h"

namespace ffi = xla::ffi;

namespace {

int dtype_of(ffi::DataType t) {
  switch (t) {
    case ffi::DataType::F32: return PJX_F32;
    case ffi::DataType::BF16: return PJX_BF16;
    case ffi::DataType::F16: return PJX_F16;
    default: return -1;  // rejected by the library with its own message
  }
}

ffi::Error to_error(int rc) {
  if (rc == PJX_OK) return ffi::Error::Success();
  const ffi::ErrorCode code = rc == PJX_ERR_BAD_ARG       ? ffi::ErrorCode::kInvalidArgument
                              : rc == PJX_ERR_UNSUPPORTED ? ffi::ErrorCode::kUnimplemented
                              : rc == PJX_ERR_WORKSPACE   ? ffi::ErrorCode::kResourceExhausted
                                                          : ffi::ErrorCode::kInternal;
  return ffi::Error(code, pjx_last_error());
}

template <typename B>
void* data_or_null(B& buf) {
  return buf.element_count() == 0 ? nullptr : buf.untyped_data();
}

// Element strides of a [Bb, Hb, Lq, Lkv] bias with broadcast axes of extent 1.
void bias_strides(const ffi::AnyBuffer& bias, int64_t* bs, int64_t* hs) {
  *bs = *hs = 0;
  if (bias.element_count() == 0) return;
  auto d = bias.dimensions();
  const int64_t plane = d[2] * d[3];
  *hs = d[1] == 1 ? 0 : plane;
  *bs = d[0] == 1 ? 0 : d[1] * plane;
}

// ---- mha_fwd / mha_fwd_res (+ _gqa): probjax/nn/pallas_kernels/kernels/attention.py:2456-2565 ----
ffi::Error MhaFwd(cudaStream_t stream, ffi::AnyBuffer q, ffi::AnyBuffer k, ffi::AnyBuffer v,
                  ffi::AnyBuffer kv_lengths, ffi::AnyBuffer bias, ffi::Result<ffi::AnyBuffer> o,
                  ffi::Result<ffi::AnyBuffer> lse, ffi::Result<ffi::AnyBuffer> status, float sm_scale,
                  int32_t band_lo, int32_t band_hi) {
  auto qd = q.dimensions(), kd = k.dimensions(), vd = v.dimensions();
  int64_t bs, hs;
  bias_strides(bias, &bs, &hs);
  return to_error(pjx_attn_fwd_band(
      q.untyped_data(), k.untyped_data(), v.untyped_data(), o->untyped_data(),
      static_cast<float*>(data_or_null(*lse)), static_cast<const int32_t*>(data_or_null(kv_lengths)),
      static_cast<const float*>(data_or_null(bias)), bs, hs, (int)qd[0], (int)qd[1], (int)kd[1], (int)qd[2],
      (int)kd[2], (int)qd[3], (int)vd[3], dtype_of(q.element_type()), band_lo, band_hi, sm_scale, PJX_IMPL_AUTO,
      static_cast<int32_t*>(data_or_null(*status)), stream));
}

// ---- mha_bwd: kernels/attention.py:2509-2534 ----
ffi::Error MhaBwd(cudaStream_t stream, ffi::AnyBuffer q, ffi::AnyBuffer k, ffi::AnyBuffer v, ffi::AnyBuffer o,
                  ffi::AnyBuffer lse, ffi::AnyBuffer d_o, ffi::AnyBuffer kv_lengths, ffi::AnyBuffer bias,
                  ffi::Result<ffi::AnyBuffer> dq, ffi::Result<ffi::AnyBuffer> dk, ffi::Result<ffi::AnyBuffer> dv,
                  ffi::Result<ffi::AnyBuffer> dbias, ffi::Result<ffi::AnyBuffer> workspace,
                  ffi::Result<ffi::AnyBuffer> status, float sm_scale, int32_t band_lo, int32_t band_hi) {
  auto qd = q.dimensions(), kd = k.dimensions(), vd = v.dimensions();
  int64_t bs, hs;
  bias_strides(bias, &bs, &hs);
  // dbias accumulates: the kernels add into it, so it starts from zero
  if (dbias->element_count() > 0)
    cudaMemsetAsync(dbias->untyped_data(), 0, dbias->size_bytes(), stream);
  return to_error(pjx_attn_bwd_band(
      q.untyped_data(), k.untyped_data(), v.untyped_data(), o.untyped_data(),
      static_cast<const float*>(lse.untyped_data()), d_o.untyped_data(), dq->untyped_data(), dk->untyped_data(),
      dv->untyped_data(), static_cast<const int32_t*>(data_or_null(kv_lengths)),
      static_cast<const float*>(data_or_null(bias)), bs, hs, static_cast<float*>(data_or_null(*dbias)), (int)qd[0],
      (int)qd[1], (int)kd[1], (int)qd[2], (int)kd[2], (int)qd[3], (int)vd[3], dtype_of(q.element_type()), band_lo,
      band_hi, sm_scale, PJX_IMPL_AUTO, workspace->untyped_data(), workspace->size_bytes(),
      static_cast<int32_t*>(data_or_null(*status)), stream));
}

// ---- forward-mode rule: mha_jvp_from_lse_kernel, kernels/attention.py:536-660 ----
ffi::Error MhaJvp(cudaStream_t stream, ffi::AnyBuffer q, ffi::AnyBuffer k, ffi::AnyBuffer v, ffi::AnyBuffer tq,
                  ffi::AnyBuffer tk, ffi::AnyBuffer tv, ffi::AnyBuffer lse, ffi::AnyBuffer kv_lengths,
                  ffi::AnyBuffer bias, ffi::Result<ffi::AnyBuffer> t_o, float sm_scale, int32_t band_lo,
                  int32_t band_hi) {
  auto qd = q.dimensions(), kd = k.dimensions(), vd = v.dimensions();
  int64_t bs, hs;
  bias_strides(bias, &bs, &hs);
  return to_error(pjx_attn_jvp_band(
      q.untyped_data(), k.untyped_data(), v.untyped_data(), data_or_null(tq), data_or_null(tk), data_or_null(tv),
      static_cast<const float*>(lse.untyped_data()), t_o->untyped_data(),
      static_cast<const int32_t*>(data_or_null(kv_lengths)), static_cast<const float*>(data_or_null(bias)), bs, hs,
      (int)qd[0], (int)qd[1], (int)kd[1], (int)qd[2], (int)kd[2], (int)qd[3], (int)vd[3],
      dtype_of(q.element_type()), band_lo, band_hi, sm_scale, stream));
}

// ---- splitkv_forward: kernels/attention_splitkv.py:137-250 (no primitive there; pallas_call) ----
ffi::Error DecodeSplitKV(cudaStream_t stream, ffi::AnyBuffer q, ffi::AnyBuffer k_cache, ffi::AnyBuffer v_cache,
                         ffi::AnyBuffer kv_lengths, ffi::Result<ffi::AnyBuffer> o, ffi::Result<ffi::AnyBuffer> lse,
                         ffi::Result<ffi::AnyBuffer> workspace, float sm_scale, int32_t split_len) {
  auto qd = q.dimensions(), kd = k_cache.dimensions(), vd = v_cache.dimensions();
  return to_error(pjx_attn_decode_splitkv(
      q.untyped_data(), k_cache.untyped_data(), v_cache.untyped_data(),
      static_cast<const int32_t*>(data_or_null(kv_lengths)), o->untyped_data(),
      static_cast<float*>(data_or_null(*lse)), (int)qd[0], (int)qd[1], (int)qd[2], (int)kd[2], (int)qd[3],
      (int)vd[3], (int)kd[1], dtype_of(q.element_type()), sm_scale, split_len,
      o->element_type() == ffi::DataType::F32 && q.element_type() != ffi::DataType::F32, workspace->untyped_data(),
      workspace->size_bytes(), stream));
}

// The same without any workspace operand: for programs whose buffer plan cannot grow.
ffi::Error DecodeSplitKVStatic(cudaStream_t stream, ffi::AnyBuffer q, ffi::AnyBuffer k_cache,
                               ffi::AnyBuffer v_cache, ffi::AnyBuffer kv_lengths, ffi::Result<ffi::AnyBuffer> o,
                               ffi::Result<ffi::AnyBuffer> lse, float sm_scale, int32_t split_len) {
  auto qd = q.dimensions(), kd = k_cache.dimensions(), vd = v_cache.dimensions();
  return to_error(pjx_attn_decode_splitkv_static(
      q.untyped_data(), k_cache.untyped_data(), v_cache.untyped_data(),
      static_cast<const int32_t*>(data_or_null(kv_lengths)), o->untyped_data(),
      static_cast<float*>(data_or_null(*lse)), (int)qd[0], (int)qd[1], (int)qd[2], (int)kd[2], (int)qd[3],
      (int)vd[3], (int)kd[1], dtype_of(q.element_type()), sm_scale, split_len, stream));
}

// Paged cache: pools [P, page, Hkv, D], block_table int32 [B, max_pages].
ffi::Error DecodePaged(cudaStream_t stream, ffi::AnyBuffer q, ffi::AnyBuffer k_pool, ffi::AnyBuffer v_pool,
                       ffi::AnyBuffer block_table, ffi::AnyBuffer kv_lengths, ffi::Result<ffi::AnyBuffer> o,
                       ffi::Result<ffi::AnyBuffer> lse, ffi::Result<ffi::AnyBuffer> workspace, float sm_scale,
                       int32_t split_len) {
  auto qd = q.dimensions(), kd = k_pool.dimensions(), vd = v_pool.dimensions(), td = block_table.dimensions();
  return to_error(pjx_attn_decode_paged(
      q.untyped_data(), k_pool.untyped_data(), v_pool.untyped_data(),
      static_cast<const int32_t*>(block_table.untyped_data()), static_cast<const int32_t*>(kv_lengths.untyped_data()),
      o->untyped_data(), static_cast<float*>(data_or_null(*lse)), (int)qd[0], (int)qd[1], (int)qd[2], (int)kd[2],
      (int)qd[3], (int)vd[3], (int)kd[1], (int)td[1], dtype_of(q.element_type()), sm_scale, split_len,
      workspace->untyped_data(), workspace->size_bytes(), stream));
}

// Exact combine of partials (after an all-gather of a sequence-sharded decode).
ffi::Error Combine(cudaStream_t stream, ffi::AnyBuffer o_parts, ffi::AnyBuffer lse_parts,
                   ffi::Result<ffi::AnyBuffer> o, ffi::Result<ffi::AnyBuffer> lse) {
  auto d = o_parts.dimensions();  // [P, N, Dv]
  return to_error(pjx_attn_combine(static_cast<const float*>(o_parts.untyped_data()),
                                   static_cast<const float*>(lse_parts.untyped_data()), (int)d[0], d[1], (int)d[2],
                                   o->untyped_data(), static_cast<float*>(data_or_null(*lse)),
                                   dtype_of(o->element_type()), stream));
}

// ---- mla_fwd / mla_fwd_absorbed: kernels/latent_attention.py:204-244 ----
// wk / wv zero-element = absorbed.  q [B, Lq, H, Dqk], cache [B, S, R], wk [H, Dqk, R], wv [H, Dv, R].
ffi::Error MlaFwd(cudaStream_t stream, ffi::AnyBuffer q, ffi::AnyBuffer cache, ffi::AnyBuffer wk, ffi::AnyBuffer wv,
                  ffi::AnyBuffer kv_lengths, ffi::AnyBuffer bias, ffi::Result<ffi::AnyBuffer> o,
                  ffi::Result<ffi::AnyBuffer> lse, ffi::Result<ffi::AnyBuffer> workspace,
                  ffi::Result<ffi::AnyBuffer> status, float sm_scale, bool causal) {
  auto qd = q.dimensions(), cd = cache.dimensions(), od = o->dimensions();
  int64_t bs, hs;
  bias_strides(bias, &bs, &hs);
  return to_error(pjx_mla_fwd(
      q.untyped_data(), cache.untyped_data(), data_or_null(wk), data_or_null(wv), o->untyped_data(),
      static_cast<float*>(data_or_null(*lse)), static_cast<const int32_t*>(data_or_null(kv_lengths)),
      static_cast<const float*>(data_or_null(bias)), bs, hs, (int)qd[0], (int)qd[1], (int)cd[1], (int)qd[2],
      (int)qd[3], (int)od[3], (int)cd[2], dtype_of(q.element_type()), causal ? 1 : 0, sm_scale, PJX_IMPL_AUTO,
      data_or_null(*workspace), workspace->size_bytes(), static_cast<int32_t*>(data_or_null(*status)), stream));
}

// ---- the steps either side of the kernel ----
// y [M, N] = x [M, K] . w [N, K]^T (probjax/nn/layers/attention.py:591-594).
ffi::Error Linear(cudaStream_t stream, ffi::AnyBuffer x, ffi::AnyBuffer w, ffi::Result<ffi::AnyBuffer> y) {
  auto wd = w.dimensions();
  const int64_t K = wd[1];
  const int64_t M = K ? (int64_t)x.element_count() / K : 0;
  return to_error(pjx_linear(x.untyped_data(), w.untyped_data(), y->untyped_data(), M, (int)wd[0], (int)K,
                             dtype_of(x.element_type()), PJX_IMPL_AUTO, nullptr, stream));
}

// Interleaved rotary embedding (probjax/nn/layers/encoding.py:171-211); x [outer..., T, H, D].
ffi::Error Rope(cudaStream_t stream, ffi::AnyBuffer x, ffi::AnyBuffer positions, ffi::Result<ffi::AnyBuffer> y,
                float offset, int32_t rotary_dim, float base) {
  auto d = x.dimensions();
  const size_t n = d.size();
  const int T = (int)d[n - 3], H = (int)d[n - 2], D = (int)d[n - 1];
  const int64_t inner = (int64_t)T * H * D;
  const int64_t outer = inner ? (int64_t)x.element_count() / inner : 0;
  return to_error(pjx_rope_interleaved(x.untyped_data(), y->untyped_data(),
                                       static_cast<const float*>(data_or_null(positions)), offset, outer, T, H, D,
                                       rotary_dim, base, dtype_of(x.element_type()), stream));
}

// Decode cache update (probjax/nn/layers/attention.py:631-643).  The caches and the positions are
// both operands and results of the custom call; the Python side aliases each pair
// (input_output_aliases), so the result buffers ARE the operand buffers and are updated in place.
ffi::Error KvCacheAppend(cudaStream_t stream, ffi::AnyBuffer k_cache_in, ffi::AnyBuffer v_cache_in,
                         ffi::AnyBuffer k_new, ffi::AnyBuffer v_new, ffi::AnyBuffer positions_in,
                         ffi::Result<ffi::AnyBuffer> k_cache, ffi::Result<ffi::AnyBuffer> v_cache,
                         ffi::Result<ffi::AnyBuffer> positions, bool advance) {
  (void)k_cache_in; (void)v_cache_in; (void)positions_in;
  auto cd = k_cache->dimensions(), vd = v_cache->dimensions(), nd = k_new.dimensions();
  return to_error(pjx_kv_cache_append(k_cache->untyped_data(), v_cache->untyped_data(), k_new.untyped_data(),
                                      v_new.untyped_data(), static_cast<int32_t*>(positions->untyped_data()),
                                      (int)cd[0], (int)cd[1], (int)nd[1], (int)cd[2], (int)cd[3], (int)vd[3],
                                      dtype_of(k_new.element_type()), advance ? 1 : 0, nullptr, stream));
}

}  // namespace

#define PJX_STREAM ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>()
#define ARG .Arg<ffi::AnyBuffer>()
#define RET .Ret<ffi::AnyBuffer>()

XLA_FFI_DEFINE_HANDLER_SYMBOL(pjx_ffi_mha_fwd, MhaFwd,
                              PJX_STREAM ARG ARG ARG ARG ARG RET RET RET.Attr<float>("sm_scale")
                                  .Attr<int32_t>("band_lo")
                                  .Attr<int32_t>("band_hi"));
XLA_FFI_DEFINE_HANDLER_SYMBOL(pjx_ffi_mha_bwd, MhaBwd,
                              PJX_STREAM ARG ARG ARG ARG ARG ARG ARG ARG RET RET RET RET RET RET.Attr<float>("sm_scale")
                                  .Attr<int32_t>("band_lo")
                                  .Attr<int32_t>("band_hi"));
XLA_FFI_DEFINE_HANDLER_SYMBOL(pjx_ffi_mha_jvp, MhaJvp,
                              PJX_STREAM ARG ARG ARG ARG ARG ARG ARG ARG ARG RET.Attr<float>("sm_scale")
                                  .Attr<int32_t>("band_lo")
                                  .Attr<int32_t>("band_hi"));
XLA_FFI_DEFINE_HANDLER_SYMBOL(pjx_ffi_decode_splitkv, DecodeSplitKV,
                              PJX_STREAM ARG ARG ARG ARG RET RET RET.Attr<float>("sm_scale").Attr<int32_t>("split_len"));
XLA_FFI_DEFINE_HANDLER_SYMBOL(pjx_ffi_decode_splitkv_static, DecodeSplitKVStatic,
                              PJX_STREAM ARG ARG ARG ARG RET RET.Attr<float>("sm_scale").Attr<int32_t>("split_len"));
XLA_FFI_DEFINE_HANDLER_SYMBOL(pjx_ffi_decode_paged, DecodePaged,
                              PJX_STREAM ARG ARG ARG ARG ARG RET RET RET.Attr<float>("sm_scale").Attr<int32_t>("split_len"));
XLA_FFI_DEFINE_HANDLER_SYMBOL(pjx_ffi_combine, Combine, PJX_STREAM ARG ARG RET RET);
XLA_FFI_DEFINE_HANDLER_SYMBOL(pjx_ffi_mla_fwd, MlaFwd,
                              PJX_STREAM ARG ARG ARG ARG ARG ARG RET RET RET RET.Attr<float>("sm_scale").Attr<bool>("causal"));
XLA_FFI_DEFINE_HANDLER_SYMBOL(pjx_ffi_linear, Linear, PJX_STREAM ARG ARG RET);
XLA_FFI_DEFINE_HANDLER_SYMBOL(pjx_ffi_rope, Rope,
                              PJX_STREAM ARG ARG RET.Attr<float>("offset").Attr<int32_t>("rotary_dim").Attr<float>("base"));
XLA_FFI_DEFINE_HANDLER_SYMBOL(pjx_ffi_kv_cache_append, KvCacheAppend,
                              PJX_STREAM ARG ARG ARG ARG ARG RET RET RET.Attr<bool>("advance"));

#else  // no jaxlib headers on the include path

// Keeps `g++ -c ffi_shim.cc` meaningful on machines without jaxlib: the translation unit then
// only says why it is empty.
extern "C" const char* pjx_ffi_unavailable(void) {
  return "built without xla/ffi/api/ffi.h (jaxlib headers not found): no FFI handlers in this object";
}

#endif
