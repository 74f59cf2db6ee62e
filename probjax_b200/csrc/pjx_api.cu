// The C ABI: argument validation (mirroring the ValueErrors the reference raises
// for the same mistakes), kernel selection and the host-buffer convenience call.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "pjx_common.cuh"

namespace pjx {

static thread_local char g_err[512] = "";
static std::atomic<int64_t> g_launches{0};

int fail(int status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return status;
}
int check_cuda(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return PJX_OK;
  return fail(PJX_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

namespace {

inline size_t align_up(size_t x, size_t a = 256) { return (x + a - 1) / a * a; }

int validate_common(const void* q, const void* k, const void* v, const void* o, int B, int Lq, int Lkv,
                    int Hq, int Hkv, int D, int Dv, int dtype) {
  if (dtype != PJX_F32 && dtype != PJX_BF16 && dtype != PJX_F16)
    return fail(PJX_ERR_BAD_ARG, "dtype must be float32, bfloat16 or float16 (got code %d)", dtype);
  if (B < 0 || Lq < 0 || Lkv < 0 || Hq < 1 || Hkv < 1 || D < 1 || Dv < 1)
    return fail(PJX_ERR_BAD_ARG, "negative or zero dimension (B=%d Lq=%d Lkv=%d Hq=%d Hkv=%d D=%d Dv=%d)", B, Lq,
                Lkv, Hq, Hkv, D, Dv);
  if (Hq % Hkv != 0)
    return fail(PJX_ERR_BAD_ARG, "query heads %d must be a multiple of kv heads %d", Hq, Hkv);
  if (B > 0 && Lq > 0 && (!q || !o)) return fail(PJX_ERR_BAD_ARG, "q and o must not be null");
  if (B > 0 && Lkv > 0 && (!k || !v)) return fail(PJX_ERR_BAD_ARG, "k and v must not be null");
  return PJX_OK;
}

}  // namespace

// Validates a caller's pjx_score_mod and converts it to the kernels' form (null: no modifiers).
int convert_score_mod(const pjx_score_mod* m, ScoreMod* out) {
  *out = ScoreMod();
  if (!m) return PJX_OK;
  if ((m->seg_q == nullptr) != (m->seg_k == nullptr))
    return fail(PJX_ERR_BAD_ARG, "score modifiers: seg_q and seg_k come together (ids of the query rows and of the keys)");
  if (m->seg_q_batch_stride < 0 || m->seg_k_batch_stride < 0 || m->row_kv_limit_batch_stride < 0 || m->rel_bias_head_stride < 0)
    return fail(PJX_ERR_BAD_ARG, "score modifiers: strides must be non-negative");
  if (m->alibi_mode < 0 || m->alibi_mode > 2 || ((m->alibi_mode != 0) != (m->alibi_slopes != nullptr)))
    return fail(PJX_ERR_BAD_ARG, "score modifiers: alibi_mode is 1 (causal) or 2 (symmetric) with slopes, 0 without");
  if (!(m->softcap >= 0.f)) return fail(PJX_ERR_BAD_ARG, "score modifiers: softcap must be positive (0 = off)");
  if (!(m->dropout_rate >= 0.f && m->dropout_rate < 1.f))
    return fail(PJX_ERR_BAD_ARG, "score modifiers: dropout_rate must be in [0, 1), got %g", (double)m->dropout_rate);
  out->seg_q = m->seg_q; out->seg_k = m->seg_k;
  out->seg_q_bs = m->seg_q_batch_stride; out->seg_k_bs = m->seg_k_batch_stride;
  out->row_kv_limit = m->row_kv_limit; out->row_limit_bs = m->row_kv_limit_batch_stride;
  out->prefix_len = m->prefix_len;
  out->rel_bias = m->rel_bias; out->rel_hs = m->rel_bias_head_stride;
  out->alibi_slopes = m->alibi_slopes; out->alibi_mode = m->alibi_mode;
  out->head_scale = m->head_scale;
  out->softcap = m->softcap;
  out->dropout_rate = m->dropout_rate;
  out->dropout_seed = m->dropout_seed;
  out->on = (out->seg_q || out->row_kv_limit || out->prefix_len || out->rel_bias || out->alibi_slopes ||
             out->head_scale || out->softcap > 0.f || out->dropout_rate > 0.f) ? 1 : 0;
  return PJX_OK;
}

namespace {

// Streams and events of the host-buffer call, one set per device, created on first use.
constexpr int kHostChunks = 8;        // batch chunks of the host-buffer pipeline
constexpr int kHostQueryChunks = 4;   // query-row chunks inside a batch chunk
constexpr int kHostEvents = kHostChunks * kHostQueryChunks;
struct HostPipe {
  cudaStream_t in = nullptr, out = nullptr;
  cudaEvent_t start = nullptr, finish = nullptr, up[kHostEvents] = {}, done[kHostEvents] = {};
  bool ready = false;
  std::mutex busy;  // held for a whole host-buffer call: the events and copy streams are not re-entrant
};
std::mutex g_pipe_mu;
HostPipe g_pipes[64];

int host_pipe(HostPipe** out) {
  int dev = 0;
  int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice");
  if (rc) return rc;
  if (dev < 0 || dev >= 64) return fail(PJX_ERR_UNSUPPORTED, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_pipe_mu);
  HostPipe& p = g_pipes[dev];
  if (!p.ready) {
    if ((rc = check_cuda(cudaStreamCreateWithFlags(&p.in, cudaStreamNonBlocking), "create upload stream"))) return rc;
    if ((rc = check_cuda(cudaStreamCreateWithFlags(&p.out, cudaStreamNonBlocking), "create download stream"))) return rc;
    if ((rc = check_cuda(cudaEventCreateWithFlags(&p.start, cudaEventDisableTiming), "create event"))) return rc;
    if ((rc = check_cuda(cudaEventCreateWithFlags(&p.finish, cudaEventDisableTiming), "create event"))) return rc;
    for (int i = 0; i < kHostEvents; ++i) {
      if ((rc = check_cuda(cudaEventCreateWithFlags(&p.up[i], cudaEventDisableTiming), "create event"))) return rc;
      if ((rc = check_cuda(cudaEventCreateWithFlags(&p.done[i], cudaEventDisableTiming), "create event"))) return rc;
    }
    p.ready = true;
  }
  *out = &p;
  return PJX_OK;
}

}  // namespace

// Split length for split_len = 0.  Measured on B200 (B=16, Hkv=8, caches of 4k..32k keys, two CTAs per
// SM = 296 slots):
//  * all sequences full (no lengths given): a whole number of CTAs per (sequence, kv head) that fits ONE
//    wave streams fastest at every cache length (32k keys: 16384-key splits 7.08 TB/s, 4096-key splits
//    6.69; a partly filled last wave costs 5-6 %, and the idle 13 % of the slots cost nothing, the kernel
//    being bound by HBM);
//  * lengths given: sequences may be ragged, and then a CTA that owns a long split of a long sequence
//    is the straggler (one CTA cannot pull much more than its fair share of the bandwidth): splits of about
//    4096 keys in several waves balance best (ragged 1k..32k: 6.47 TB/s against 5.0 with 16384-key splits);
//  * small problems (fewer keys than one wave of 2048-key CTAs): one wave either way.
int decode_default_split_len(int B, int Hkv, int capacity, bool ragged) {
  if (B < 1 || Hkv < 1 || capacity < 1) return 64;
  const double total = (double)B * Hkv * capacity;
  const double slots = 148.0 * 2;
  const double len_fill = total / slots;
  const long units = (long)B * Hkv;
  double len;
  if (units <= (long)slots && (!ragged || len_fill < 2048.0)) {
    const long per_unit = (long)slots / units;  // >= 1
    len = (double)((capacity + per_unit - 1) / per_unit);
  } else {
    const double len_waves = total / (slots * 3.5);
    len = len_fill < 2048.0 ? len_fill : 2048.0;
    if (len_waves > len) len = len_waves;
  }
  long l64 = ((long)len + 63) / 64 * 64;
  if (l64 < 256) l64 = 256;
  const long cap64 = ((long)capacity + 63) / 64 * 64;
  if (l64 > cap64) l64 = cap64;
  return (int)l64;
}

}  // namespace pjx

using namespace pjx;

extern "C" {

int pjx_version(void) { return 100; }

const char* pjx_status_string(int status) {
  switch (status) {
    case PJX_OK: return "ok";
    case PJX_ERR_BAD_ARG: return "bad argument";
    case PJX_ERR_UNSUPPORTED: return "unsupported call";
    case PJX_ERR_WORKSPACE: return "workspace missing or too small";
    case PJX_ERR_DEVICE_TIMEOUT: return "a bounded wait inside a kernel expired";
    case PJX_ERR_CUDA: return "CUDA call failed";
  }
  return "unknown status";
}

const char* pjx_last_error(void) { return g_err; }

int64_t pjx_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int pjx_attn_fwd_band(const void* q, const void* k, const void* v, void* o, float* lse, const int32_t* kv_lengths,
                      const float* bias, int64_t bias_batch_stride, int64_t bias_head_stride, int B, int Lq, int Lkv,
                      int Hq, int Hkv, int D, int Dv, int dtype, int band_lo, int band_hi, float sm_scale, int impl,
                      int32_t* status, void* stream) {
  return pjx_attn_fwd_mod(q, k, v, o, lse, kv_lengths, bias, bias_batch_stride, bias_head_stride, B, Lq, Lkv, Hq, Hkv, D,
                          Dv, dtype, band_lo, band_hi, sm_scale, nullptr, impl, status, stream);
}

int pjx_attn_fwd_mod(const void* q, const void* k, const void* v, void* o, float* lse, const int32_t* kv_lengths,
                     const float* bias, int64_t bias_batch_stride, int64_t bias_head_stride, int B, int Lq, int Lkv,
                     int Hq, int Hkv, int D, int Dv, int dtype, int band_lo, int band_hi, float sm_scale,
                     const pjx_score_mod* mod, int impl, int32_t* status, void* stream) {
  int rc = validate_common(q, k, v, o, B, Lq, Lkv, Hq, Hkv, D, Dv, dtype);
  if (rc) return rc;
  ScoreMod sm;
  if ((rc = convert_score_mod(mod, &sm))) return rc;
  if (impl != PJX_IMPL_AUTO && impl != PJX_IMPL_GENERIC && impl != PJX_IMPL_SM100)
    return fail(PJX_ERR_BAD_ARG, "impl must be 0 (auto), 1 (generic) or 2 (tcgen05), got %d", impl);
  if (bias && (bias_batch_stride < 0 || bias_head_stride < 0))
    return fail(PJX_ERR_BAD_ARG, "bias strides must be non-negative");
  if (Lq >= PJX_BAND_NO_UPPER || Lkv >= PJX_BAND_NO_UPPER)
    return fail(PJX_ERR_BAD_ARG, "sequence lengths must be below 2^30");
  if (B == 0 || Lq == 0) return PJX_OK;
  FwdParams p;
  p.q = q; p.k = k; p.v = v; p.o = o; p.lse = lse;
  p.kv_lengths = kv_lengths;
  p.bias = bias; p.bias_bs = bias_batch_stride; p.bias_hs = bias_head_stride;
  p.B = B; p.Lq = Lq; p.Lkv = Lkv; p.Hq = Hq; p.Hkv = Hkv; p.D = D; p.Dv = Dv;
  p.band_lo = band_lo <= PJX_BAND_NO_LOWER ? PJX_BAND_NO_LOWER : band_lo;
  p.band_hi = band_hi >= PJX_BAND_NO_UPPER ? PJX_BAND_NO_UPPER : band_hi;
  if (p.band_lo > PJX_BAND_NO_UPPER) p.band_lo = PJX_BAND_NO_UPPER;  // nothing visible; keeps row + band in range
  if (p.band_hi < PJX_BAND_NO_LOWER) p.band_hi = PJX_BAND_NO_LOWER;
  p.causal = p.band_hi == 0 && p.band_lo == PJX_BAND_NO_LOWER;
  p.sm_scale = sm_scale;
  p.status = status;
  p.mod = sm;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (impl == PJX_IMPL_SM100) return launch_fwd_sm100(p, dtype, st);
  if (impl == PJX_IMPL_AUTO && fwd_sm100_supported(p, dtype, nullptr)) return launch_fwd_sm100(p, dtype, st);
  return launch_fwd_generic(p, dtype, st);
}

int pjx_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, const int32_t* kv_lengths,
                 const float* bias, int64_t bias_batch_stride, int64_t bias_head_stride, int B, int Lq, int Lkv,
                 int Hq, int Hkv, int D, int Dv, int dtype, int causal, float sm_scale, int impl, int32_t* status,
                 void* stream) {
  return pjx_attn_fwd_band(q, k, v, o, lse, kv_lengths, bias, bias_batch_stride, bias_head_stride, B, Lq, Lkv, Hq,
                           Hkv, D, Dv, dtype, PJX_BAND_NO_LOWER, causal ? 0 : PJX_BAND_NO_UPPER, sm_scale, impl,
                           status, stream);
}

int pjx_linear(const void* x, const void* w, void* y, int64_t M, int N, int K, int dtype, int impl, int32_t* status,
               void* stream) {
  if (dtype != PJX_F32 && dtype != PJX_BF16 && dtype != PJX_F16)
    return fail(PJX_ERR_BAD_ARG, "dtype must be float32, bfloat16 or float16 (got code %d)", dtype);
  if (M < 0 || N < 0 || K < 1) return fail(PJX_ERR_BAD_ARG, "linear: negative dimension or K < 1");
  if (impl != PJX_IMPL_AUTO && impl != PJX_IMPL_GENERIC && impl != PJX_IMPL_SM100)
    return fail(PJX_ERR_BAD_ARG, "impl must be 0 (auto), 1 (generic) or 2 (tcgen05), got %d", impl);
  if (M == 0 || N == 0) return PJX_OK;
  if (!x || !w || !y) return fail(PJX_ERR_BAD_ARG, "linear: null buffer");
  return launch_gemm_tn2(x, w, y, N, nullptr, nullptr, 0, M, K, dtype, impl, status, static_cast<cudaStream_t>(stream));
}

int pjx_linear_strided(const void* x, int64_t x_row_pitch, const void* w, void* y, int64_t y_row_pitch, int64_t M, int N,
                       int K, int dtype, int impl, int32_t* status, void* stream) {
  if (dtype != PJX_F32 && dtype != PJX_BF16 && dtype != PJX_F16)
    return fail(PJX_ERR_BAD_ARG, "dtype must be float32, bfloat16 or float16 (got code %d)", dtype);
  if (M < 0 || N < 0 || K < 1) return fail(PJX_ERR_BAD_ARG, "linear: negative dimension or K < 1");
  if (x_row_pitch < K || y_row_pitch < N) return fail(PJX_ERR_BAD_ARG, "linear: a row pitch is shorter than its row");
  if (impl != PJX_IMPL_AUTO && impl != PJX_IMPL_GENERIC && impl != PJX_IMPL_SM100)
    return fail(PJX_ERR_BAD_ARG, "impl must be 0 (auto), 1 (generic) or 2 (tcgen05), got %d", impl);
  if (M == 0 || N == 0) return PJX_OK;
  if (!x || !w || !y) return fail(PJX_ERR_BAD_ARG, "linear: null buffer");
  return launch_gemm_tn2(x, w, y, N, nullptr, nullptr, 0, M, K, dtype, impl, status, static_cast<cudaStream_t>(stream),
                         x_row_pitch, y_row_pitch);
}

int pjx_attn_decode_default_split_len(int B, int Hkv, int capacity) {
  return decode_default_split_len(B, Hkv, capacity, true);
}

// Limits every decode entry point shares: index arithmetic in int and a (split, kv head, batch) grid.
static int decode_limits(int B, int Hkv, int capacity) {
  if (capacity >= PJX_BAND_NO_UPPER) return fail(PJX_ERR_UNSUPPORTED, "decode: cache capacity must be below 2^30 (got %d)", capacity);
  if (B > 65535 || Hkv > 65535)
    return fail(PJX_ERR_UNSUPPORTED, "decode: at most 65535 sequences and 65535 kv heads per call (got B=%d, Hkv=%d)", B, Hkv);
  return PJX_OK;
}

static int decode_geometry(int B, int Hkv, int capacity, int split_len, int* out_len, int* out_splits,
                           bool ragged = true) {
  if (split_len == 0) split_len = decode_default_split_len(B, Hkv, capacity, ragged);
  if (split_len < 64 || split_len % 64 != 0)
    return fail(PJX_ERR_BAD_ARG, "split_len must be a positive multiple of 64 (got %d)", split_len);
  *out_len = split_len;
  *out_splits = capacity > 0 ? (capacity + split_len - 1) / split_len : 1;
  return PJX_OK;
}

static size_t decode_partial_bytes(size_t parts, int Dv) {
  return align_up(parts * Dv * sizeof(float)) + align_up(parts * sizeof(float));
}

size_t pjx_attn_decode_workspace_bytes(int B, int Lq, int Hq, int Hkv, int Dv, int capacity, int split_len) {
  if (B < 1 || Hkv < 1 || Hq < 1 || Lq < 1 || Dv < 1 || Hq % Hkv) return 0;
  const size_t rows = (size_t)(Hq / Hkv) * Lq;
  size_t need = 0;
  for (int ragged = 0; ragged < 2; ++ragged) {  // split_len = 0: enough for either default
    int len, ns;
    if (decode_geometry(B, Hkv, capacity, split_len, &len, &ns, ragged != 0)) return 0;
    const size_t n = decode_partial_bytes((size_t)B * Hkv * ns * rows, Dv);
    if (n > need) need = n;
  }
  return need;
}

// Points p at its partial arrays in `workspace` for fixed splits of `split_len` keys (0 = choose).
static int decode_place_partials(DecodeParams& p, int dtype, int split_len, void* workspace, size_t workspace_bytes,
                                 bool allow_flat) {
  (void)dtype; (void)allow_flat;
  int rc;
  if ((rc = decode_geometry(p.B, p.Hkv, p.capacity, split_len, &p.split_len, &p.num_splits, p.kv_lengths != nullptr)))
    return rc;
  const size_t parts = (size_t)p.B * p.Hkv * p.num_splits * p.rows;
  const size_t need = decode_partial_bytes(parts, p.Dv);
  if (!workspace || workspace_bytes < need)
    return fail(PJX_ERR_WORKSPACE, "decode workspace: need %zu bytes, got %zu", need, workspace ? workspace_bytes : (size_t)0);
  p.o_part = static_cast<float*>(workspace);
  p.lse_part = reinterpret_cast<float*>(static_cast<char*>(workspace) + align_up(parts * p.Dv * sizeof(float)));
  return PJX_OK;
}

int pjx_attn_decode_splitkv(const void* q, const void* k_cache, const void* v_cache, const int32_t* kv_lengths,
                            void* o, float* lse, int B, int Lq, int Hq, int Hkv, int D, int Dv, int capacity,
                            int dtype, float sm_scale, int split_len, int o_is_f32, void* workspace,
                            size_t workspace_bytes, void* stream) {
  int rc = validate_common(q, k_cache, v_cache, o, B, Lq, capacity, Hq, Hkv, D, Dv, dtype);
  if (rc) return rc;
  if ((rc = decode_limits(B, Hkv, capacity))) return rc;
  if (B == 0 || Lq == 0) return PJX_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  DecodeParams p;
  p.q = q; p.k = k_cache; p.v = v_cache; p.kv_lengths = kv_lengths; p.o = o; p.lse = lse;
  p.B = B; p.Lq = Lq; p.Hq = Hq; p.Hkv = Hkv; p.D = D; p.Dv = Dv; p.capacity = capacity;
  p.rows = (Hq / Hkv) * Lq;
  p.sm_scale = sm_scale;
  p.o_is_f32 = o_is_f32 != 0;
  const bool aligned =
      ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache)) & 15) == 0;
  if (!decode_fast_supported(p, dtype) || !aligned || capacity == 0) {
    // Shapes the streaming kernel does not take: the generic forward with the
    // key-length mask computes the same function.
    if (o_is_f32 && dtype != PJX_F32)
      return fail(PJX_ERR_UNSUPPORTED, "float32 partial output needs the split-KV kernel (bf16/fp16, D = Dv in {64,128}, (Hq/Hkv)*Lq <= 16)");
    return pjx_attn_fwd(q, k_cache, v_cache, o, lse, kv_lengths, nullptr, 0, 0, B, Lq, capacity, Hq, Hkv, D, Dv,
                        dtype, 0, sm_scale, PJX_IMPL_GENERIC, nullptr, stream);
  }
  if ((rc = decode_place_partials(p, dtype, split_len, workspace, workspace_bytes, true))) return rc;
  return launch_decode(p, dtype, st);
}

int pjx_attn_decode_paged(const void* q, const void* k_pool, const void* v_pool, const int32_t* block_table,
                          const int32_t* kv_lengths, void* o, float* lse, int B, int Lq, int Hq, int Hkv, int D, int Dv,
                          int page_size, int max_pages, int dtype, float sm_scale, int split_len, void* workspace,
                          size_t workspace_bytes, void* stream) {
  if (page_size < 64 || page_size % 64 != 0)
    return fail(PJX_ERR_BAD_ARG, "page_size must be a positive multiple of 64 (got %d)", page_size);
  if (max_pages < 0 || (int64_t)max_pages * page_size >= PJX_BAND_NO_UPPER)
    return fail(PJX_ERR_BAD_ARG, "max_pages * page_size must be below 2^30");
  const int capacity = max_pages * page_size;
  int rc = validate_common(q, k_pool, v_pool, o, B, Lq, capacity, Hq, Hkv, D, Dv, dtype);
  if (rc) return rc;
  if ((rc = decode_limits(B, Hkv, capacity))) return rc;
  if (B == 0 || Lq == 0) return PJX_OK;
  if (!block_table || !kv_lengths) return fail(PJX_ERR_BAD_ARG, "paged decode needs a block table and key lengths");
  DecodeParams p;
  p.q = q; p.k = k_pool; p.v = v_pool; p.kv_lengths = kv_lengths; p.o = o; p.lse = lse;
  p.B = B; p.Lq = Lq; p.Hq = Hq; p.Hkv = Hkv; p.D = D; p.Dv = Dv; p.capacity = capacity;
  p.rows = (Hq / Hkv) * Lq;
  p.sm_scale = sm_scale;
  p.o_is_f32 = 0;
  p.block_table = block_table; p.page_size = page_size; p.max_pages = max_pages;
  const bool aligned =
      ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_pool) | reinterpret_cast<uintptr_t>(v_pool)) & 15) == 0;
  if (!decode_fast_supported(p, dtype) || !aligned || capacity == 0)
    return fail(PJX_ERR_UNSUPPORTED,
                "the paged decode takes bf16/fp16, D = Dv in {64,128}, (Hq/Hkv)*Lq <= 16, at least one page and 16-byte aligned q/k/v");
  if ((rc = decode_place_partials(p, dtype, split_len, workspace, workspace_bytes, true))) return rc;
  return launch_decode(p, dtype, static_cast<cudaStream_t>(stream));
}

size_t pjx_attn_decode_sharded_buffer_bytes(int B, int Lq, int Hq, int Dv, int world) {
  if (B < 1 || Lq < 1 || Hq < 1 || Dv < 1 || world < 1 || world > kMaxExchangeRanks) return 0;
  return align_up(exchange_buffer_bytes(world, (int64_t)B * Lq * Hq, Dv));
}

// Shared body of the two sharded entry points (contiguous local cache, or local pages).
static int decode_sharded_impl(const void* q, const void* k_local, const void* v_local, const int32_t* block_table,
                               int page_size, int max_pages, const int32_t* local_lengths, void* o, float* lse, int B,
                               int Lq, int Hq, int Hkv, int D, int Dv, int capacity_local, int dtype, float sm_scale,
                               int split_len, void* workspace, size_t workspace_bytes, int rank, int world,
                               void* const* exchange_buffers, uint32_t step, int flags, int32_t* status, void* stream) {
  int rc = validate_common(q, k_local, v_local, o, B, Lq, capacity_local, Hq, Hkv, D, Dv, dtype);
  if (flags & ~PJX_DECODE_OVERLAP_PREVIOUS) return fail(PJX_ERR_BAD_ARG, "unknown flag bits 0x%x", flags);
  if (rc) return rc;
  if (world < 1 || world > kMaxExchangeRanks || rank < 0 || rank >= world)
    return fail(PJX_ERR_BAD_ARG, "rank %d / world %d out of range (at most %d ranks)", rank, world, kMaxExchangeRanks);
  if (!exchange_buffers) return fail(PJX_ERR_BAD_ARG, "exchange_buffers must hold one device pointer per rank");
  for (int i = 0; i < world; ++i)
    if (!exchange_buffers[i] || (reinterpret_cast<uintptr_t>(exchange_buffers[i]) & 15))
      return fail(PJX_ERR_BAD_ARG, "exchange buffer of rank %d is null or not 16-byte aligned", i);
  if (step == 0) return fail(PJX_ERR_BAD_ARG, "step counts from 1 and must grow by one per call");
  if ((rc = decode_limits(B, Hkv, capacity_local))) return rc;
  if (B == 0 || Lq == 0) return PJX_OK;
  DecodeParams p;
  p.q = q; p.k = k_local; p.v = v_local; p.kv_lengths = local_lengths; p.o = o; p.lse = lse;
  p.B = B; p.Lq = Lq; p.Hq = Hq; p.Hkv = Hkv; p.D = D; p.Dv = Dv; p.capacity = capacity_local;
  p.rows = (Hq / Hkv) * Lq;
  p.sm_scale = sm_scale;
  p.o_is_f32 = 0;
  p.block_table = block_table; p.page_size = page_size; p.max_pages = max_pages;
  const bool aligned =
      ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_local) | reinterpret_cast<uintptr_t>(v_local)) & 15) == 0;
  if (!decode_fast_supported(p, dtype) || !aligned || capacity_local == 0)
    return fail(PJX_ERR_UNSUPPORTED,
                "the sharded decode takes bf16/fp16, D = Dv in {64,128}, (Hq/Hkv)*Lq <= 16, a non-empty local cache and 16-byte aligned q/k/v");
  if (split_len == 0 && (int64_t)B * Hkv <= 296) {
    // one wave of CTAs whatever the cache length: the exchange then runs inside the split kernel
    const int per_unit = 296 / (B * Hkv);
    int len = ((capacity_local + per_unit - 1) / per_unit + 63) / 64 * 64;
    split_len = len < 256 ? 256 : len;
  }
  if ((rc = decode_geometry(B, Hkv, capacity_local, split_len, &p.split_len, &p.num_splits))) return rc;
  const size_t need = pjx_attn_decode_workspace_bytes(B, Lq, Hq, Hkv, Dv, capacity_local, p.split_len);
  if (!workspace || workspace_bytes < need)
    return fail(PJX_ERR_WORKSPACE, "decode workspace: need %zu bytes, got %zu", need, workspace ? workspace_bytes : (size_t)0);
  const size_t parts = (size_t)B * Hkv * p.num_splits * p.rows;
  p.o_part = static_cast<float*>(workspace);
  p.lse_part = reinterpret_cast<float*>(static_cast<char*>(workspace) + align_up(parts * Dv * sizeof(float)));
  p.ex_world = world; p.ex_rank = rank; p.ex_step = step; p.status = status;
  // The one-kernel exchange has CTAs wait for peers while they hold their SM slots, so it is
  // only used when every CTA of the grid is resident at once; larger grids take three kernels.
  int slots = 0;
  if ((rc = decode_coresident_ctas(dtype, D, &slots))) return rc;
  p.ex_fused = ((int64_t)p.num_splits * Hkv * B <= slots) && (reinterpret_cast<uintptr_t>(o) & 7) == 0;
  p.ex_overlap = (flags & PJX_DECODE_OVERLAP_PREVIOUS) ? 1 : 0;  // only the one-launch form uses it
  for (int i = 0; i < world; ++i) p.ex_buf[i] = static_cast<unsigned char*>(exchange_buffers[i]);
  return launch_decode(p, dtype, static_cast<cudaStream_t>(stream));
}

int pjx_attn_decode_sharded(const void* q, const void* k_local, const void* v_local, const int32_t* local_lengths,
                            void* o, float* lse, int B, int Lq, int Hq, int Hkv, int D, int Dv, int capacity_local,
                            int dtype, float sm_scale, int split_len, void* workspace, size_t workspace_bytes,
                            int rank, int world, void* const* exchange_buffers, uint32_t step, int flags,
                            int32_t* status, void* stream) {
  return decode_sharded_impl(q, k_local, v_local, nullptr, 0, 0, local_lengths, o, lse, B, Lq, Hq, Hkv, D, Dv,
                             capacity_local, dtype, sm_scale, split_len, workspace, workspace_bytes, rank, world,
                             exchange_buffers, step, flags, status, stream);
}

int pjx_attn_decode_sharded_paged(const void* q, const void* k_pool, const void* v_pool, const int32_t* block_table,
                                  const int32_t* local_lengths, void* o, float* lse, int B, int Lq, int Hq, int Hkv,
                                  int D, int Dv, int page_size, int max_pages, int dtype, float sm_scale, int split_len,
                                  void* workspace, size_t workspace_bytes, int rank, int world,
                                  void* const* exchange_buffers, uint32_t step, int flags, int32_t* status,
                                  void* stream) {
  if (page_size < 64 || page_size % 64 != 0)
    return fail(PJX_ERR_BAD_ARG, "page_size must be a positive multiple of 64 (got %d)", page_size);
  if (max_pages < 1 || (int64_t)max_pages * page_size >= PJX_BAND_NO_UPPER)
    return fail(PJX_ERR_BAD_ARG, "max_pages * page_size must be positive and below 2^30");
  if (!block_table || !local_lengths) return fail(PJX_ERR_BAD_ARG, "paged decode needs a block table and key lengths");
  return decode_sharded_impl(q, k_pool, v_pool, block_table, page_size, max_pages, local_lengths, o, lse, B, Lq, Hq, Hkv,
                             D, Dv, max_pages * page_size, dtype, sm_scale, split_len, workspace, workspace_bytes, rank,
                             world, exchange_buffers, step, flags, status, stream);
}

int pjx_attn_combine(const float* o_parts, const float* lse_parts, int n_parts, int64_t n_rows, int Dv, void* o,
                     float* lse, int dtype, void* stream) {
  if (n_parts < 1 || n_rows < 0 || Dv < 1) return fail(PJX_ERR_BAD_ARG, "combine: n_parts=%d n_rows=%lld Dv=%d", n_parts, (long long)n_rows, Dv);
  if (n_rows > 0 && (!o_parts || !lse_parts || !o)) return fail(PJX_ERR_BAD_ARG, "combine: null buffer");
  if (n_rows > 2147483647LL) return fail(PJX_ERR_UNSUPPORTED, "combine: too many rows");
  return launch_combine_parts(o_parts, lse_parts, n_parts, n_rows, Dv, o, lse, dtype, static_cast<cudaStream_t>(stream));
}

// Row groups of the absorbed latent decode: the largest number of heads per group that divides H
// and keeps heads x query tokens within the 16 rows of one tensor-core operand.
static int latent_heads_per_group(int H, int Lq) {
  if (Lq < 1 || Lq > 16) return 0;
  for (int g = 16 / Lq; g >= 1; --g)
    if (H % g == 0) return g;
  return 0;
}

static int latent_decode_split_len(int B, int groups, int capacity, int split_len) {
  if (split_len != 0) return split_len;
  // one CTA per SM (148): a whole number of CTAs per (sequence, row group) that fills one wave
  const int64_t units = (int64_t)B * groups;
  const int64_t per_unit = units >= 148 ? 1 : 148 / units;
  int64_t len = ((capacity + per_unit - 1) / per_unit + 63) / 64 * 64;
  if (len < 256) len = 256;
  return (int)len;
}

size_t pjx_mla_decode_workspace_bytes(int B, int Lq, int H, int R, int capacity, int split_len) {
  const int gh = latent_heads_per_group(H, Lq);
  if (B < 1 || H < 1 || R < 1 || capacity < 1 || gh == 0) return 0;
  const int groups = H / gh;
  const int len = latent_decode_split_len(B, groups, capacity, split_len);
  if (len < 64 || len % 64) return 0;
  const size_t ns = ((size_t)capacity + len - 1) / len;
  const size_t parts = (size_t)B * groups * ns * gh * Lq;
  return align_up(parts * R * sizeof(float)) + align_up(parts * sizeof(float));
}

int pjx_mla_decode_absorbed(const void* q, const void* cache, const int32_t* kv_lengths, void* o, float* lse, int B,
                            int Lq, int H, int R, int capacity, int dtype, float sm_scale, int split_len,
                            void* workspace, size_t workspace_bytes, void* stream) {
  return pjx_mla_decode_absorbed_impl(q, cache, kv_lengths, o, lse, B, Lq, H, R, capacity, dtype, sm_scale, split_len,
                                      PJX_IMPL_AUTO, workspace, workspace_bytes, nullptr, stream);
}

int pjx_mla_decode_absorbed_impl(const void* q, const void* cache, const int32_t* kv_lengths, void* o, float* lse,
                                 int B, int Lq, int H, int R, int capacity, int dtype, float sm_scale, int split_len,
                                 int impl, void* workspace, size_t workspace_bytes, int32_t* status, void* stream) {
  if (B < 0 || Lq < 0 || H < 1 || R < 1 || capacity < 0) return fail(PJX_ERR_BAD_ARG, "mla decode: bad dimension");
  int rc = decode_limits(B, H, capacity);
  if (rc) return rc;
  if (B == 0 || Lq == 0) return PJX_OK;
  if (!q || !cache || !o) return fail(PJX_ERR_BAD_ARG, "mla decode: null buffer");
  const int gh = latent_heads_per_group(H, Lq);
  const bool aligned = ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(cache)) & 15) == 0;
  if (gh == 0 || !decode_latent_supported(R, dtype) || !aligned || capacity == 0)
    return fail(PJX_ERR_UNSUPPORTED,
                "the absorbed latent decode takes bf16/fp16, a latent width of 128, 256, 512 or 576, at most 16 query "
                "tokens, a non-empty cache and 16-byte aligned q / cache");
  DecodeParams p;
  p.q = q; p.k = cache; p.v = cache; p.kv_lengths = kv_lengths; p.o = o; p.lse = lse;
  p.B = B; p.Lq = Lq; p.Hq = H; p.Hkv = H / gh; p.D = R; p.Dv = R; p.capacity = capacity;
  p.rows = gh * Lq;
  p.sm_scale = sm_scale;
  p.o_is_f32 = 0;
  p.split_len = latent_decode_split_len(B, p.Hkv, capacity, split_len);
  if (p.split_len < 64 || p.split_len % 64 != 0)
    return fail(PJX_ERR_BAD_ARG, "split_len must be a positive multiple of 64 (got %d)", p.split_len);
  p.num_splits = (capacity + p.split_len - 1) / p.split_len;
  const size_t need = pjx_mla_decode_workspace_bytes(B, Lq, H, R, capacity, p.split_len);
  if (!workspace || workspace_bytes < need)
    return fail(PJX_ERR_WORKSPACE, "mla decode workspace: need %zu bytes, got %zu", need, workspace ? workspace_bytes : (size_t)0);
  const size_t parts = (size_t)B * p.Hkv * p.num_splits * p.rows;
  p.o_part = static_cast<float*>(workspace);
  p.lse_part = reinterpret_cast<float*>(static_cast<char*>(workspace) + align_up(parts * R * sizeof(float)));
  p.status = status;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (impl != PJX_IMPL_AUTO && impl != PJX_IMPL_GENERIC && impl != PJX_IMPL_SM100)
    return fail(PJX_ERR_BAD_ARG, "mla decode: unknown impl %d", impl);
  // AUTO: the tcgen05 kernel where the step streams at least 64 MiB of latent (measured 13-57 % faster there:
  // B16 H16 R576 32k keys 4.28 against 3.78 TB/s, B64 8k keys 4.67 against 3.65, H = 128 0.76 against 1.20 ms);
  // below that the two are within a few per cent and the mma.sync kernel has the shorter prologue
  const bool big = (double)B * p.Hkv * capacity * R * 2.0 >= 64.0 * 1024 * 1024;
  const bool tc = (impl == PJX_IMPL_SM100 || (impl == PJX_IMPL_AUTO && big)) && decode_latent_tc_supported(p, dtype);
  if (impl == PJX_IMPL_SM100 && !tc)
    return fail(PJX_ERR_UNSUPPORTED, "the tcgen05 latent decode needs a status word and a cache of fewer than 2^31 rows");
  if ((rc = tc ? launch_decode_latent_tc_splits(p, dtype, st) : launch_decode_latent_splits(p, dtype, st))) return rc;
  return launch_decode_combine(p, dtype, st);
}

// ---------------------------------------------------------------------------
// Absorbed latent attention over many query tokens at latent widths the regular
// forward kernels do not take (R = 512, 576): every query token becomes a
// one-token sequence of the latent decode kernels -- its 16 heads are the 16 rows
// of the tensor-core operand, its keys are the cache row's keys up to its band
// limit -- and the tokens are walked in chunks so that the partials stay small.
// ---------------------------------------------------------------------------
static constexpr int kAbsorbedPrefillSeqs = 2048;  // one-token sequences per launch (rounded to whole batch rows)

static int absorbed_prefill_chunk(int B, int Lq) {
  int t = kAbsorbedPrefillSeqs / (B < 1 ? 1 : B);
  if (t < 1) t = 1;
  return t < Lq ? t : Lq;
}

static size_t absorbed_prefill_parts(int B, int H) {
  const int gh = latent_heads_per_group(H, 1);
  if (gh == 0 || B < 1) return 0;
  size_t units = (size_t)B * (kAbsorbedPrefillSeqs / B < 1 ? 1 : kAbsorbedPrefillSeqs / B) * (H / gh);
  if (units < 148) units = 148;  // fewer units are cut into at most 148 splits in all
  return units * gh;
}

static bool absorbed_prefill_applies(int H, int R, int dtype, int band_lo, const float* bias, const pjx_score_mod* mod,
                                     const void* q, const void* cache) {
  if (R <= 256 || !decode_latent_supported(R, dtype) || latent_heads_per_group(H, 1) == 0) return false;
  if (bias || mod || band_lo > PJX_BAND_NO_LOWER) return false;
  return ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(cache)) & 15) == 0;
}

static int absorbed_prefill(const void* q, const void* cache, const int32_t* kv_lengths, void* o, float* lse, int B,
                            int Lq, int S, int H, int R, int dtype, int band_hi, float sm_scale, int impl,
                            void* workspace, size_t workspace_bytes, int32_t* status, cudaStream_t st) {
  int rc = decode_limits(B, H, S);
  if (rc) return rc;
  if (S == 0) return fail(PJX_ERR_UNSUPPORTED, "absorbed latent attention at this width needs a non-empty cache");
  const int gh = latent_heads_per_group(H, 1);
  const size_t parts_max = absorbed_prefill_parts(B, H);
  const size_t need = align_up(parts_max * R * sizeof(float)) + align_up(parts_max * sizeof(float));
  if (!workspace || workspace_bytes < need)
    return fail(PJX_ERR_WORKSPACE, "mla workspace: need %zu bytes, got %zu", need, workspace ? workspace_bytes : (size_t)0);
  DecodeParams p;
  p.q = q; p.k = cache; p.v = cache; p.kv_lengths = kv_lengths; p.o = o; p.lse = lse;
  p.Lq = 1; p.Hq = H; p.Hkv = H / gh; p.D = R; p.Dv = R; p.capacity = S;
  p.rows = gh;
  p.sm_scale = sm_scale;
  p.o_is_f32 = 0;
  p.status = status;
  p.o_part = static_cast<float*>(workspace);
  p.lse_part = reinterpret_cast<float*>(static_cast<char*>(workspace) + align_up(parts_max * R * sizeof(float)));
  p.seq_total = Lq;
  // key j is visible to token t iff j <= t + band_hi
  p.seq_visible = band_hi >= S ? S : (band_hi < -Lq ? -Lq : band_hi + 1);
  const int chunk = absorbed_prefill_chunk(B, Lq);
  for (int t0 = 0; t0 < Lq; t0 += chunk) {
    p.seq_first = t0;
    p.seq_tokens = Lq - t0 < chunk ? Lq - t0 : chunk;
    p.B = B * p.seq_tokens;
    // keys this chunk can see at most: no split reaches beyond them
    int cap = S;
    if (t0 + p.seq_tokens - 1 + p.seq_visible < cap) cap = t0 + p.seq_tokens - 1 + p.seq_visible;
    if (cap < 1) cap = 1;
    p.split_len = latent_decode_split_len(p.B, p.Hkv, cap, 0);
    p.num_splits = (cap + p.split_len - 1) / p.split_len;
    if ((size_t)p.B * p.Hkv * p.num_splits * p.rows > parts_max)
      return fail(PJX_ERR_WORKSPACE, "absorbed latent attention: partials of a chunk exceed the workspace");
    const bool big = (double)p.B * p.Hkv * cap * R * 2.0 >= 64.0 * 1024 * 1024;
    const bool tc = (impl == PJX_IMPL_SM100 || (impl == PJX_IMPL_AUTO && big)) && decode_latent_tc_supported(p, dtype);
    if (impl == PJX_IMPL_SM100 && !tc)
      return fail(PJX_ERR_UNSUPPORTED, "the tcgen05 latent decode needs a status word and a cache of fewer than 2^31 rows");
    if ((rc = tc ? launch_decode_latent_tc_splits(p, dtype, st) : launch_decode_latent_splits(p, dtype, st))) return rc;
    if ((rc = launch_decode_combine(p, dtype, st))) return rc;
  }
  return PJX_OK;
}

size_t pjx_mla_workspace_bytes(int B, int S, int H, int Dqk, int Dv, int R, int dtype, int has_projections) {
  (void)S;
  if (!has_projections) {
    // absorbed attention at the wide latents runs through the latent decode kernels and keeps their partials here
    if (R <= 256 || !decode_latent_supported(R, dtype)) return 0;
    const size_t parts = absorbed_prefill_parts(B, H);
    return parts ? align_up(parts * R * sizeof(float)) + align_up(parts * sizeof(float)) : 0;
  }
  const size_t es = dtype_size(dtype);
  return align_up((size_t)B * S * H * Dqk * es) + align_up((size_t)B * S * H * Dv * es);
}

int pjx_mla_fwd(const void* q, const void* cache, const void* wk, const void* wv, void* o, float* lse,
                const int32_t* kv_lengths, const float* bias, int64_t bias_batch_stride, int64_t bias_head_stride,
                int B, int Lq, int S, int H, int Dqk, int Dv, int R, int dtype, int causal, float sm_scale, int impl,
                void* workspace, size_t workspace_bytes, int32_t* status, void* stream) {
  return pjx_mla_fwd_mod(q, cache, wk, wv, o, lse, kv_lengths, bias, bias_batch_stride, bias_head_stride, B, Lq, S, H,
                         Dqk, Dv, R, dtype, PJX_BAND_NO_LOWER, causal ? 0 : PJX_BAND_NO_UPPER, sm_scale, nullptr, impl,
                         workspace, workspace_bytes, status, stream);
}

int pjx_mla_fwd_mod(const void* q, const void* cache, const void* wk, const void* wv, void* o, float* lse,
                    const int32_t* kv_lengths, const float* bias, int64_t bias_batch_stride, int64_t bias_head_stride,
                    int B, int Lq, int S, int H, int Dqk, int Dv, int R, int dtype, int band_lo, int band_hi,
                    float sm_scale, const pjx_score_mod* mod, int impl, void* workspace, size_t workspace_bytes,
                    int32_t* status, void* stream) {
  // probjax/nn/pallas_kernels/kernels/latent_attention.py:668-696
  if ((wk == nullptr) != (wv == nullptr))
    return fail(PJX_ERR_BAD_ARG, "provide both wk and wv (materialized) or neither (absorbed); mixing the two is not supported");
  if (B < 0 || Lq < 0 || S < 0 || H < 1 || Dqk < 1 || Dv < 1 || R < 1)
    return fail(PJX_ERR_BAD_ARG, "mla: bad dimension");
  if (!wk && Dqk != R)
    return fail(PJX_ERR_BAD_ARG, "absorbed mode (wk=None) requires qk_head_dim == kv_lora_rank (%d != %d)", Dqk, R);
  if (!wk && Dv != R) return fail(PJX_ERR_BAD_ARG, "absorbed mode: the output width equals the latent width (%d != %d)", Dv, R);
  if (B == 0 || Lq == 0) return PJX_OK;
  if (!q || !cache || !o) return fail(PJX_ERR_BAD_ARG, "mla: null buffer");
  if (!wk) {
    // K = V = latent, one shared KV head (latent_attention.py:604-607).
    if (absorbed_prefill_applies(H, R, dtype, band_lo, bias, mod, q, cache))
      return absorbed_prefill(q, cache, kv_lengths, o, lse, B, Lq, S, H, R, dtype, band_hi, sm_scale, impl, workspace,
                              workspace_bytes, status, static_cast<cudaStream_t>(stream));
    return pjx_attn_fwd_mod(q, cache, cache, o, lse, kv_lengths, bias, bias_batch_stride, bias_head_stride, B, Lq, S,
                            H, 1, R, R, dtype, band_lo, band_hi, sm_scale, mod, impl, status, stream);
  }
  const size_t need = pjx_mla_workspace_bytes(B, S, H, Dqk, Dv, R, dtype, 1);
  if (!workspace || workspace_bytes < need)
    return fail(PJX_ERR_WORKSPACE, "mla workspace: need %zu bytes, got %zu", need, workspace ? workspace_bytes : (size_t)0);
  const size_t es = dtype_size(dtype);
  void* kmat = workspace;
  void* vmat = static_cast<char*>(workspace) + align_up((size_t)B * S * H * Dqk * es);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int rc;
  if ((rc = launch_gemm_tn2(cache, wk, kmat, H * Dqk, wv, vmat, H * Dv, (int64_t)B * S, R, dtype, impl, status, st))) return rc;
  return pjx_attn_fwd_mod(q, kmat, vmat, o, lse, kv_lengths, bias, bias_batch_stride, bias_head_stride, B, Lq, S, H, H,
                          Dqk, Dv, dtype, band_lo, band_hi, sm_scale, mod, impl, status, stream);
}

size_t pjx_attn_fwd_host_staging_bytes(int bias_batch, int bias_heads, int has_lse, int B, int Lq, int Lkv, int Hq,
                                       int Hkv, int D, int Dv, int dtype) {
  const size_t es = dtype_size(dtype);
  size_t n = 0;
  n += align_up((size_t)B * Lq * Hq * D * es);
  n += align_up((size_t)B * Lkv * Hkv * D * es);
  n += align_up((size_t)B * Lkv * Hkv * Dv * es);
  n += align_up((size_t)B * Lq * Hq * Dv * es);
  n += align_up((size_t)B * Hq * Lq * sizeof(float) * (has_lse ? 1 : 0));
  n += align_up((size_t)B * sizeof(int32_t));
  n += align_up((size_t)bias_batch * bias_heads * Lq * Lkv * sizeof(float));
  n += align_up(sizeof(int32_t));
  return n;
}

int pjx_attn_fwd_host(const void* q, const void* k, const void* v, void* o, float* lse, const int32_t* kv_lengths,
                      const float* bias, int bias_batch, int bias_heads, int B, int Lq, int Lkv, int Hq, int Hkv,
                      int D, int Dv, int dtype, int causal, float sm_scale, int impl, void* staging,
                      size_t staging_bytes, void* stream) {
  int rc = validate_common(q, k, v, o, B, Lq, Lkv, Hq, Hkv, D, Dv, dtype);
  if (rc) return rc;
  if (bias && !((bias_batch == 1 || bias_batch == B) && (bias_heads == 1 || bias_heads == Hq)))
    return fail(PJX_ERR_BAD_ARG, "bias must be [B|1, H|1, Lq, Lkv]; got leading dims (%d, %d)", bias_batch, bias_heads);
  if (!bias) bias_batch = bias_heads = 0;
  const size_t need = pjx_attn_fwd_host_staging_bytes(bias_batch, bias_heads, lse != nullptr, B, Lq, Lkv, Hq, Hkv, D, Dv, dtype);
  if (!staging || staging_bytes < need)
    return fail(PJX_ERR_WORKSPACE, "host forward staging: need %zu bytes, got %zu", need, staging ? staging_bytes : (size_t)0);
  if (B == 0 || Lq == 0) return PJX_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  HostPipe* hp = nullptr;
  if ((rc = host_pipe(&hp))) return rc;
  // One call at a time per device: a second host thread waits here (the call synchronises before
  // it returns anyway, so nothing is lost by serialising).
  std::lock_guard<std::mutex> one_call(hp->busy);
  const size_t es = dtype_size(dtype);
  char* base = static_cast<char*>(staging);
  size_t off = 0;
  auto take = [&](size_t bytes) { char* ptr = base + off; off += align_up(bytes); return ptr; };
  const size_t qb = (size_t)B * Lq * Hq * D * es, kb = (size_t)B * Lkv * Hkv * D * es,
               vb = (size_t)B * Lkv * Hkv * Dv * es, ob = (size_t)B * Lq * Hq * Dv * es,
               lb = lse ? (size_t)B * Hq * Lq * sizeof(float) : 0, nb = (size_t)B * sizeof(int32_t),
               bb = (size_t)bias_batch * bias_heads * Lq * Lkv * sizeof(float);
  char *dq = take(qb), *dk = take(kb), *dv = take(vb), *dout = take(ob), *dl = take(lb), *dn = take(nb), *db = take(bb),
       *ds = take(sizeof(int32_t));
  const int64_t bhs = bias ? (bias_heads == 1 ? 0 : (int64_t)Lq * Lkv) : 0;
  const int64_t bbs = bias ? (bias_batch == 1 ? 0 : (int64_t)bias_heads * Lq * Lkv) : 0;

  // Three streams: copies in, kernels (the caller's stream), copies out. The batch is
  // cut into chunks, and without a bias or an LSE result the query rows of a chunk are cut
  // again (K and V go up once, then each block of query rows is uploaded, computed with the
  // mask band shifted by its first row, and downloaded), so that uploads, kernels and
  // downloads overlap (PCIe is full duplex) and only one small block trails the last upload.
  const int nchunk = B < kHostChunks ? B : kHostChunks;
  const int per = (B + nchunk - 1) / nchunk;
  int nq = 1;
  if (!bias && !lse) nq = Lq / 1024 < 1 ? 1 : (Lq / 1024 > kHostQueryChunks ? kHostQueryChunks : Lq / 1024);
  const int rows_per = ((Lq + nq - 1) / nq + 255) / 256 * 256;  // whole 256-row CTAs
  if ((rc = check_cuda(cudaEventRecord(hp->start, st), "record start"))) return rc;
  if ((rc = check_cuda(cudaStreamWaitEvent(hp->in, hp->start, 0), "order upload stream"))) return rc;
  if ((rc = check_cuda(cudaStreamWaitEvent(hp->out, hp->start, 0), "order download stream"))) return rc;
  if (kv_lengths && (rc = check_cuda(cudaMemcpyAsync(dn, kv_lengths, nb, cudaMemcpyHostToDevice, hp->in), "copy kv_lengths to device"))) return rc;
  if (bias && (rc = check_cuda(cudaMemcpyAsync(db, bias, bb, cudaMemcpyHostToDevice, hp->in), "copy bias to device"))) return rc;
  if ((rc = check_cuda(cudaMemsetAsync(ds, 0, sizeof(int32_t), hp->in), "clear status"))) return rc;
  const size_t q1 = (size_t)Lq * Hq * D * es, k1 = (size_t)Lkv * Hkv * D * es, v1 = (size_t)Lkv * Hkv * Dv * es,
               o1 = (size_t)Lq * Hq * Dv * es, l1 = (size_t)Hq * Lq * sizeof(float);
  const size_t qrow = (size_t)Hq * D * es, orow = (size_t)Hq * Dv * es;
  int c = 0;
  for (int b0 = 0; b0 < B; b0 += per) {
    const int nb_c = (b0 + per <= B) ? per : B - b0;
    const char* hk = static_cast<const char*>(k) + b0 * k1;
    const char* hv = static_cast<const char*>(v) + b0 * v1;
    if (k1 && (rc = check_cuda(cudaMemcpyAsync(dk + b0 * k1, hk, nb_c * k1, cudaMemcpyHostToDevice, hp->in), "copy k to device"))) return rc;
    if (v1 && (rc = check_cuda(cudaMemcpyAsync(dv + b0 * v1, hv, nb_c * v1, cudaMemcpyHostToDevice, hp->in), "copy v to device"))) return rc;
    for (int l0 = 0; l0 < Lq; l0 += (nq > 1 ? rows_per : Lq), ++c) {
      const int rows = nq > 1 ? (l0 + rows_per <= Lq ? rows_per : Lq - l0) : Lq;
      // rows l0 .. l0+rows of every batch row of the chunk (one strided copy when the chunk holds several)
      const char* hq = static_cast<const char*>(q) + b0 * q1 + l0 * qrow;
      if (nq == 1) {
        if ((rc = check_cuda(cudaMemcpyAsync(dq + b0 * q1, hq, nb_c * q1, cudaMemcpyHostToDevice, hp->in), "copy q to device"))) return rc;
      } else if (nb_c == 1) {  // one batch row: the block of query rows is contiguous
        if ((rc = check_cuda(cudaMemcpyAsync(dq + b0 * q1 + l0 * qrow, hq, rows * qrow, cudaMemcpyHostToDevice, hp->in), "copy q rows to device"))) return rc;
      } else if ((rc = check_cuda(cudaMemcpy2DAsync(dq + b0 * q1 + l0 * qrow, q1, hq, q1, rows * qrow, nb_c, cudaMemcpyHostToDevice, hp->in), "copy q rows to device"))) {
        return rc;
      }
      if ((rc = check_cuda(cudaEventRecord(hp->up[c], hp->in), "record upload"))) return rc;
      if ((rc = check_cuda(cudaStreamWaitEvent(st, hp->up[c], 0), "wait for upload"))) return rc;
      if (nq == 1) {
        rc = pjx_attn_fwd(dq + b0 * q1, dk + b0 * k1, dv + b0 * v1, dout + b0 * o1,
                          lse ? reinterpret_cast<float*>(dl + b0 * l1) : nullptr,
                          kv_lengths ? reinterpret_cast<const int32_t*>(dn) + b0 : nullptr,
                          bias ? reinterpret_cast<const float*>(db) + (int64_t)b0 * bbs : nullptr, bbs, bhs, nb_c, Lq, Lkv,
                          Hq, Hkv, D, Dv, dtype, causal, sm_scale, impl, reinterpret_cast<int32_t*>(ds), stream);
      } else {
        // a block of query rows per batch row: the batch rows of the chunk are launched one by one
        // (their row blocks are not adjacent in memory)
        for (int bi = 0; bi < nb_c && !rc; ++bi)
          rc = pjx_attn_fwd_band(dq + (b0 + bi) * q1 + l0 * qrow, dk + (b0 + bi) * k1, dv + (b0 + bi) * v1,
                                 dout + (b0 + bi) * o1 + l0 * orow, nullptr,
                                 kv_lengths ? reinterpret_cast<const int32_t*>(dn) + b0 + bi : nullptr, nullptr, 0, 0, 1,
                                 rows, Lkv, Hq, Hkv, D, Dv, dtype, PJX_BAND_NO_LOWER, causal ? l0 : PJX_BAND_NO_UPPER,
                                 sm_scale, impl, reinterpret_cast<int32_t*>(ds), stream);
      }
      if (rc) return rc;
      if ((rc = check_cuda(cudaEventRecord(hp->done[c], st), "record kernel"))) return rc;
      if ((rc = check_cuda(cudaStreamWaitEvent(hp->out, hp->done[c], 0), "wait for kernel"))) return rc;
      if (nq == 1) {
        if ((rc = check_cuda(cudaMemcpyAsync(static_cast<char*>(o) + b0 * o1, dout + b0 * o1, nb_c * o1, cudaMemcpyDeviceToHost, hp->out), "copy o to host"))) return rc;
        if (lse && (rc = check_cuda(cudaMemcpyAsync(reinterpret_cast<char*>(lse) + b0 * l1, dl + b0 * l1, nb_c * l1, cudaMemcpyDeviceToHost, hp->out), "copy lse to host"))) return rc;
      } else if (nb_c == 1) {
        if ((rc = check_cuda(cudaMemcpyAsync(static_cast<char*>(o) + b0 * o1 + l0 * orow, dout + b0 * o1 + l0 * orow, rows * orow, cudaMemcpyDeviceToHost, hp->out), "copy o rows to host"))) return rc;
      } else if ((rc = check_cuda(cudaMemcpy2DAsync(static_cast<char*>(o) + b0 * o1 + l0 * orow, o1, dout + b0 * o1 + l0 * orow, o1, rows * orow, nb_c, cudaMemcpyDeviceToHost, hp->out), "copy o rows to host"))) {
        return rc;
      }
    }
  }
  int32_t hs = 0;
  if ((rc = check_cuda(cudaMemcpyAsync(&hs, ds, sizeof(int32_t), cudaMemcpyDeviceToHost, hp->out), "copy status to host"))) return rc;
  if ((rc = check_cuda(cudaEventRecord(hp->finish, hp->out), "record finish"))) return rc;
  if ((rc = check_cuda(cudaStreamWaitEvent(st, hp->finish, 0), "join download stream"))) return rc;
  if ((rc = check_cuda(cudaStreamSynchronize(st), "synchronise after host forward"))) return rc;
  if (hs) return fail(hs, "the forward kernel reported status %d (%s)", hs, pjx_status_string(hs));
  return PJX_OK;
}

int pjx_read_status(const int32_t* status, void* stream) {
  if (!status) return PJX_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int32_t hs = 0;
  int rc;
  if ((rc = check_cuda(cudaMemcpyAsync(&hs, status, sizeof(int32_t), cudaMemcpyDeviceToHost, st), "read status"))) return rc;
  if ((rc = check_cuda(cudaStreamSynchronize(st), "synchronise for status"))) return rc;
  if (hs) return fail(hs, "kernel status %d (%s)", hs, pjx_status_string(hs));
  return PJX_OK;
}

}  // extern "C"
