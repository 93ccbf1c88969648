// extern "C" entry points declared in include/haste_ffi.h: argument validation, error strings and
// dispatch to the kernel launchers.  Nothing here throws; every failure is a status code plus a
// thread-local message.
#include "common.cuh"
#include "launchers.h"
#include "runtime.h"

namespace haste {

static thread_local char g_err[512] = "no error";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}
int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(HASTE_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
  return HASTE_OK;
}
int validate_shape(const char* who, int64_t B, int64_t D, int64_t F, int64_t L, int64_t G) {
  if (B < 1 || D < 1 || L < 1) return fail(HASTE_ERR_BAD_ARG, "%s: B=%lld D=%lld L=%lld must be positive", who, (long long)B, (long long)D, (long long)L);
  if (!(G == 16 || G == 32 || G == 64 || G == 128)) return fail(HASTE_ERR_UNSUPPORTED, "%s: group size %lld not in {16,32,64,128}", who, (long long)G);
  if (F < 16 || F > 128 || (F % 16) != 0) return fail(HASTE_ERR_UNSUPPORTED, "%s: fan_in %lld must be a multiple of 16 in [16,128]", who, (long long)F);
  if (B >= (1ll << 24)) return fail(HASTE_ERR_UNSUPPORTED, "%s: batch %lld too large (< 2^24)", who, (long long)B);
  if (D >= (1ll << 31) || (L + G - 1) / G >= (1ll << 31)) return fail(HASTE_ERR_UNSUPPORTED, "%s: D or group count exceeds int32", who);
  return HASTE_OK;
}

// Shape dispatch of the fused step: the tcgen05 kernel where its tile shapes apply — (G=128, F=64) or (G=64, F=128),
// B % 8 == 0 (16-byte rows of xt for the tensor map), D*B < 2^32 (32-bit dxt row offsets), L < 2^31 — the warp-mma
// kernel for every other supported shape.
static int g_max_ctas = 0;   // 0 = one CTA per SM

static bool train_step_sm100_supported(int64_t B, int64_t D, int64_t F, int64_t L, int64_t G) {
  return ((G == 128 && F == 64) || (G == 64 && F == 128)) && (B % 8) == 0 && D * B < (int64_t(1) << 32) && L < (int64_t(1) << 31);
}

int launch_train_step(const int32_t* loc, const void* xt, const int32_t* tgt_ptr, const uint32_t* tgt_ent, float* dxt, float* loss,
                      const UpdateArgs& u, int64_t B, int64_t D, int64_t F, int64_t L, int64_t G, int loss_kind, float grad_scale,
                      cudaStream_t st, const StepDump* dump) {
  if (train_step_sm100_supported(B, D, F, L, G)) {
    if (G == 128) return launch_train_step_sm100_g128f64(loc, xt, tgt_ptr, tgt_ent, dxt, loss, u, B, D, L, loss_kind, grad_scale, g_max_ctas, st, dump);
    return launch_train_step_sm100_g64f128(loc, xt, tgt_ptr, tgt_ent, dxt, loss, u, B, D, L, loss_kind, grad_scale, g_max_ctas, st, dump);
  }
  if (dump != nullptr) return fail(HASTE_ERR_UNSUPPORTED, "debug outputs exist only in the tcgen05 fused step ((G,F) = (128,64) or (64,128), B%%8==0)");
  return launch_train_step_mma(loc, xt, tgt_ptr, tgt_ent, dxt, loss, u, B, D, F, L, G, loss_kind, grad_scale, st);
}

}  // namespace haste

using namespace haste;

#define REQUIRE_PTR(p, who) \
  if ((p) == nullptr) return fail(HASTE_ERR_BAD_ARG, "%s: argument '%s' is NULL", who, #p)
#define REQUIRE_ALIGNED(p, who) \
  if (!aligned16(p)) return fail(HASTE_ERR_BAD_ARG, "%s: argument '%s' must be 16-byte aligned", who, #p)

extern "C" {

const char* haste_last_error_string(void) { return g_err; }
int haste_version(void) { return 200; }

int haste_ffi_set_max_ctas(int32_t n) {
  if (n < 0) return fail(HASTE_ERR_BAD_ARG, "haste_ffi_set_max_ctas: n=%d < 0", n);
  g_max_ctas = n;
  return HASTE_OK;
}

int haste_ffi_forward(const int32_t* loc, const void* xt, const void* w, const void* bias, void* z, int64_t B, int64_t D, int64_t F,
                      int64_t L, int64_t G, int64_t ldz, haste_stream_t stream) {
  const char* who = "haste_ffi_forward";
  REQUIRE_PTR(loc, who); REQUIRE_PTR(xt, who); REQUIRE_PTR(w, who); REQUIRE_PTR(z, who);
  REQUIRE_ALIGNED(xt, who); REQUIRE_ALIGNED(w, who);
  if (int rc = validate_shape(who, B, D, F, L, G)) return rc;
  if (ldz < L) return fail(HASTE_ERR_BAD_ARG, "%s: ldz=%lld < L=%lld", who, (long long)ldz, (long long)L);
  return launch_forward(loc, xt, w, bias, z, B, D, F, L, G, ldz, ldz, static_cast<cudaStream_t>(stream));
}

int haste_ffi_forward_into(const int32_t* loc, const void* xt, const void* w, const void* bias, void* z, int64_t B, int64_t D, int64_t F,
                           int64_t L, int64_t G, int64_t ldz, int64_t zcols, haste_stream_t stream) {
  const char* who = "haste_ffi_forward_into";
  REQUIRE_PTR(loc, who); REQUIRE_PTR(xt, who); REQUIRE_PTR(w, who); REQUIRE_PTR(z, who);
  REQUIRE_ALIGNED(xt, who); REQUIRE_ALIGNED(w, who);
  if (int rc = validate_shape(who, B, D, F, L, G)) return rc;
  if (zcols < L || ldz < zcols) return fail(HASTE_ERR_BAD_ARG, "%s: need L <= zcols <= ldz (L=%lld zcols=%lld ldz=%lld)", who, (long long)L, (long long)zcols, (long long)ldz);
  return launch_forward(loc, xt, w, bias, z, B, D, F, L, G, ldz, zcols, static_cast<cudaStream_t>(stream));
}

int haste_ffi_backward_features(const void* w, const int32_t* loc, const void* dy, float* dxt, int64_t B, int64_t D, int64_t F, int64_t L,
                                int64_t G, int64_t ldy, uint32_t flags, haste_stream_t stream) {
  const char* who = "haste_ffi_backward_features";
  REQUIRE_PTR(loc, who); REQUIRE_PTR(w, who); REQUIRE_PTR(dy, who); REQUIRE_PTR(dxt, who);
  REQUIRE_ALIGNED(w, who); REQUIRE_ALIGNED(dxt, who);
  if (int rc = validate_shape(who, B, D, F, L, G)) return rc;
  if (ldy < L) return fail(HASTE_ERR_BAD_ARG, "%s: ldy=%lld < L=%lld", who, (long long)ldy, (long long)L);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (flags & HASTE_F_ZERO_DXT) {
    cudaError_t e = cudaMemsetAsync(dxt, 0, sizeof(float) * D * B, st);
    if (e != cudaSuccess) return fail(HASTE_ERR_LAUNCH, "%s: cudaMemsetAsync: %s", who, cudaGetErrorString(e));
  }
  if (backward_sm100_supported(nullptr, w, dy, nullptr, B, D, F, L, G))
    return launch_backward_sm100(nullptr, w, loc, dy, dxt, nullptr, nullptr, nullptr, B, D, F, L, G, ldy, st);
  return launch_bwd_features(w, loc, dy, dxt, B, D, F, L, G, ldy, st);
}

int haste_ffi_backward_weights(const void* xt, const int32_t* loc, const void* dy, void* dw, void* dbias, int64_t B, int64_t D, int64_t F,
                               int64_t L, int64_t G, int64_t ldy, haste_stream_t stream) {
  const char* who = "haste_ffi_backward_weights";
  REQUIRE_PTR(loc, who); REQUIRE_PTR(xt, who); REQUIRE_PTR(dy, who); REQUIRE_PTR(dw, who);
  REQUIRE_ALIGNED(xt, who); REQUIRE_ALIGNED(dw, who);
  if (int rc = validate_shape(who, B, D, F, L, G)) return rc;
  if (ldy < L) return fail(HASTE_ERR_BAD_ARG, "%s: ldy=%lld < L=%lld", who, (long long)ldy, (long long)L);
  if (backward_sm100_supported(xt, nullptr, dy, dw, B, D, F, L, G))
    return launch_backward_sm100(xt, nullptr, loc, dy, nullptr, dw, dbias, nullptr, B, D, F, L, G, ldy, static_cast<cudaStream_t>(stream));
  return launch_bwd_weights(xt, loc, dy, dw, dbias, nullptr, B, D, F, L, G, ldy, static_cast<cudaStream_t>(stream));
}

int haste_ffi_backward(const void* xt, const void* w, const int32_t* loc, const void* dy, float* dxt, void* dw, void* dbias, int64_t B,
                       int64_t D, int64_t F, int64_t L, int64_t G, int64_t ldy, uint32_t flags, haste_stream_t stream) {
  const char* who = "haste_ffi_backward";
  REQUIRE_PTR(loc, who); REQUIRE_PTR(xt, who); REQUIRE_PTR(w, who); REQUIRE_PTR(dy, who); REQUIRE_PTR(dxt, who); REQUIRE_PTR(dw, who);
  REQUIRE_ALIGNED(xt, who); REQUIRE_ALIGNED(w, who); REQUIRE_ALIGNED(dxt, who); REQUIRE_ALIGNED(dw, who);
  if (int rc = validate_shape(who, B, D, F, L, G)) return rc;
  if (ldy < L) return fail(HASTE_ERR_BAD_ARG, "%s: ldy=%lld < L=%lld", who, (long long)ldy, (long long)L);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (flags & HASTE_F_ZERO_DXT) {
    cudaError_t e = cudaMemsetAsync(dxt, 0, sizeof(float) * D * B, st);
    if (e != cudaSuccess) return fail(HASTE_ERR_LAUNCH, "%s: cudaMemsetAsync: %s", who, cudaGetErrorString(e));
  }
  if (backward_sm100_supported(xt, w, dy, dw, B, D, F, L, G)) return launch_backward_sm100(xt, w, loc, dy, dxt, dw, dbias, nullptr, B, D, F, L, G, ldy, st);
  if (int rc = launch_bwd_features(w, loc, dy, dxt, B, D, F, L, G, ldy, st)) return rc;
  return launch_bwd_weights(xt, loc, dy, dw, dbias, nullptr, B, D, F, L, G, ldy, st);
}

int haste_pad_rows_bf16(const void* src, int64_t ld_src, void* dst, int64_t ld_dst, int64_t rows, int64_t cols, haste_stream_t stream) {
  const char* who = "haste_pad_rows_bf16";
  REQUIRE_PTR(src, who); REQUIRE_PTR(dst, who); REQUIRE_ALIGNED(dst, who);
  if (rows < 1 || cols < 1 || ld_src < cols || ld_dst < cols || (ld_dst % 8) != 0) return fail(HASTE_ERR_BAD_ARG, "%s: bad sizes", who);
  return launch_pad_rows(src, ld_src, dst, ld_dst, rows, cols, static_cast<cudaStream_t>(stream));
}

int haste_ffi_bww_sr_sgd(const void* xt, const int32_t* loc, const void* dy, void* w, void* bias, float* mom_w, float* mom_b, int64_t B,
                         int64_t D, int64_t F, int64_t L, int64_t G, int64_t ldy, int64_t label0, float lr, float wd, float mu,
                         uint64_t seed, uint32_t step, uint32_t flags, haste_stream_t stream) {
  const char* who = "haste_ffi_bww_sr_sgd";
  REQUIRE_PTR(loc, who); REQUIRE_PTR(xt, who); REQUIRE_PTR(dy, who); REQUIRE_PTR(w, who);
  REQUIRE_ALIGNED(xt, who); REQUIRE_ALIGNED(w, who);
  if (mom_w) REQUIRE_ALIGNED(mom_w, who);
  if (int rc = validate_shape(who, B, D, F, L, G)) return rc;
  if (ldy < L) return fail(HASTE_ERR_BAD_ARG, "%s: ldy=%lld < L=%lld", who, (long long)ldy, (long long)L);
  UpdateArgs u;
  u.w = static_cast<__nv_bfloat16*>(w); u.bias = static_cast<__nv_bfloat16*>(bias);
  u.mom_w = (mu != 0.f) ? mom_w : nullptr; u.mom_b = (mu != 0.f) ? mom_b : nullptr;
  u.lr = lr; u.wd = wd; u.mu = mu; u.seed = seed; u.step = step; u.flags = flags; u.label0 = label0;
  if (backward_sm100_supported(xt, nullptr, dy, w, B, D, F, L, G))
    return launch_backward_sm100(xt, nullptr, loc, dy, nullptr, nullptr, nullptr, &u, B, D, F, L, G, ldy, static_cast<cudaStream_t>(stream));
  return launch_bwd_weights(xt, loc, dy, nullptr, nullptr, &u, B, D, F, L, G, ldy, static_cast<cudaStream_t>(stream));
}

int haste_targets_bucket(const int32_t* coo, int64_t nnz, int64_t label0, int64_t L, int64_t G, int32_t* tgt_ptr, uint32_t* tgt_ent,
                         int32_t* scratch, haste_stream_t stream) {
  const char* who = "haste_targets_bucket";
  if (nnz < 0 || L < 1 || G < 1 || G > 256) return fail(HASTE_ERR_BAD_ARG, "%s: bad sizes nnz=%lld L=%lld G=%lld", who, (long long)nnz, (long long)L, (long long)G);
  if (nnz > 0) { REQUIRE_PTR(coo, who); REQUIRE_PTR(tgt_ent, who); }
  REQUIRE_PTR(tgt_ptr, who); REQUIRE_PTR(scratch, who);
  return launch_targets_bucket(coo, nnz, label0, L, G, tgt_ptr, tgt_ent, scratch, static_cast<cudaStream_t>(stream));
}

int haste_targets_bucket_noalloc(const int32_t* coo, int64_t nnz, int64_t label0, int64_t L, int64_t G, int32_t* tgt_ptr,
                                 uint32_t* tgt_ent, haste_stream_t stream) {
  const char* who = "haste_targets_bucket_noalloc";
  if (nnz < 0 || L < 1 || G < 1 || G > 256) return fail(HASTE_ERR_BAD_ARG, "%s: bad sizes nnz=%lld L=%lld G=%lld", who, (long long)nnz, (long long)L, (long long)G);
  if (nnz > 0) { REQUIRE_PTR(coo, who); REQUIRE_PTR(tgt_ent, who); }
  REQUIRE_PTR(tgt_ptr, who);
  return launch_targets_bucket_noalloc(coo, nnz, label0, L, G, tgt_ptr, tgt_ent, static_cast<cudaStream_t>(stream));
}

int haste_ffi_step_prepare(const void* x, void* xt, float* dxt, float* loss, const int32_t* coo, int64_t nnz, int64_t label0, int64_t L,
                           int64_t G, int32_t* tgt_ptr, uint32_t* tgt_ent, int64_t B, int64_t D, haste_stream_t stream) {
  const char* who = "haste_ffi_step_prepare";
  REQUIRE_PTR(x, who); REQUIRE_PTR(xt, who); REQUIRE_PTR(dxt, who); REQUIRE_PTR(tgt_ptr, who);
  if (nnz < 0 || L < 1 || G < 1 || G > 256 || B < 1 || D < 1) return fail(HASTE_ERR_BAD_ARG, "%s: bad sizes", who);
  if (nnz > 0) { REQUIRE_PTR(coo, who); REQUIRE_PTR(tgt_ent, who); }
  return launch_step_prepare(x, xt, dxt, loss, coo, nnz, label0, L, G, tgt_ptr, tgt_ent, B, D, static_cast<cudaStream_t>(stream));
}

static int train_step_impl(const StepDump* dump, const int32_t* loc, const void* xt, void* w, void* bias, float* mom_w, float* mom_b, const int32_t* tgt_ptr,
                         const uint32_t* tgt_ent, float* dxt, float* loss, int64_t B, int64_t D, int64_t F, int64_t L, int64_t G,
                         int64_t label0, int32_t loss_kind, float grad_scale, float lr, float wd, float mu, uint64_t seed, uint32_t step,
                         uint32_t flags, haste_stream_t stream) {
  const char* who = dump ? "haste_ffi_train_step_dbg" : "haste_ffi_train_step";
  REQUIRE_PTR(loc, who); REQUIRE_PTR(xt, who); REQUIRE_PTR(w, who); REQUIRE_PTR(tgt_ptr, who); REQUIRE_PTR(dxt, who);
  REQUIRE_ALIGNED(xt, who); REQUIRE_ALIGNED(w, who); REQUIRE_ALIGNED(dxt, who);
  if (mom_w) REQUIRE_ALIGNED(mom_w, who);
  if (int rc = validate_shape(who, B, D, F, L, G)) return rc;
  if (loss_kind != HASTE_LOSS_BCE && loss_kind != HASTE_LOSS_SQHINGE) return fail(HASTE_ERR_BAD_ARG, "%s: unknown loss_kind %d", who, loss_kind);
  if ((flags & HASTE_F_LOSS) && loss == nullptr) return fail(HASTE_ERR_BAD_ARG, "%s: HASTE_F_LOSS needs a loss pointer", who);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (flags & HASTE_F_ZERO_DXT) {
    cudaError_t e = cudaMemsetAsync(dxt, 0, sizeof(float) * D * B, st);
    if (e != cudaSuccess) return fail(HASTE_ERR_LAUNCH, "%s: cudaMemsetAsync: %s", who, cudaGetErrorString(e));
  }
  UpdateArgs u;
  u.w = static_cast<__nv_bfloat16*>(w); u.bias = static_cast<__nv_bfloat16*>(bias);
  u.mom_w = (mu != 0.f) ? mom_w : nullptr; u.mom_b = (mu != 0.f) ? mom_b : nullptr;
  u.lr = lr; u.wd = wd; u.mu = mu; u.seed = seed; u.step = step; u.flags = flags; u.label0 = label0;
  return launch_train_step(loc, xt, tgt_ptr, tgt_ent, dxt, loss, u, B, D, F, L, G, loss_kind, grad_scale, st, dump);
}

int haste_ffi_train_step(const int32_t* loc, const void* xt, void* w, void* bias, float* mom_w, float* mom_b, const int32_t* tgt_ptr,
                         const uint32_t* tgt_ent, float* dxt, float* loss, int64_t B, int64_t D, int64_t F, int64_t L, int64_t G,
                         int64_t label0, int32_t loss_kind, float grad_scale, float lr, float wd, float mu, uint64_t seed, uint32_t step,
                         uint32_t flags, haste_stream_t stream) {
  return train_step_impl(nullptr, loc, xt, w, bias, mom_w, mom_b, tgt_ptr, tgt_ent, dxt, loss, B, D, F, L, G, label0, loss_kind, grad_scale,
                         lr, wd, mu, seed, step, flags, stream);
}

int haste_ffi_step(const void* x, const int32_t* coo, int64_t nnz, const int32_t* loc, void* xt, void* w, void* bias, float* mom_w,
                   float* mom_b, int32_t* tgt_ptr, uint32_t* tgt_ent, float* dxt, float* loss, int64_t B, int64_t D, int64_t F, int64_t L,
                   int64_t G, int64_t label0, int32_t loss_kind, float grad_scale, float lr, float wd, float mu, uint64_t seed,
                   uint32_t step, uint32_t flags, haste_stream_t stream) {
  if (int rc = haste_ffi_step_prepare(x, xt, dxt, loss, coo, nnz, label0, L, G, tgt_ptr, tgt_ent, B, D, stream)) return rc;
  // the step follows its own preparation kernel in the same stream: its set-up may overlap that kernel's tail
  dependent_launch_scope(1);
  const int rc = train_step_impl(nullptr, loc, xt, w, bias, mom_w, mom_b, tgt_ptr, tgt_ent, dxt, loss, B, D, F, L, G, label0, loss_kind,
                                 grad_scale, lr, wd, mu, seed, step, flags & ~static_cast<uint32_t>(HASTE_F_ZERO_DXT), stream);
  dependent_launch_scope(0);
  return rc;
}

int haste_ffi_train_step_dbg(const int32_t* loc, const void* xt, void* w, void* bias, float* mom_w, float* mom_b, const int32_t* tgt_ptr,
                             const uint32_t* tgt_ent, float* dxt, float* loss, int64_t B, int64_t D, int64_t F, int64_t L, int64_t G,
                             int64_t label0, int32_t loss_kind, float grad_scale, float lr, float wd, float mu, uint64_t seed,
                             uint32_t step, uint32_t flags, void* z_dump, int64_t ldz, void* dw_dump, void* dbias_dump,
                             haste_stream_t stream) {
  StepDump d{z_dump, ldz, dw_dump, dbias_dump};
  return train_step_impl(&d, loc, xt, w, bias, mom_w, mom_b, tgt_ptr, tgt_ent, dxt, loss, B, D, F, L, G, label0, loss_kind, grad_scale, lr,
                         wd, mu, seed, step, flags, stream);
}

int haste_sr_round(const float* x, void* out, int64_t n, uint64_t seed, haste_stream_t stream) {
  const char* who = "haste_sr_round";
  if (n < 0) return fail(HASTE_ERR_BAD_ARG, "%s: n < 0", who);
  if (n > 0) { REQUIRE_PTR(x, who); REQUIRE_PTR(out, who); }
  if (n >= (1ll << 31)) return fail(HASTE_ERR_UNSUPPORTED, "%s: the reference stream uses int32 offsets; n=%lld too large", who, (long long)n);
  return launch_sr_round(x, out, n, seed, static_cast<cudaStream_t>(stream));
}

int haste_sgd_sr_update(void* w, const void* grad, float* mom, int64_t rows, int64_t cols, int64_t row0, float lr, float wd, float mu,
                        uint64_t seed, uint32_t step, uint32_t flags, haste_stream_t stream) {
  const char* who = "haste_sgd_sr_update";
  if (rows < 0 || cols < 1) return fail(HASTE_ERR_BAD_ARG, "%s: bad shape [%lld,%lld]", who, (long long)rows, (long long)cols);
  if (rows > 0) { REQUIRE_PTR(w, who); REQUIRE_PTR(grad, who); }
  return launch_sgd_sr(w, grad, (mu != 0.f) ? mom : nullptr, rows, cols, row0, lr, wd, mu, seed, step, flags, static_cast<cudaStream_t>(stream));
}

int haste_dxt_to_dx_sr(const float* dxt, void* dx, int64_t B, int64_t D, uint64_t seed, haste_stream_t stream) {
  const char* who = "haste_dxt_to_dx_sr";
  REQUIRE_PTR(dxt, who); REQUIRE_PTR(dx, who);
  if (B < 1 || D < 1) return fail(HASTE_ERR_BAD_ARG, "%s: bad shape", who);
  return launch_dxt_to_dx(dxt, dx, B, D, seed, static_cast<cudaStream_t>(stream));
}

int haste_transpose_bf16(const void* x, void* xt, int64_t B, int64_t D, haste_stream_t stream) {
  const char* who = "haste_transpose_bf16";
  REQUIRE_PTR(x, who); REQUIRE_PTR(xt, who);
  if (B < 1 || D < 1) return fail(HASTE_ERR_BAD_ARG, "%s: bad shape", who);
  return launch_transpose(x, xt, B, D, static_cast<cudaStream_t>(stream));
}

int haste_ffi_rewire(void* w, int32_t* loc, float* mom_w, int64_t D, int64_t F, int64_t L, int64_t G, int64_t group0, int32_t prune_mode,
                     float threshold, int32_t n_prune, int32_t regrow_mode, int32_t init_mode, int32_t regroup, uint64_t seed,
                     uint32_t step, int32_t* changed, haste_stream_t stream) {
  const char* who = "haste_ffi_rewire";
  REQUIRE_PTR(w, who); REQUIRE_PTR(loc, who); REQUIRE_ALIGNED(w, who);
  if (int rc = validate_shape(who, 1, D, F, L, G)) return rc;
  if (prune_mode < 0 || prune_mode > 1 || regrow_mode < 0 || regrow_mode > 1 || init_mode < 0 || init_mode > 1)
    return fail(HASTE_ERR_BAD_ARG, "%s: bad mode", who);
  if (n_prune < 0 || n_prune > F) return fail(HASTE_ERR_BAD_ARG, "%s: n_prune=%d outside [0,F]", who, n_prune);
  if (regrow_mode == 1 && D < 2 * F) return fail(HASTE_ERR_UNSUPPORTED, "%s: 'unused' regrow needs D >= 2*F", who);
  return launch_rewire(w, loc, mom_w, D, F, L, G, group0, 0, prune_mode, threshold, n_prune, regrow_mode, init_mode, regroup, seed, step,
                       nullptr, changed, static_cast<cudaStream_t>(stream));
}

int haste_ffi_rewire_ex(void* w, int32_t* loc, float* mom_w, int64_t D, int64_t F, int64_t L, int64_t G, int64_t group0, int32_t score_mode,
                        int32_t prune_mode, float threshold, int64_t n_prune, int32_t regrow_mode, int32_t init_mode, int32_t regroup,
                        uint64_t seed, uint32_t step, void* scratch, int32_t* changed, haste_stream_t stream) {
  const char* who = "haste_ffi_rewire_ex";
  REQUIRE_PTR(w, who); REQUIRE_PTR(loc, who); REQUIRE_ALIGNED(w, who);
  if (int rc = validate_shape(who, 1, D, F, L, G)) return rc;
  if (score_mode < 0 || score_mode > 1 || prune_mode < 0 || prune_mode > 2 || regrow_mode < 0 || regrow_mode > 1 || init_mode < 0 || init_mode > 1)
    return fail(HASTE_ERR_BAD_ARG, "%s: bad mode", who);
  const int64_t NG = (L + G - 1) / G;
  if (prune_mode == 1 && (n_prune < 0 || n_prune > F)) return fail(HASTE_ERR_BAD_ARG, "%s: n_prune=%lld outside [0,F]", who, (long long)n_prune);
  if (prune_mode == 2) {
    if (n_prune < 1 || n_prune > NG * F) return fail(HASTE_ERR_BAD_ARG, "%s: n_prune=%lld outside [1,NG*F]", who, (long long)n_prune);
    REQUIRE_PTR(scratch, who); REQUIRE_ALIGNED(scratch, who);
  }
  if (regrow_mode == 1 && D < 2 * F) return fail(HASTE_ERR_UNSUPPORTED, "%s: 'unused' regrow needs D >= 2*F", who);
  return launch_rewire(w, loc, mom_w, D, F, L, G, group0, score_mode, prune_mode, threshold, n_prune, regrow_mode, init_mode, regroup, seed,
                       step, scratch, changed, static_cast<cudaStream_t>(stream));
}

int haste_ffi_rewire_select_begin(const void* w, int64_t F, int64_t L, int64_t G, int32_t score_mode, void* scratch, haste_stream_t stream) {
  const char* who = "haste_ffi_rewire_select_begin";
  REQUIRE_PTR(w, who); REQUIRE_PTR(scratch, who); REQUIRE_ALIGNED(w, who); REQUIRE_ALIGNED(scratch, who);
  if (int rc = validate_shape(who, 1, 1, F, L, G)) return rc;
  if (score_mode < 0 || score_mode > 1) return fail(HASTE_ERR_BAD_ARG, "%s: bad score_mode", who);
  return launch_rewire_select_begin(w, F, L, G, score_mode, scratch, static_cast<cudaStream_t>(stream));
}

int haste_ffi_rewire_select_refine(int64_t F, int64_t L, int64_t G, int64_t k_layer, void* scratch, haste_stream_t stream) {
  const char* who = "haste_ffi_rewire_select_refine";
  REQUIRE_PTR(scratch, who);
  if (int rc = validate_shape(who, 1, 1, F, L, G)) return rc;
  if (k_layer < 1 || k_layer >= (1ll << 32)) return fail(HASTE_ERR_BAD_ARG, "%s: k_layer=%lld outside [1, 2^32)", who, (long long)k_layer);
  return launch_rewire_select_refine(F, L, G, k_layer, scratch, static_cast<cudaStream_t>(stream));
}

int haste_ffi_rewire_select_finish(int64_t F, int64_t L, int64_t G, void* scratch, haste_stream_t stream) {
  const char* who = "haste_ffi_rewire_select_finish";
  REQUIRE_PTR(scratch, who);
  if (int rc = validate_shape(who, 1, 1, F, L, G)) return rc;
  return launch_rewire_select_finish(F, L, G, scratch, static_cast<cudaStream_t>(stream));
}

int haste_ffi_rewire_prepared(void* w, int32_t* loc, float* mom_w, int64_t D, int64_t F, int64_t L, int64_t G, int64_t group0,
                              int32_t score_mode, uint32_t tie_base, int32_t regrow_mode, int32_t init_mode, int32_t regroup, uint64_t seed,
                              uint32_t step, void* scratch, int32_t* changed, haste_stream_t stream) {
  const char* who = "haste_ffi_rewire_prepared";
  REQUIRE_PTR(w, who); REQUIRE_PTR(loc, who); REQUIRE_PTR(scratch, who); REQUIRE_ALIGNED(w, who); REQUIRE_ALIGNED(scratch, who);
  if (int rc = validate_shape(who, 1, D, F, L, G)) return rc;
  if (score_mode < 0 || score_mode > 1 || regrow_mode < 0 || regrow_mode > 1 || init_mode < 0 || init_mode > 1)
    return fail(HASTE_ERR_BAD_ARG, "%s: bad mode", who);
  if (regrow_mode == 1 && D < 2 * F) return fail(HASTE_ERR_UNSUPPORTED, "%s: 'unused' regrow needs D >= 2*F", who);
  return launch_rewire(w, loc, mom_w, D, F, L, G, group0, score_mode, 3, 0.f, 0, regrow_mode, init_mode, regroup, seed, step, scratch, changed,
                       static_cast<cudaStream_t>(stream), tie_base);
}

int haste_topk_update(const void* z, int64_t ldz, int64_t B, int64_t C, int64_t col0, int32_t k, float* vals, int32_t* idx,
                      haste_stream_t stream) {
  const char* who = "haste_topk_update";
  if (B < 0 || C < 0 || ldz < C || col0 < 0) return fail(HASTE_ERR_BAD_ARG, "%s: bad sizes", who);
  if (k < 1 || k > 128) return fail(HASTE_ERR_UNSUPPORTED, "%s: k=%d outside [1,128]", who, k);
  if (col0 + C >= (1ll << 31)) return fail(HASTE_ERR_UNSUPPORTED, "%s: label ids must fit in int32", who);
  if (B > 0 && C > 0) { REQUIRE_PTR(z, who); REQUIRE_PTR(vals, who); REQUIRE_PTR(idx, who); }
  return launch_topk_update(z, ldz, B, C, col0, k, vals, idx, static_cast<cudaStream_t>(stream));
}

int haste_ffi_topk(const int32_t* loc, const void* xt, const void* w, const void* bias, void* zbuf, int64_t ldz, int64_t B, int64_t D,
                   int64_t F, int64_t L, int64_t G, int64_t groups_per_chunk, int32_t k, int64_t label0, float* vals, int32_t* idx,
                   haste_stream_t stream) {
  const char* who = "haste_ffi_topk";
  REQUIRE_PTR(loc, who); REQUIRE_PTR(xt, who); REQUIRE_PTR(w, who); REQUIRE_PTR(zbuf, who); REQUIRE_PTR(vals, who); REQUIRE_PTR(idx, who);
  REQUIRE_ALIGNED(xt, who); REQUIRE_ALIGNED(w, who); REQUIRE_ALIGNED(zbuf, who);
  if (int rc = validate_shape(who, B, D, F, L, G)) return rc;
  if (k < 1 || k > 128) return fail(HASTE_ERR_UNSUPPORTED, "%s: k=%d outside [1,128]", who, k);
  if (groups_per_chunk < 1 || label0 < 0) return fail(HASTE_ERR_BAD_ARG, "%s: bad chunk size or label offset", who);
  if (ldz < groups_per_chunk * G || (ldz % 8) != 0)
    return fail(HASTE_ERR_BAD_ARG, "%s: the logit buffer needs a row stride of at least groups_per_chunk * G columns, a multiple of 8", who);
  if (label0 + L >= (1ll << 31)) return fail(HASTE_ERR_UNSUPPORTED, "%s: label ids must fit in int32", who);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t NG = (L + G - 1) / G;
  const char* wb = static_cast<const char*>(w);
  const char* bb = static_cast<const char*>(bias);
  for (int64_t g0 = 0; g0 < NG; g0 += groups_per_chunk) {
    const int64_t g1 = g0 + groups_per_chunk < NG ? g0 + groups_per_chunk : NG;
    const int64_t l0 = g0 * G, l1 = g1 * G < L ? g1 * G : L, C = l1 - l0;
    const int64_t zw = (C + 7) / 8 * 8;        // the forward writes zeros into the columns that pad the last group's row
    if (int rc = launch_forward(loc + g0 * F, xt, wb + l0 * F * 2, bias ? bb + l0 * 2 : nullptr, zbuf, B, D, F, C, G, ldz, zw, st)) return rc;
    if (int rc = launch_topk_update(zbuf, ldz, B, C, label0 + l0, k, vals, idx, st)) return rc;
  }
  return HASTE_OK;
}

int haste_ffi_check_locations(const int32_t* loc, int64_t n, int64_t D, haste_stream_t stream) {
  const char* who = "haste_ffi_check_locations";
  REQUIRE_PTR(loc, who);
  return launch_check_loc(loc, n, D, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
