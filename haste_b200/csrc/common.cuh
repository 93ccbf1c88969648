// Shared device/host helpers for the FFI kernels: error reporting, Philox4x32-10, stochastic
// rounding, the fp32 SGD arithmetic, and small bf16 utilities.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>

#include "../../include/haste_ffi.h"

namespace haste {

// ---------------------------------------------------------------- host error plumbing
int fail(int code, const char* fmt, ...);
int check_launch(const char* what);
int validate_shape(const char* who, int64_t B, int64_t D, int64_t F, int64_t L, int64_t G);

__host__ __device__ __forceinline__ int64_t imin64(int64_t a, int64_t b) { return a < b ? a : b; }
static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---------------------------------------------------------------- Philox4x32-10
// Same generator as triton.language.random.philox_impl (which the reference reaches through
// tl.randint at shared_ffi/sr_triton.py:11): round constants 0xD2511F53 / 0xCD9E8D57, key
// increments 0x9E3779B9 / 0xBB67AE85, ten rounds.
__device__ __forceinline__ uint4 philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                               uint32_t k0, uint32_t k1) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    c0 = hi1 ^ c1 ^ k0;
    c2 = hi0 ^ c3 ^ k1;
    c1 = lo1;
    c3 = lo0;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return make_uint4(c0, c1, c2, c3);
}

// 16 random bits for element (row, col) of a [rows, cols] parameter.
//   reference stream: tl.randint(seed, row*cols + col) & 0xFFFF  (int32 offsets, counter word 0)
//   packed stream   : key (seed_lo, step), counter (row, col>>3, 0, 0); slot col uses half (col&1)
//                     of word ((col&7)>>1) — callers that own 8 consecutive slots call
//                     philox4x32_10 once and unpack themselves.
__device__ __forceinline__ uint32_t rand16_reference(uint64_t seed, int64_t flat) {
  const uint4 r = philox4x32_10(static_cast<uint32_t>(flat), 0u, 0u, 0u, static_cast<uint32_t>(seed),
                                static_cast<uint32_t>(seed >> 32));
  return r.x & 0xFFFFu;
}
__device__ __forceinline__ uint4 rand_packed8(uint64_t seed, uint32_t step, int64_t row, int col8) {
  return philox4x32_10(static_cast<uint32_t>(row), static_cast<uint32_t>(col8), 0u, 0u,
                       static_cast<uint32_t>(seed), step);
}
__device__ __forceinline__ uint32_t unpack16(const uint4& r, int slot_in_8) {
  const uint32_t wsel = (slot_in_8 >> 1);
  const uint32_t w = wsel == 0 ? r.x : wsel == 1 ? r.y : wsel == 2 ? r.z : r.w;
  return (w >> (16 * (slot_in_8 & 1))) & 0xFFFFu;
}
__device__ __forceinline__ uint32_t rand16(uint32_t flags, uint64_t seed, uint32_t step, int64_t row, int col,
                                           int cols) {
  if (flags & HASTE_F_RNG_PACKED) return unpack16(rand_packed8(seed, step, row, col >> 3), col & 7);
  return rand16_reference(seed, row * cols + col);
}

// ---------------------------------------------------------------- rounding
// Stochastic rounding of shared_ffi/sr_triton.py:10-16: add 16 random bits to the fp32 pattern as
// an integer and keep the high half.
__device__ __forceinline__ uint16_t sr_bf16_bits(float v, uint32_t r16) {
  return static_cast<uint16_t>((__float_as_uint(v) + r16) >> 16);
}
__device__ __forceinline__ uint16_t rn_bf16_bits(float v) {
  return __bfloat16_as_ushort(__float2bfloat16_rn(v));
}
__device__ __forceinline__ float bf16_bits_to_float(uint16_t b) { return __uint_as_float(static_cast<uint32_t>(b) << 16); }
__device__ __forceinline__ float round_to_bf16_f(float v) { return bf16_bits_to_float(rn_bf16_bits(v)); }

// ---------------------------------------------------------------- SGD arithmetic (fp32)
// sr_triton.py:140-158.  CONTRACT = fused multiply-add (what the compiled Triton kernel emits with
// fp fusion on); otherwise multiply and add are rounded separately.
template <bool CONTRACT>
__device__ __forceinline__ float sgd_math(float w, float g, float* m, float lr, float wd, float mu) {
  if (CONTRACT) {
    g = __fmaf_rn(wd, w, g);
    if (m) {
      *m = __fmaf_rn(mu, *m, g);
      g = *m;
    }
    return __fmaf_rn(-lr, g, w);
  } else {
    g = __fadd_rn(g, __fmul_rn(wd, w));
    if (m) {
      *m = __fadd_rn(__fmul_rn(mu, *m), g);
      g = *m;
    }
    return __fsub_rn(w, __fmul_rn(lr, g));
  }
}
__device__ __forceinline__ uint16_t sgd_update_bits(uint16_t wbits, float g, float* m, float lr, float wd, float mu,
                                                    uint32_t flags, uint32_t r16) {
  const float w = bf16_bits_to_float(wbits);
  const float wn = (flags & HASTE_F_CONTRACT) ? sgd_math<true>(w, g, m, lr, wd, mu)
                                              : sgd_math<false>(w, g, m, lr, wd, mu);
  return (flags & HASTE_F_SR) ? sr_bf16_bits(wn, r16) : rn_bf16_bits(wn);
}

// ---------------------------------------------------------------- losses
// Returns dLoss/dz for one logit (already rounded to bf16) and adds the loss term to *loss_acc.
//   BCE with logits, sum reduction (src/runner.py:469-478): grad = sigmoid(z) - y.
//   squared hinge, targets +-1: loss = max(0, 1 - s z)^2, grad = -2 s max(0, 1 - s z).
template <int LOSS, bool WITH_LOSS>
__device__ __forceinline__ float loss_grad(float z, bool pos, float& loss_acc) {
  if (LOSS == HASTE_LOSS_BCE) {
    const float e = __expf(-fabsf(z));                 // exp(-|z|) in (0,1]
    const float inv = __frcp_rn(1.0f + e);
    const float sig = z >= 0.f ? inv : e * inv;
    if (WITH_LOSS) loss_acc += fmaxf(z, 0.f) - (pos ? z : 0.f) + __logf(1.0f + e);
    return sig - (pos ? 1.f : 0.f);
  } else {
    const float s = pos ? 1.f : -1.f;
    const float m = fmaxf(0.f, 1.f - s * z);
    if (WITH_LOSS) loss_acc += m * m;
    return -2.f * s * m;
  }
}

}  // namespace haste
