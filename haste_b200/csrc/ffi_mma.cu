// Grouped fixed-fan-in GEMM kernels on warp-level mma (m16n8k16 bf16, fp32 accumulate).
//
// These kernels serve every (G,F,B) shape: the forward, the backward entry points and the fused
// step of the two benchmark layer shapes dispatch to the tcgen05 kernels, everything else (other
// group sizes and fan-ins, batch sizes that are not multiples of 8, misaligned bases) runs here.
// One device routine, warp_gemm_tn, serves all three products because the three
// shared-memory tiles of a group can each play two roles without being transposed:
//     Xs [F][BT]  gathered rows of xt (batch contiguous)
//     Ws [G][F]   the group's weight rows
//     Ys [BT][G]  the group's slice of dY
//   forward            Z [b][l]  = sum_k Xs[k][b] * Ws[l][k]
//   backward-weights   dW[l][k]  = sum_b Ys[b][l] * Xs[k][b]
//   backward-features  dXg[k][b] = sum_l Ws[l][k] * Ys[b][l]
// i.e. always C[m][n] += sum_kk A[kk][m] * Bm[n][kk] with A stored kk-major rows (m contiguous) and
// Bm stored n-major rows (kk contiguous).
#include "common.cuh"
#include "launchers.h"

namespace haste {

constexpr int NT = 256;   // threads per CTA
constexpr int BT = 128;   // batch rows per tile
constexpr int PAD = 8;    // bf16 elements of row padding (16 B): keeps ldmatrix conflict-free

// ---------------------------------------------------------------- mma primitives
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x2(uint32_t (&r)[2], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// C[m0 + 16*mi + .., n0 + 8*ni + ..] += sum_{kk<K} A[kk][m] * Bm[n][kk]  for mi < mi_n, ni < ni_n.
// Accumulator fragment: c[0],c[1] -> (row lane/4, cols 2*(lane%4)+{0,1}); c[2],c[3] -> row + 8.
template <int MI, int NI>
__device__ __forceinline__ void warp_gemm_tn(float (&acc)[MI][NI][4], const __nv_bfloat16* A, int lda,
                                             const __nv_bfloat16* Bm, int ldb, int m0, int n0, int K, int mi_n,
                                             int ni_n, int lane) {
  const int ai = lane >> 3, aj = lane & 7;
  const int bi = (lane >> 3) & 1;
  for (int k0 = 0; k0 < K; k0 += 16) {
    uint32_t a[MI][4];
#pragma unroll
    for (int mi = 0; mi < MI; ++mi)
      if (mi < mi_n) ldsm_x4_trans(a[mi], A + (k0 + (ai >> 1) * 8 + aj) * lda + m0 + mi * 16 + (ai & 1) * 8);
#pragma unroll
    for (int ni = 0; ni < NI; ++ni) {
      if (ni < ni_n) {
        uint32_t b[2];
        ldsm_x2(b, Bm + (n0 + ni * 8 + aj) * ldb + k0 + bi * 8);
#pragma unroll
        for (int mi = 0; mi < MI; ++mi)
          if (mi < mi_n) mma16816(acc[mi][ni], a[mi], b);
      }
    }
  }
}

template <int MI, int NI>
__device__ __forceinline__ void zero_acc(float (&acc)[MI][NI][4]) {
#pragma unroll
  for (int i = 0; i < MI; ++i)
#pragma unroll
    for (int j = 0; j < NI; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[i][j][c] = 0.f;
}

// ---------------------------------------------------------------- tile loaders
// rows x cols (cols % 8 == 0) bf16 tile -> shared, zero fill outside [rows_valid, cols_valid).
// ROWPTR(r) returns the global pointer of row r (nullptr = zero row).
template <class ROWPTR>
__device__ __forceinline__ void load_tile(__nv_bfloat16* s, int lds, int rows, int cols, int cols_valid, ROWPTR rowptr,
                                          int tid) {
  const int chunks = cols >> 3;
  for (int idx = tid; idx < rows * chunks; idx += NT) {
    const int r = idx / chunks, c = (idx - r * chunks) << 3;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    const __nv_bfloat16* p = rowptr(r);
    if (p != nullptr && c < cols_valid) {
      p += c;
      if (c + 8 <= cols_valid && (reinterpret_cast<uintptr_t>(p) & 15u) == 0) {
        v = __ldg(reinterpret_cast<const uint4*>(p));
      } else {
        uint16_t e[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) e[i] = (c + i < cols_valid) ? __ldg(reinterpret_cast<const uint16_t*>(p) + i) : uint16_t(0);
        v.x = e[0] | (uint32_t(e[1]) << 16); v.y = e[2] | (uint32_t(e[3]) << 16);
        v.z = e[4] | (uint32_t(e[5]) << 16); v.w = e[6] | (uint32_t(e[7]) << 16);
      }
    }
    *reinterpret_cast<uint4*>(s + r * lds + c) = v;
  }
}


__device__ __forceinline__ void load_loc(int* locs, const int32_t* loc_row, int F, int D, int tid) {
  for (int k = tid; k < F; k += NT) {
    int v = __ldg(loc_row + k);
    locs[k] = min(max(v, 0), D - 1);   // clamp: an out-of-range index can never address outside xt/dxt
  }
}

__device__ __forceinline__ void load_W(__nv_bfloat16* Ws, int ldw, const __nv_bfloat16* w, int64_t l0, int rows_real, int G,
                                       int F, int tid) {
  load_tile(Ws, ldw, G, F, F, [&](int r) { return r < rows_real ? w + (l0 + r) * F : nullptr; }, tid);
}
__device__ __forceinline__ void load_X(__nv_bfloat16* Xs, int ldx, const __nv_bfloat16* xt, const int* locs, int F, int64_t B,
                                       int64_t b0, int tid) {
  const int valid = static_cast<int>(imin64(BT, B - b0));
  load_tile(Xs, ldx, F, BT, valid, [&](int r) { return xt + static_cast<int64_t>(locs[r]) * B + b0; }, tid);
}
__device__ __forceinline__ void load_Y(__nv_bfloat16* Ys, int ldy_s, const __nv_bfloat16* dy, int64_t ldy, int64_t B, int64_t b0,
                                       int64_t l0, int rows_real, int G, int tid) {
  const int bvalid = static_cast<int>(imin64(BT, B - b0));
  load_tile(Ys, ldy_s, BT, G, rows_real, [&](int r) { return r < bvalid ? dy + (b0 + r) * ldy + l0 : nullptr; }, tid);
}

// ================================================================ forward
template <int G>
__global__ void __launch_bounds__(NT) ffi_forward_kernel(const int32_t* __restrict__ loc, const __nv_bfloat16* __restrict__ xt,
                                                         const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ bias,
                                                         __nv_bfloat16* __restrict__ z, int64_t B, int D, int F, int64_t L,
                                                         int64_t ldz, int64_t zw) {
  extern __shared__ __align__(16) unsigned char smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = blockIdx.x;
  const int64_t b0 = static_cast<int64_t>(blockIdx.y) * BT;
  const int64_t l0 = static_cast<int64_t>(g) * G;
  const int rows_real = static_cast<int>(imin64(G, L - l0));
  const int ldx = BT + PAD, ldw = F + PAD, ldc = G + PAD;
  int* locs = reinterpret_cast<int*>(smem);
  __nv_bfloat16* Xs = reinterpret_cast<__nv_bfloat16*>(smem + 512);
  __nv_bfloat16* Ws = Xs + F * ldx;
  __nv_bfloat16* Cs = Ws + G * ldw;

  load_loc(locs, loc + static_cast<int64_t>(g) * F, F, D, tid);
  load_W(Ws, ldw, w, l0, rows_real, G, F, tid);
  __syncthreads();
  load_X(Xs, ldx, xt, locs, F, B, b0, tid);
  __syncthreads();

  float acc[1][G / 8][4];
  zero_acc(acc);
  const int m0 = warp * 16;
  warp_gemm_tn<1, G / 8>(acc, Xs, ldx, Ws, ldw, m0, 0, F, 1, G / 8, lane);

  const int qr = lane >> 2, qc = (lane & 3) * 2;
#pragma unroll
  for (int ni = 0; ni < G / 8; ++ni) {
    const int c = ni * 8 + qc;
    float b0v = 0.f, b1v = 0.f;
    if (bias != nullptr) {
      if (c < rows_real) b0v = __bfloat162float(bias[l0 + c]);
      if (c + 1 < rows_real) b1v = __bfloat162float(bias[l0 + c + 1]);
    }
    *reinterpret_cast<__nv_bfloat162*>(Cs + (m0 + qr) * ldc + c) = __floats2bfloat162_rn(acc[0][ni][0] + b0v, acc[0][ni][1] + b1v);
    *reinterpret_cast<__nv_bfloat162*>(Cs + (m0 + qr + 8) * ldc + c) = __floats2bfloat162_rn(acc[0][ni][2] + b0v, acc[0][ni][3] + b1v);
  }
  __syncthreads();
  // coalesced store of the [BT][G] tile; columns up to zw (the writable width of a row) are written (zeros past L)
  const int cvalid = static_cast<int>(imin64(G, zw - l0));
  const int bvalid = static_cast<int>(imin64(BT, B - b0));
  constexpr int CH = G / 8;
  for (int idx = tid; idx < BT * CH; idx += NT) {
    const int r = idx / CH, c = (idx % CH) * 8;
    if (r >= bvalid || c >= cvalid) continue;
    __nv_bfloat16* dst = z + (b0 + r) * ldz + l0 + c;
    const uint4 v = *reinterpret_cast<const uint4*>(Cs + r * ldc + c);
    if (c + 8 <= cvalid && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
      *reinterpret_cast<uint4*>(dst) = v;
    } else {
      const uint16_t* e = reinterpret_cast<const uint16_t*>(&v);
      for (int i = 0; i < 8 && c + i < cvalid; ++i) reinterpret_cast<uint16_t*>(dst)[i] = e[i];
    }
  }
}

// ================================================================ backward features
__device__ __forceinline__ void red_add_v2(float* p, float a, float b) {
  asm volatile("red.global.add.v2.f32 [%0], {%1, %2};\n" ::"l"(p), "f"(a), "f"(b) : "memory");
}

// Adds the [F][BT] accumulator tile (rows = slots, cols = batch) into dxt rows loc[k].
template <int MI>
__device__ __forceinline__ void scatter_dx(const float (&acc)[MI][2][4], float* dxt, const int* locs, int F, int64_t B,
                                           int64_t b0, int n0, int lane) {
  const int qr = lane >> 2, qc = (lane & 3) * 2;
  const bool even = (B & 1) == 0;
#pragma unroll
  for (int mi = 0; mi < MI; ++mi) {
    if (mi * 16 >= F) continue;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int k = mi * 16 + qr + h * 8;
      float* row = dxt + static_cast<int64_t>(locs[k]) * B;
#pragma unroll
      for (int ni = 0; ni < 2; ++ni) {
        const int64_t b = b0 + n0 + ni * 8 + qc;
        const float v0 = acc[mi][ni][h * 2], v1 = acc[mi][ni][h * 2 + 1];
        if (even && b + 1 < B) {
          red_add_v2(row + b, v0, v1);
        } else {
          if (b < B) atomicAdd(row + b, v0);
          if (b + 1 < B) atomicAdd(row + b + 1, v1);
        }
      }
    }
  }
}

template <int G, int FMAX>
__global__ void __launch_bounds__(NT) ffi_bwd_features_kernel(const __nv_bfloat16* __restrict__ w, const int32_t* __restrict__ loc,
                                                              const __nv_bfloat16* __restrict__ dy, float* __restrict__ dxt, int64_t B,
                                                              int D, int F, int64_t L, int64_t ldy) {
  extern __shared__ __align__(16) unsigned char smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = blockIdx.x;
  const int64_t b0 = static_cast<int64_t>(blockIdx.y) * BT;
  const int64_t l0 = static_cast<int64_t>(g) * G;
  const int rows_real = static_cast<int>(imin64(G, L - l0));
  const int ldw = F + PAD, ldys = G + PAD;
  int* locs = reinterpret_cast<int*>(smem);
  __nv_bfloat16* Ws = reinterpret_cast<__nv_bfloat16*>(smem + 512);
  __nv_bfloat16* Ys = Ws + G * ldw;
  load_loc(locs, loc + static_cast<int64_t>(g) * F, F, D, tid);
  load_W(Ws, ldw, w, l0, rows_real, G, F, tid);
  load_Y(Ys, ldys, dy, ldy, B, b0, l0, rows_real, G, tid);
  __syncthreads();
  float acc[FMAX / 16][2][4];
  zero_acc(acc);
  const int n0 = warp * 16;
  warp_gemm_tn<FMAX / 16, 2>(acc, Ws, ldw, Ys, ldys, 0, n0, G, F / 16, 2, lane);
  scatter_dx<FMAX / 16>(acc, dxt, locs, F, B, b0, n0, lane);
}

// ================================================================ backward weights (+ fused update)
template <int G, int FMAX>
struct BwwTiling {
  static constexpr int WARPS_M = G / 16;                       // 1,2,4,8
  static constexpr int WARPS_N = 8 / WARPS_M;                  // 8,4,2,1
  static constexpr int NI = (FMAX / 8 / WARPS_N) > 0 ? (FMAX / 8 / WARPS_N) : 1;
};


// Quad-cooperative random bits, packed stream: the 8 slots of one 8-wide n-tile of a label row are
// the four words of ONE Philox call, and lane t of the quad owns slots 2t,2t+1 = word t.  The
// quad's calls (2 rows x NI n-tiles) are dealt round-robin to its 4 lanes and the words exchanged.
template <int NI>
__device__ __forceinline__ void quad_packed_bits(uint32_t (&word)[NI][2], uint64_t seed, uint32_t step, int64_t row_lo,
                                                 int64_t row_hi, int n0, int lane) {
  const int t = lane & 3, qbase = lane & ~3;
  constexpr int Q = NI * 2;
#pragma unroll
  for (int c0 = 0; c0 < Q; c0 += 4) {
    const int c = c0 + t;
    uint4 r = make_uint4(0, 0, 0, 0);
    if (c < Q) r = rand_packed8(seed, step, (c & 1) ? row_hi : row_lo, (n0 >> 3) + (c >> 1));
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) {
      if (c0 + cc < Q) {
        const uint32_t x = __shfl_sync(0xffffffffu, r.x, qbase + cc), y = __shfl_sync(0xffffffffu, r.y, qbase + cc);
        const uint32_t zz = __shfl_sync(0xffffffffu, r.z, qbase + cc), ww = __shfl_sync(0xffffffffu, r.w, qbase + cc);
        word[(c0 + cc) >> 1][(c0 + cc) & 1] = t == 0 ? x : t == 1 ? y : t == 2 ? zz : ww;
      }
    }
  }
}

// Epilogue of backward-weights on the [G][F] accumulator owned as (row qr / qr+8, cols n0+ni*8+qc..+1).
template <int NI, bool FUSED>
__device__ __forceinline__ void bww_epilogue(const float (&acc)[1][NI][4], __nv_bfloat16* dw, const UpdateArgs& u, int64_t l0,
                                             int rows_real, int F, int m0, int n0, int lane) {
  const int qr = lane >> 2, qc = (lane & 3) * 2;
  const int r_lo = m0 + qr, r_hi = m0 + qr + 8;
  uint32_t word[NI][2];
  if (FUSED && (u.flags & HASTE_F_SR) && (u.flags & HASTE_F_RNG_PACKED))
    quad_packed_bits<NI>(word, u.seed, u.step, u.label0 + l0 + r_lo, u.label0 + l0 + r_hi, n0, lane);
#pragma unroll
  for (int ni = 0; ni < NI; ++ni) {
    const int k = n0 + ni * 8 + qc;
    if (k >= F) continue;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = h ? r_hi : r_lo;
      if (r >= rows_real) continue;
      const int64_t off = (l0 + r) * F + k;
      // the gradient is rounded to bf16 first, exactly what the unfused kernel stores
      const __nv_bfloat162 g2 = __floats2bfloat162_rn(acc[0][ni][h * 2], acc[0][ni][h * 2 + 1]);
      if (!FUSED) {
        *reinterpret_cast<__nv_bfloat162*>(dw + off) = g2;
      } else {
        const uint32_t wb = *reinterpret_cast<const uint32_t*>(u.w + off);
        uint32_t r0 = 0, r1 = 0;
        if (u.flags & HASTE_F_SR) {
          if (u.flags & HASTE_F_RNG_PACKED) {
            r0 = word[ni][h] & 0xFFFFu; r1 = word[ni][h] >> 16;
          } else {
            const int64_t grow = u.label0 + l0 + r;
            r0 = rand16_reference(u.seed, grow * F + k); r1 = rand16_reference(u.seed, grow * F + k + 1);
          }
        }
        float2 m = make_float2(0.f, 0.f);
        const bool use_m = u.mom_w != nullptr;
        if (use_m) m = *reinterpret_cast<const float2*>(u.mom_w + off);
        const uint16_t n0b = sgd_update_bits(wb & 0xFFFFu, __low2float(g2), use_m ? &m.x : nullptr, u.lr, u.wd, u.mu, u.flags, r0);
        const uint16_t n1b = sgd_update_bits(wb >> 16, __high2float(g2), use_m ? &m.y : nullptr, u.lr, u.wd, u.mu, u.flags, r1);
        *reinterpret_cast<uint32_t*>(u.w + off) = uint32_t(n0b) | (uint32_t(n1b) << 16);
        if (use_m) *reinterpret_cast<float2*>(u.mom_w + off) = m;
      }
    }
  }
}

// bias: gradient = column sum of dY (fp32), rounded to bf16, then the same update with flat index l
__device__ __forceinline__ void bias_update(float dsum, int64_t l, const UpdateArgs& u) {
  const float g = round_to_bf16_f(dsum);
  const int64_t gl = u.label0 + l;
  uint32_t r = 0;
  if (u.flags & HASTE_F_SR) r = rand16(u.flags, u.seed ^ ((u.flags & HASTE_F_RNG_PACKED) ? 0x62696173ull : 0ull), u.step, gl, 0, 1);
  float m = 0.f;
  const bool use_m = u.mom_b != nullptr;
  if (use_m) m = u.mom_b[l];
  const uint16_t nb = sgd_update_bits(__bfloat16_as_ushort(u.bias[l]), g, use_m ? &m : nullptr, u.lr, u.wd, u.mu, u.flags, r);
  u.bias[l] = __ushort_as_bfloat16(nb);
  if (use_m) u.mom_b[l] = m;
}

template <int G, int FMAX, bool FUSED>
__global__ void __launch_bounds__(NT) ffi_bwd_weights_kernel(const __nv_bfloat16* __restrict__ xt, const int32_t* __restrict__ loc,
                                                             const __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ dw,
                                                             __nv_bfloat16* __restrict__ dbias, UpdateArgs u, int64_t B, int D, int F,
                                                             int64_t L, int64_t ldy) {
  using T = BwwTiling<G, FMAX>;
  extern __shared__ __align__(16) unsigned char smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = blockIdx.x;
  const int64_t l0 = static_cast<int64_t>(g) * G;
  const int rows_real = static_cast<int>(imin64(G, L - l0));
  const int ldx = BT + PAD, ldys = G + PAD;
  int* locs = reinterpret_cast<int*>(smem);
  __nv_bfloat16* Xs = reinterpret_cast<__nv_bfloat16*>(smem + 512);
  __nv_bfloat16* Ys = Xs + F * ldx;
  load_loc(locs, loc + static_cast<int64_t>(g) * F, F, D, tid);
  __syncthreads();

  float acc[1][T::NI][4];
  zero_acc(acc);
  const int wm = warp % T::WARPS_M, wn = warp / T::WARPS_M;
  const int m0 = wm * 16, n0 = wn * T::NI * 8;
  const int ni_n = max(0, min(T::NI, (F - n0) / 8));
  float bsum = 0.f;
  for (int64_t b0 = 0; b0 < B; b0 += BT) {
    load_X(Xs, ldx, xt, locs, F, B, b0, tid);
    load_Y(Ys, ldys, dy, ldy, B, b0, l0, rows_real, G, tid);
    __syncthreads();
    if (ni_n > 0) warp_gemm_tn<1, T::NI>(acc, Ys, ldys, Xs, ldx, m0, n0, BT, 1, ni_n, lane);
    if (tid < G) {
      float s = 0.f;
      for (int r = 0; r < BT; ++r) s += __bfloat162float(Ys[r * ldys + tid]);
      bsum += s;
    }
    __syncthreads();
  }
  bww_epilogue<T::NI, FUSED>(acc, dw, u, l0, rows_real, F, m0, n0, lane);
  if (tid < rows_real) {
    if (!FUSED) {
      if (dbias != nullptr) dbias[l0 + tid] = __float2bfloat16_rn(bsum);
    } else if (u.bias != nullptr) {
      bias_update(bsum, l0 + tid, u);
    }
  }
}

// ================================================================ fused train step (mma variant)
template <int G, int FMAX, int LOSS, bool WITH_LOSS>
__global__ void __launch_bounds__(NT, 1) ffi_train_step_mma_kernel(const int32_t* __restrict__ loc, const __nv_bfloat16* __restrict__ xt,
                                                                   const int32_t* __restrict__ tgt_ptr, const uint32_t* __restrict__ tgt_ent,
                                                                   float* __restrict__ dxt, float* __restrict__ loss, UpdateArgs u,
                                                                   int64_t B, int D, int F, int64_t L, float grad_scale) {
  using T = BwwTiling<G, FMAX>;
  extern __shared__ __align__(16) unsigned char smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = blockIdx.x;
  const int64_t l0 = static_cast<int64_t>(g) * G;
  const int rows_real = static_cast<int>(imin64(G, L - l0));
  const int ldx = BT + PAD, ldw = F + PAD, ldys = G + PAD;
  constexpr int YW = (G + 31) / 32;                         // bitmap words per batch row
  int* locs = reinterpret_cast<int*>(smem);                 // 512 B
  uint32_t* ybits = reinterpret_cast<uint32_t*>(smem + 512);  // BT*YW*4 B
  float* bias_s = reinterpret_cast<float*>(smem + 512 + BT * YW * 4);   // G floats
  __nv_bfloat16* Xs = reinterpret_cast<__nv_bfloat16*>(smem + 512 + BT * YW * 4 + G * 4);
  __nv_bfloat16* Ws = Xs + F * ldx;
  __nv_bfloat16* Ys = Ws + G * ldw;

  load_loc(locs, loc + static_cast<int64_t>(g) * F, F, D, tid);
  load_W(Ws, ldw, u.w, l0, rows_real, G, F, tid);
  if (tid < G) bias_s[tid] = (u.bias != nullptr && tid < rows_real) ? __bfloat162float(u.bias[l0 + tid]) : 0.f;
  const int t_beg = __ldg(tgt_ptr + g), t_end = __ldg(tgt_ptr + g + 1);
  __syncthreads();

  float accw[1][T::NI][4];
  zero_acc(accw);
  const int wm = warp % T::WARPS_M, wn = warp / T::WARPS_M;
  const int m0w = wm * 16, n0w = wn * T::NI * 8;
  const int ni_w = max(0, min(T::NI, (F - n0w) / 8));
  const int qr = lane >> 2, qc = (lane & 3) * 2;
  float bsum = 0.f, loss_acc = 0.f;

  for (int64_t b0 = 0; b0 < B; b0 += BT) {
    const int bvalid = static_cast<int>(imin64(BT, B - b0));
    load_X(Xs, ldx, xt, locs, F, B, b0, tid);
    for (int i = tid; i < BT * YW; i += NT) ybits[i] = 0u;
    __syncthreads();
    for (int i = t_beg + tid; i < t_end; i += NT) {
      const uint32_t e = __ldg(tgt_ent + i);
      const int64_t b = static_cast<int64_t>(e >> 8) - b0;
      const int c = e & 0xFF;
      if (b >= 0 && b < BT) atomicOr(&ybits[b * YW + (c >> 5)], 1u << (c & 31));
    }
    __syncthreads();
    {  // forward tile + loss gradient -> Ys
      float acc[1][G / 8][4];
      zero_acc(acc);
      const int m0 = warp * 16;
      warp_gemm_tn<1, G / 8>(acc, Xs, ldx, Ws, ldw, m0, 0, F, 1, G / 8, lane);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int r = m0 + qr + h * 8;
        const bool rvalid = r < bvalid;
#pragma unroll
        for (int ni = 0; ni < G / 8; ++ni) {
          const int c = ni * 8 + qc;
          const uint32_t yb = ybits[r * YW + (c >> 5)] >> (c & 31);
          float gq[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const float zv = round_to_bf16_f(acc[0][ni][h * 2 + e] + bias_s[c + e]);
            float gl = 0.f, la = 0.f;
            if (rvalid && c + e < rows_real) {
              gl = loss_grad<LOSS, WITH_LOSS>(zv, (yb >> e) & 1u, la) * grad_scale;
              if (WITH_LOSS) loss_acc += la;
            }
            gq[e] = gl;
          }
          *reinterpret_cast<__nv_bfloat162*>(Ys + r * ldys + c) = __floats2bfloat162_rn(gq[0], gq[1]);
        }
      }
    }
    __syncthreads();
    {  // backward features: dXg[k][b] = sum_l Ws[l][k] * Ys[b][l]
      float acc[FMAX / 16][2][4];
      zero_acc(acc);
      const int n0 = warp * 16;
      warp_gemm_tn<FMAX / 16, 2>(acc, Ws, ldw, Ys, ldys, 0, n0, G, F / 16, 2, lane);
      scatter_dx<FMAX / 16>(acc, dxt, locs, F, B, b0, n0, lane);
    }
    if (ni_w > 0) warp_gemm_tn<1, T::NI>(accw, Ys, ldys, Xs, ldx, m0w, n0w, BT, 1, ni_w, lane);
    if (u.bias != nullptr && tid < G) {
      float s = 0.f;
      for (int r = 0; r < BT; ++r) s += __bfloat162float(Ys[r * ldys + tid]);
      bsum += s;
    }
    __syncthreads();
  }
  bww_epilogue<T::NI, true>(accw, nullptr, u, l0, rows_real, F, m0w, n0w, lane);
  if (u.bias != nullptr && tid < rows_real) bias_update(bsum, l0 + tid, u);
  if (WITH_LOSS) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) loss_acc += __shfl_xor_sync(0xffffffffu, loss_acc, o);
    if (lane == 0) atomicAdd(loss, loss_acc * grad_scale);
  }
}

// ================================================================ host launchers
static size_t fwd_smem(int G, int F) { return 512 + size_t(F) * (BT + PAD) * 2 + size_t(G) * (F + PAD) * 2 + size_t(BT) * (G + PAD) * 2; }
static size_t bwx_smem(int G, int F) { return 512 + size_t(G) * (F + PAD) * 2 + size_t(BT) * (G + PAD) * 2; }
static size_t bww_smem(int G, int F) { return 512 + size_t(F) * (BT + PAD) * 2 + size_t(BT) * (G + PAD) * 2; }
static size_t step_smem(int G, int F) {
  return 512 + size_t(BT) * ((G + 31) / 32) * 4 + size_t(G) * 4 + size_t(F) * (BT + PAD) * 2 + size_t(G) * (F + PAD) * 2 +
         size_t(BT) * (G + PAD) * 2;
}

template <class K>
static int set_smem(K kernel, size_t bytes) {
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes));
  if (e != cudaSuccess) return fail(HASTE_ERR_LAUNCH, "cudaFuncSetAttribute(%zu B): %s", bytes, cudaGetErrorString(e));
  return HASTE_OK;
}

#define HASTE_DISPATCH_G(G, ...)                    \
  switch (G) {                                      \
    case 16: { constexpr int G_ = 16; __VA_ARGS__; } break;   \
    case 32: { constexpr int G_ = 32; __VA_ARGS__; } break;   \
    case 64: { constexpr int G_ = 64; __VA_ARGS__; } break;   \
    case 128: { constexpr int G_ = 128; __VA_ARGS__; } break; \
    default: return fail(HASTE_ERR_UNSUPPORTED, "group size %d not in {16,32,64,128}", int(G)); \
  }
#define HASTE_DISPATCH_F(F, ...)                                   \
  if (F <= 32) { constexpr int F_ = 32; __VA_ARGS__; }             \
  else if (F <= 64) { constexpr int F_ = 64; __VA_ARGS__; }        \
  else { constexpr int F_ = 128; __VA_ARGS__; }

int launch_forward(const int32_t* loc, const void* xt, const void* w, const void* bias, void* z, int64_t B, int64_t D, int64_t F,
                   int64_t L, int64_t G, int64_t ldz, int64_t zw, cudaStream_t st) {
  // Shape dispatch: the tcgen05 kernel where its tile shapes apply, the warp-mma kernel otherwise
  if (zw >= 8 && forward_sm100_supported(z, xt, w, B, F, L, G, ldz)) return launch_forward_sm100(loc, xt, w, bias, z, B, D, F, L, G, ldz, zw, st);
  const int64_t NG = (L + G - 1) / G;
  dim3 grid(static_cast<unsigned>(NG), static_cast<unsigned>((B + BT - 1) / BT));
  const size_t sm = fwd_smem(int(G), int(F));
  HASTE_DISPATCH_G(G, {
    auto k = ffi_forward_kernel<G_>;
    if (int rc = set_smem(k, sm)) return rc;
    k<<<grid, NT, sm, st>>>(loc, (const __nv_bfloat16*)xt, (const __nv_bfloat16*)w, (const __nv_bfloat16*)bias, (__nv_bfloat16*)z, B,
                            int(D), int(F), L, ldz, zw);
  });
  return check_launch("ffi_forward_kernel");
}

int launch_bwd_features(const void* w, const int32_t* loc, const void* dy, float* dxt, int64_t B, int64_t D, int64_t F, int64_t L,
                        int64_t G, int64_t ldy, cudaStream_t st) {
  const int64_t NG = (L + G - 1) / G;
  dim3 grid(static_cast<unsigned>(NG), static_cast<unsigned>((B + BT - 1) / BT));
  const size_t sm = bwx_smem(int(G), int(F));
  HASTE_DISPATCH_G(G, HASTE_DISPATCH_F(F, {
    auto k = ffi_bwd_features_kernel<G_, F_>;
    if (int rc = set_smem(k, sm)) return rc;
    k<<<grid, NT, sm, st>>>((const __nv_bfloat16*)w, loc, (const __nv_bfloat16*)dy, dxt, B, int(D), int(F), L, ldy);
  }));
  return check_launch("ffi_bwd_features_kernel");
}

int launch_bwd_weights(const void* xt, const int32_t* loc, const void* dy, void* dw, void* dbias, const UpdateArgs* upd, int64_t B,
                       int64_t D, int64_t F, int64_t L, int64_t G, int64_t ldy, cudaStream_t st) {
  const int64_t NG = (L + G - 1) / G;
  dim3 grid(static_cast<unsigned>(NG));
  const size_t sm = bww_smem(int(G), int(F));
  UpdateArgs u{};
  if (upd) u = *upd;
  HASTE_DISPATCH_G(G, HASTE_DISPATCH_F(F, {
    if (upd) {
      auto k = ffi_bwd_weights_kernel<G_, F_, true>;
      if (int rc = set_smem(k, sm)) return rc;
      k<<<grid, NT, sm, st>>>((const __nv_bfloat16*)xt, loc, (const __nv_bfloat16*)dy, nullptr, nullptr, u, B, int(D), int(F), L, ldy);
    } else {
      auto k = ffi_bwd_weights_kernel<G_, F_, false>;
      if (int rc = set_smem(k, sm)) return rc;
      k<<<grid, NT, sm, st>>>((const __nv_bfloat16*)xt, loc, (const __nv_bfloat16*)dy, (__nv_bfloat16*)dw, (__nv_bfloat16*)dbias, u, B,
                              int(D), int(F), L, ldy);
    }
  }));
  return check_launch("ffi_bwd_weights_kernel");
}

int launch_train_step_mma(const int32_t* loc, const void* xt, const int32_t* tgt_ptr, const uint32_t* tgt_ent, float* dxt, float* loss,
                          const UpdateArgs& u, int64_t B, int64_t D, int64_t F, int64_t L, int64_t G, int loss_kind, float grad_scale,
                          cudaStream_t st) {
  const int64_t NG = (L + G - 1) / G;
  dim3 grid(static_cast<unsigned>(NG));
  const size_t sm = step_smem(int(G), int(F));
  const bool wl = (u.flags & HASTE_F_LOSS) && loss != nullptr;
#define HASTE_LAUNCH_STEP(LOSSK, WL)                                                                          \
  {                                                                                                           \
    auto k = ffi_train_step_mma_kernel<G_, F_, LOSSK, WL>;                                                    \
    if (int rc = set_smem(k, sm)) return rc;                                                                  \
    k<<<grid, NT, sm, st>>>(loc, (const __nv_bfloat16*)xt, tgt_ptr, tgt_ent, dxt, loss, u, B, int(D), int(F), L, grad_scale); \
  }
  HASTE_DISPATCH_G(G, HASTE_DISPATCH_F(F, {
    if (loss_kind == HASTE_LOSS_BCE) { if (wl) HASTE_LAUNCH_STEP(HASTE_LOSS_BCE, true) else HASTE_LAUNCH_STEP(HASTE_LOSS_BCE, false) }
    else { if (wl) HASTE_LAUNCH_STEP(HASTE_LOSS_SQHINGE, true) else HASTE_LAUNCH_STEP(HASTE_LOSS_SQHINGE, false) }
  }));
#undef HASTE_LAUNCH_STEP
  return check_launch("ffi_train_step_mma_kernel");
}

}  // namespace haste

