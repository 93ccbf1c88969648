// Unfused backward of the FFI layer on tcgen05 / TMEM, group size 128, fan-in 64: one pass over dY [B, ldy]
// produces both gradients of the autograd surface,
//     dxt[loc[g,k], b] += sum_{l in g} w[l,k] * dy[b,l]          (fp32, reduced into dxt with red.global.add)
//     dw [l, k]         = sum_b dy[b,l] * xt[loc[g,k], b]          (bf16, round to nearest)
//     dbias[l]          = sum_b dy[b,l]                            (bf16; via a row of ones appended to the X tile)
// so dY is read from HBM once instead of once per gradient.  HBM-bound by that read (2*B*L bytes).
//
// Persistent, one CTA per SM.  Same operand layouts as the fused train step: per 128-row batch tile the Y tile
// (dY slice, now copied in by the producers instead of computed by an epilogue), the X tile and the W tile sit
// in 128-byte-swizzled shared memory; backward-features takes Y as K-major A and W as MN-major B,
// backward-weights takes Y as MN-major A and X as K-major B.  Warp roles (672 threads): warps 0, 2 and 16-20 are
// producers (cp.async; one producer warp per ring stage), warp 1 issues backward-features, warp 3
// backward-weights, warps 4-11 drain dXg (TMEM -> registers -> coalesced red.global.add.f32), warps 12-15 turn
// the dW accumulator into bf16 rows of dw / dbias at the end of each group.  Requires 16-byte-aligned dY rows (ldy % 8 == 0).
#include "common.cuh"
#include "launchers.h"
#include "runtime.h"
#include "sm100.cuh"

namespace haste {
namespace b100 {
using namespace sm100;

constexpr int G = 128, F = 64, BT = 128;
constexpr int FR = F + 16;                    // X block rows: F gathered rows, one row of ones, 15 zero rows
constexpr int NXS = 4;
constexpr int XBLK = FR * 128, XSTAGE = 2 * XBLK;   // 20 KB
constexpr int WSTAGE = G * 128;                     // 16 KB
constexpr int YBLK = BT * 128, YSTAGE = 2 * YBLK;   // 32 KB
constexpr int NYS = 3;
constexpr int OFF_X = 0;
constexpr int OFF_W = OFF_X + NXS * XSTAGE;
constexpr int OFF_Y = OFF_W + 2 * WSTAGE;
constexpr int OFF_LOC = OFF_Y + NYS * YSTAGE;       // int [2][F]
constexpr int OFF_BAR = OFF_LOC + 2 * F * 4;
constexpr int OFF_MISC = OFF_BAR + 40 * 8;
constexpr int SMEM_BYTES = OFF_MISC + 64 + 1024;
static_assert(SMEM_BYTES <= 232448, "shared memory budget");
constexpr int B_XFULL = 0, B_XEMPTY = NXS, B_YFULL = 2 * NXS, B_YEMPTY = B_YFULL + NYS, B_WFULL = B_YEMPTY + NYS,
              B_WEMPTY = B_WFULL + 2, B_DXFULL = B_WEMPTY + 2, B_DXEMPTY = B_DXFULL + 2, B_DWFULL = B_DXEMPTY + 2,
              B_DWEMPTY = B_DWFULL + 2, B_LEMPTY = B_DWEMPTY + 2, NBAR = B_LEMPTY + 2;
static_assert(NBAR <= 40, "barrier space");
constexpr int N_EB = 8, N_EC = 4;
constexpr int N_XPROD = 5;                    // producer warps beyond the two among the first four warps
constexpr int NTHREADS = (4 + N_EB + N_EC + N_XPROD) * 32;
constexpr uint32_t TM_DX = 0, TM_DW = 128, TM_DW_STRIDE = 80, TM_COLS = 512;
constexpr long long WAIT_LIMIT = 4000000000ll;

struct BwdArgs {
  const int32_t* loc;
  const __nv_bfloat16* xt;
  const __nv_bfloat16* w;
  const __nv_bfloat16* dy;
  float* dxt;
  __nv_bfloat16* dw;
  __nv_bfloat16* dbias;
  int* err;
  int64_t B, L, ldy;
  int D, NG;
};

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__global__ void __launch_bounds__(NTHREADS, 1) ffi_backward_sm100_kernel(BwdArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const uint32_t sbase = smem_u32(sm);
  int* loc_s = reinterpret_cast<int*>(sm + OFF_LOC);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + OFF_MISC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + OFF_MISC + 8);
  auto bar = [&](int i) { return sbase + OFF_BAR + i * 8; };
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int T = static_cast<int>((a.B + BT - 1) / BT);

  if (tid == 0) {
    for (int i = 0; i < NXS; ++i) { mbar_init(bar(B_XFULL + i), 1); mbar_init(bar(B_XEMPTY + i), 1); }
    for (int i = 0; i < NYS; ++i) { mbar_init(bar(B_YFULL + i), 1); mbar_init(bar(B_YEMPTY + i), 2); }   // both issuers commit
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(B_WFULL + i), 1);  mbar_init(bar(B_WEMPTY + i), 1);
      mbar_init(bar(B_DXFULL + i), 1); mbar_init(bar(B_DXEMPTY + i), N_EB);
      mbar_init(bar(B_DWFULL + i), 1); mbar_init(bar(B_DWEMPTY + i), N_EC);
      mbar_init(bar(B_LEMPTY + i), N_EB);        // the scatter warps are done with the group's index row
    }
    mbar_fence_init();
    *abort_flag = 0;
  }
  // rows F..FR-1 of every X block: row F = ones (bias-gradient column), the rest zeros; written once
  for (int i = tid; i < NXS * 2 * 16 * 8; i += NTHREADS) {
    const int chunk = i & 7, row = (i >> 3) & 15, blk = i >> 7;
    const uint32_t v = (row == 0) ? 0x3F803F80u : 0u;
    *reinterpret_cast<uint4*>(sm + OFF_X + blk * XBLK + (F + row) * 128 + chunk * 16) = make_uint4(v, v, v, v);
  }
  fence_proxy_async();
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), TM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const int n_my_groups = (a.NG > static_cast<int>(blockIdx.x)) ? (a.NG - 1 - static_cast<int>(blockIdx.x)) / static_cast<int>(gridDim.x) + 1 : 0;

  if (warp == 0 || warp == 2 || warp >= 4 + N_EB + N_EC) {
    // ================================================================ producers
    // Each producer warp has one item in flight at a time and pays the full memory latency for it (dY tiles come
    // from HBM), so the load rate is the number of producer warps over that latency.  Every ring stage has its
    // own producer warp — NYS warps for the dY ring, NXS for the X ring, the first X warp also loads the W tiles —
    // so one warp sees all phases of its stage's barriers in order (a producer dealt arbitrary items could run a
    // full ring ahead of a slower one and mistake an old phase of the one-bit parity for the one it waits for).
    static_assert(2 + N_XPROD == NXS + NYS, "one producer warp per ring stage");
    const int p = warp < 4 ? (warp >> 1) : 2 + warp - (4 + N_EB + N_EC);
    const bool y_prod = p < NYS;
    const int my_stage = y_prod ? p : p - NYS;
    const bool w_prod = p == NYS;
    int it = 0;
    auto land = [&](uint32_t full_bar) {
      cp_async_commit();
      cp_async_wait<0>();
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(full_bar);
    };
    for (int gi = 0; gi < n_my_groups; ++gi) {
      const int g = blockIdx.x + gi * gridDim.x;
      const int ws = gi & 1;
      const int64_t l0 = static_cast<int64_t>(g) * G;
      const int rows_real = static_cast<int>(imin64(G, a.L - l0));
      const int32_t* lrow = a.loc + static_cast<int64_t>(g) * F;
      const int loc_lo = min(max(__ldg(lrow + lane), 0), a.D - 1);
      const int loc_hi = min(max(__ldg(lrow + lane + 32), 0), a.D - 1);
      if (w_prod) {
        mbar_wait(bar(B_WEMPTY + ws), ((gi >> 1) & 1) ^ 1, abort_flag, a.err, 31, WAIT_LIMIT, 100);
        mbar_wait(bar(B_LEMPTY + ws), ((gi >> 1) & 1) ^ 1, abort_flag, a.err, 31, WAIT_LIMIT, 100);
        __syncwarp();
        loc_s[ws * F + lane] = loc_lo;
        loc_s[ws * F + lane + 32] = loc_hi;
        const uint32_t wb = sbase + OFF_W + ws * WSTAGE;
#pragma unroll 4
        for (int i = 0; i < 32; ++i) {
          const int idx = i * 32 + lane, r = idx >> 3, c = idx & 7;
          cp_async16(wb + r * 128 + ((c ^ (r & 7)) << 4), a.w + (l0 + r) * F + c * 8, r < rows_real);
        }
        land(bar(B_WFULL + ws));
      }
      for (int t = 0; t < T; ++t, ++it) {
        const int64_t b0 = static_cast<int64_t>(t) * BT;
        if (!y_prod && it % NXS == my_stage) {            // ---- X item
          const int xs = it % NXS;
          mbar_wait(bar(B_XEMPTY + xs), ((it / NXS) & 1) ^ 1, abort_flag, a.err, 32, WAIT_LIMIT, 100);
          __syncwarp();
          const uint32_t xb = sbase + OFF_X + xs * XSTAGE;
          const int j = lane & 15;
          const bool valid = b0 + j * 8 < a.B;
          const uint32_t dcol = (j >> 3) * XBLK + ((j & 7) << 4);
#pragma unroll 4
          for (int i = 0; i < 32; ++i) {
            const int k = i * 2 + (lane >> 4);
            const int lk = __shfl_sync(0xffffffffu, (i < 16) ? loc_lo : loc_hi, k & 31);
            const __nv_bfloat16* src = a.xt + static_cast<int64_t>(lk) * a.B + b0 + j * 8;
            cp_async16(xb + ((dcol + k * 128) ^ ((k & 7) << 4)), valid ? src : a.xt, valid);
          }
          land(bar(B_XFULL + xs));
        }
        if (y_prod && it % NYS == my_stage) {            // ---- Y item: dy[b0 .. b0+127, l0 .. l0+127] -> two 64-label blocks
          const int ys = it % NYS;
          mbar_wait(bar(B_YEMPTY + ys), ((it / NYS) & 1) ^ 1, abort_flag, a.err, 33, WAIT_LIMIT, 100);
          __syncwarp();
          const uint32_t yb = sbase + OFF_Y + ys * YSTAGE;
          const int c16 = lane & 15;                          // 16-byte chunk (8 labels) inside the 128-label row
          const int64_t col = l0 + c16 * 8;
          const bool cvalid = col + 8 <= a.ldy;             // columns L..ldy-1 of dy are zero by contract; past ldy: zero fill
          const uint32_t dcol = (c16 >> 3) * YBLK + ((c16 & 7) << 4);
#pragma unroll 4
          for (int i = 0; i < 64; ++i) {
            const int r = i * 2 + (lane >> 4);
            const bool valid = cvalid && (b0 + r < a.B);
            const __nv_bfloat16* src = a.dy + (b0 + r) * a.ldy + col;
            cp_async16(yb + ((dcol + r * 128) ^ ((r & 7) << 4)), valid ? src : a.dy, valid);
          }
          land(bar(B_YFULL + ys));
        }
      }
    }
  } else if (warp == 1 || warp == 3) {
    // ================================================================ MMA issuers
    // Each warp runs its control flow converged; one elected lane issues the products and commits (descriptors
    // stay in uniform registers this way).
    {
      constexpr uint32_t ID_BWX = make_idesc(128, F, 0, 1);
      constexpr uint32_t ID_BWW = make_idesc(128, FR, 1, 0);
      const uint64_t D_XB = make_sdesc(sbase + OFF_X, 16, 1024);      // X tile as K-major  B   (backward-weights)
      const uint64_t D_WM = make_sdesc(sbase + OFF_W, WSTAGE, 1024);  // W tile as MN-major B   (backward-features)
      const uint64_t D_YA = make_sdesc(sbase + OFF_Y, 16, 1024);      // Y tile as K-major  A   (backward-features)
      const uint64_t D_YM = make_sdesc(sbase + OFF_Y, YBLK, 1024);    // Y tile as MN-major A   (backward-weights)
      if (warp == 1) {
        const uint32_t wm_lo = static_cast<uint32_t>(D_WM), wm_hi = static_cast<uint32_t>(D_WM >> 32);
        const uint32_t ya_lo = static_cast<uint32_t>(D_YA), ya_hi = static_cast<uint32_t>(D_YA >> 32);
        const uint32_t id_bwx = ID_BWX;
        int it = 0, ys = 0, yph = 0;
        for (int gi = 0; gi < n_my_groups; ++gi) {
          const int ws = gi & 1;
          mbar_wait(bar(B_WFULL + ws), (gi >> 1) & 1, abort_flag, a.err, 34, WAIT_LIMIT);
          for (int t = 0; t < T; ++t, ++it) {
            const int ds = it & 1;
            mbar_wait(bar(B_YFULL + ys), yph, abort_flag, a.err, 35, WAIT_LIMIT);
            mbar_wait(bar(B_DXEMPTY + ds), ((it >> 1) & 1) ^ 1, abort_flag, a.err, 36, WAIT_LIMIT);
            tc_fence_after();
            const uint32_t ya = ya_lo + static_cast<uint32_t>(ys) * (YSTAGE >> 4), wm = wm_lo + (ws ? (WSTAGE >> 4) : 0u);
            const uint32_t tdx = tmem + TM_DX + (ds ? F : 0);
            if (elect_one()) {
              umma_bf16_lohi<false>(tdx, ya, ya_hi, wm, wm_hi, id_bwx);
#pragma unroll
              for (int ks = 1; ks < G / 16; ++ks)
                umma_bf16_lohi<true>(tdx, ya + (((ks >> 2) * YBLK + (ks & 3) * 32) >> 4), ya_hi, wm + ((ks * 2048) >> 4), wm_hi, id_bwx);
              tc_commit(bar(B_DXFULL + ds));
              tc_commit(bar(B_YEMPTY + ys));
              if (t + 1 == T) tc_commit(bar(B_WEMPTY + ws));
            }
            __syncwarp();
            if (++ys == NYS) { ys = 0; yph ^= 1; }
          }
        }
      } else {
        const uint32_t xb_lo = static_cast<uint32_t>(D_XB), xb_hi = static_cast<uint32_t>(D_XB >> 32);
        const uint32_t ym_lo = static_cast<uint32_t>(D_YM), ym_hi = static_cast<uint32_t>(D_YM >> 32);
        const uint32_t id_bww = ID_BWW;
        int it = 0, xs = 0, xph = 0, ys = 0, yph = 0;
        for (int gi = 0; gi < n_my_groups; ++gi) {
          const uint32_t tdw = tmem + TM_DW + ((gi & 1) ? TM_DW_STRIDE : 0u);
          mbar_wait(bar(B_DWEMPTY + (gi & 1)), ((gi >> 1) & 1) ^ 1, abort_flag, a.err, 37, WAIT_LIMIT);
          for (int t = 0; t < T; ++t, ++it) {
            mbar_wait(bar(B_XFULL + xs), xph, abort_flag, a.err, 38, WAIT_LIMIT);
            mbar_wait(bar(B_YFULL + ys), yph, abort_flag, a.err, 39, WAIT_LIMIT);
            tc_fence_after();
            const uint32_t ym = ym_lo + static_cast<uint32_t>(ys) * (YSTAGE >> 4), xb = xb_lo + static_cast<uint32_t>(xs) * (XSTAGE >> 4);
            if (elect_one()) {
              umma_bf16_lohi_rt(tdw, ym, ym_hi, xb, xb_hi, id_bww, t > 0);
#pragma unroll
              for (int ks = 1; ks < BT / 16; ++ks)
                umma_bf16_lohi<true>(tdw, ym + ((ks * 2048) >> 4), ym_hi, xb + (((ks >> 2) * XBLK + (ks & 3) * 32) >> 4), xb_hi, id_bww);
              tc_commit(bar(B_YEMPTY + ys));
              tc_commit(bar(B_XEMPTY + xs));
              if (t + 1 == T) tc_commit(bar(B_DWFULL + (gi & 1)));
            }
            __syncwarp();
            if (++xs == NXS) { xs = 0; xph ^= 1; }
            if (++ys == NYS) { ys = 0; yph ^= 1; }
          }
        }
      }
    }
  } else if (warp >= 4 && warp < 4 + N_EB) {
    // ================================================================ dXg scatter
    const int q = warp & 3, kh = (warp - 4) >> 2;
    const int row = q * 32 + lane;
    int it = 0;
    for (int gi = 0; gi < n_my_groups; ++gi) {
      const int ws = gi & 1;
      mbar_wait(bar(B_WFULL + ws), (gi >> 1) & 1, abort_flag, a.err, 40, WAIT_LIMIT);
      const int4* loc4 = reinterpret_cast<const int4*>(loc_s + ws * F);
      for (int t = 0; t < T; ++t, ++it) {
        const int64_t b0 = static_cast<int64_t>(t) * BT;
        const int ds = it & 1;
        mbar_wait(bar(B_DXFULL + ds), (it >> 1) & 1, abort_flag, a.err, 41, WAIT_LIMIT);
        tc_fence_after();
        uint32_t r0[32];
        tmem_ld32(tmem + (static_cast<uint32_t>(q * 32) << 16) + TM_DX + (ds ? F : 0) + kh * 32, r0);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(B_DXEMPTY + ds));
        if ((b0 + row < a.B) && !*abort_flag) {
          float* dbase = a.dxt + b0 + row;
#pragma unroll
          for (int k4 = 0; k4 < 32; k4 += 4) {
            const int4 lc = loc4[kh * 8 + (k4 >> 2)];
            atomicAdd(dbase + static_cast<int64_t>(lc.x) * a.B, __uint_as_float(r0[k4 + 0]));
            atomicAdd(dbase + static_cast<int64_t>(lc.y) * a.B, __uint_as_float(r0[k4 + 1]));
            atomicAdd(dbase + static_cast<int64_t>(lc.z) * a.B, __uint_as_float(r0[k4 + 2]));
            atomicAdd(dbase + static_cast<int64_t>(lc.w) * a.B, __uint_as_float(r0[k4 + 3]));
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(B_LEMPTY + ws));
    }
  } else if (warp >= 4 + N_EB && warp < 4 + N_EB + N_EC) {
    // ================================================================ dW / dbias rows out of the accumulator
    const int q = warp & 3;
    const int row = q * 32 + lane;                  // label row inside the group == TMEM lane
    for (int gi = 0; gi < n_my_groups; ++gi) {
      const int g = blockIdx.x + gi * gridDim.x;
      const int64_t l0 = static_cast<int64_t>(g) * G;
      const int rows_real = static_cast<int>(imin64(G, a.L - l0));
      mbar_wait(bar(B_DWFULL + (gi & 1)), (gi >> 1) & 1, abort_flag, a.err, 42, WAIT_LIMIT);
      tc_fence_after();
      const uint32_t ta = tmem + (static_cast<uint32_t>(q * 32) << 16) + TM_DW + ((gi & 1) ? TM_DW_STRIDE : 0u);
      uint32_t r0[32], r1[32], rb[8];
      tmem_ld32(ta, r0);
      tmem_ld32(ta + 32, r1);
      tmem_ld8(ta + F, rb);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(B_DWEMPTY + (gi & 1)));
      if (row < rows_real && !*abort_flag) {
        uint4* out = reinterpret_cast<uint4*>(a.dw + (l0 + row) * F);
#pragma unroll
        for (int c = 0; c < 4; ++c)
          out[c] = make_uint4(pack2(__uint_as_float(r0[8 * c]), __uint_as_float(r0[8 * c + 1])), pack2(__uint_as_float(r0[8 * c + 2]), __uint_as_float(r0[8 * c + 3])),
                              pack2(__uint_as_float(r0[8 * c + 4]), __uint_as_float(r0[8 * c + 5])), pack2(__uint_as_float(r0[8 * c + 6]), __uint_as_float(r0[8 * c + 7])));
#pragma unroll
        for (int c = 0; c < 4; ++c)
          out[4 + c] = make_uint4(pack2(__uint_as_float(r1[8 * c]), __uint_as_float(r1[8 * c + 1])), pack2(__uint_as_float(r1[8 * c + 2]), __uint_as_float(r1[8 * c + 3])),
                                  pack2(__uint_as_float(r1[8 * c + 4]), __uint_as_float(r1[8 * c + 5])), pack2(__uint_as_float(r1[8 * c + 6]), __uint_as_float(r1[8 * c + 7])));
        if (a.dbias != nullptr) a.dbias[l0 + row] = __float2bfloat16_rn(__uint_as_float(rb[0]));
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, TM_COLS);
}

}  // namespace b100

bool backward_sm100_supported(const void* dy, const void* dw, int64_t B, int64_t F, int64_t G, int64_t ldy) {
  return G == b100::G && F == b100::F && (B % 8) == 0 && (ldy % 8) == 0 && aligned16(dy) && aligned16(dw);
}

int launch_backward_sm100(const void* xt, const void* w, const int32_t* loc, const void* dy, float* dxt, void* dw, void* dbias, int64_t B,
                          int64_t D, int64_t F, int64_t L, int64_t G, int64_t ldy, cudaStream_t st) {
  using namespace b100;
  if (int rc = report_pending_status("tcgen05 backward")) return rc;
  int* err_dev = nullptr;
  if (int rc = device_status_word(&err_dev)) return rc;
  BwdArgs a;
  a.loc = loc; a.xt = static_cast<const __nv_bfloat16*>(xt); a.w = static_cast<const __nv_bfloat16*>(w);
  a.dy = static_cast<const __nv_bfloat16*>(dy); a.dxt = dxt; a.dw = static_cast<__nv_bfloat16*>(dw);
  a.dbias = static_cast<__nv_bfloat16*>(dbias); a.err = err_dev;
  a.B = B; a.L = L; a.ldy = ldy; a.D = static_cast<int>(D); a.NG = static_cast<int>((L + G - 1) / G);
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = a.NG < sms ? a.NG : sms;
  cudaError_t e = cudaFuncSetAttribute(ffi_backward_sm100_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  if (e != cudaSuccess) return fail(HASTE_ERR_LAUNCH, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  ffi_backward_sm100_kernel<<<grid, NTHREADS, SMEM_BYTES, st>>>(a);
  return check_launch("ffi_backward_sm100_kernel");
}

}  // namespace haste
