// Fused FFI train step on the 5th-generation tensor cores (tcgen05 + TMEM), group size 128, fan-in 64.
//
// One persistent CTA per SM walks label groups g = blockIdx.x, += gridDim.x.  Per group and per 128-row
// batch tile three UMMA products run out of the same three shared-memory tiles (none is ever transposed or
// re-gathered; the 128-byte-swizzled "row block" layout serves both operand majors):
//     X tile [F rows = slots][128 batch]   gathered rows of xt           (+ one row of ones: bias gradient)
//     W tile [G rows = labels][F]          the group's weights
//     Y tile [128 batch][G]                dLoss/dlogit for the tile, written by the epilogue warps
//   forward            Z [b,l]  (TMEM, 128 cols)  = X^T(MN-major A) * W (K-major B),          K = F
//   backward-features  dXg[b,k] (TMEM,  64 cols)  = Y (K-major A)   * W (MN-major B),        K = G
//   backward-weights   dW [l,k] (TMEM, 64+16 cols, accumulated over the batch tiles)
//                                                 = Y^T(MN-major A) * X (K-major B),          K = 128
// Warp roles (512 threads): warp 0 producer (cp.async gather of X tiles through a 4-stage ring, W double
// buffered), warp 1 issues every tcgen05.mma, warps 4-11 turn Z into dY (bias, bf16 rounding, loss gradient,
// target bits) and store it swizzled, warps 12-15 drain dXg (TMEM -> fp32 staging -> bulk reduce-add into
// dxt rows) and at the end of a group apply SGD + weight decay + stochastic rounding to the weights and bias
// straight from the dW accumulator.  Logits, dY and dW never reach global memory.
// All hand-offs are mbarriers with bounded waits; a wait that gives up raises a CTA-wide abort flag, every
// role drains its loops without touching global memory, TMEM is freed and the host sees HASTE_ERR_TIMEOUT.
#include "common.cuh"
#include "launchers.h"
#include "sm100.cuh"

namespace haste {
namespace s100 {
using namespace sm100;

constexpr int G = 128, F = 64, BT = 128;
constexpr int FR = F + 16;                    // rows of an X block: F gathered rows, one row of ones, 15 zero rows
constexpr int NXS = 4;                        // X ring stages
constexpr int XBLK = FR * 128;                // one 64-batch block of an X stage (bytes)
constexpr int XSTAGE = 2 * XBLK;
constexpr int WSTAGE = G * 128;
constexpr int YBLK = BT * 128;
constexpr int YSTAGE = 2 * YBLK;
constexpr int STG = F * BT * 4;
constexpr int OFF_X = 0;
constexpr int OFF_W = OFF_X + NXS * XSTAGE;
constexpr int OFF_Y = OFF_W + 2 * WSTAGE;
constexpr int OFF_STG = OFF_Y + 2 * YSTAGE;
constexpr int OFF_BIAS = OFF_STG + STG;              // float [2][G]
constexpr int OFF_LOC = OFF_BIAS + 2 * G * 4;        // int   [2][F]
constexpr int OFF_YB = OFF_LOC + 2 * F * 4;          // u32   [2][BT][4]  target bits
constexpr int OFF_BAR = OFF_YB + 2 * BT * 4 * 4;     // mbarriers
constexpr int OFF_MISC = OFF_BAR + 32 * 8;           // tmem base address, abort flag
constexpr int SMEM_BYTES = OFF_MISC + 64 + 1024;     // + slack for the 1024-byte alignment of the base
static_assert(SMEM_BYTES <= 232448, "shared memory budget");

// barrier indices
constexpr int B_XFULL = 0, B_XEMPTY = NXS, B_WFULL = 2 * NXS, B_WEMPTY = B_WFULL + 2, B_ZFULL = B_WEMPTY + 2,
              B_ZEMPTY = B_ZFULL + 2, B_YFULL = B_ZEMPTY + 2, B_YEMPTY = B_YFULL + 2, B_DXFULL = B_YEMPTY + 2,
              B_DXEMPTY = B_DXFULL + 2, B_DWFULL = B_DXEMPTY + 2, B_DWEMPTY = B_DWFULL + 1, B_MEMPTY = B_DWEMPTY + 1,
              NBAR = B_MEMPTY + 2;
static_assert(NBAR <= 32, "barrier space");

// TMEM columns
constexpr uint32_t TM_Z = 0, TM_DX = 256, TM_DW = 384, TM_COLS = 512;
constexpr int NTHREADS = 512;
constexpr long long WAIT_LIMIT = 4000000000ll;   // clock cycles (~2 s) before a wait gives up

struct StepArgs {
  const int32_t* loc;
  const __nv_bfloat16* xt;
  const int32_t* tgt_ptr;
  const uint32_t* tgt_ent;
  float* dxt;
  float* loss;
  int* err;
  int64_t B, L;
  int D, NG;
  float grad_scale;
  // optional debug outputs (NULL in production): the bf16 logits and the bf16 gradients the update consumed
  __nv_bfloat16* z_dump;
  int64_t ldz;
  __nv_bfloat16* dw_dump;
  __nv_bfloat16* db_dump;
};

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int LOSS, bool WITH_LOSS, bool HAS_BIAS>
__global__ void __launch_bounds__(NTHREADS, 1) ffi_train_step_sm100_kernel(StepArgs a, UpdateArgs u) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const uint32_t sbase = smem_u32(sm);
  float* bias_s = reinterpret_cast<float*>(sm + OFF_BIAS);
  int* loc_s = reinterpret_cast<int*>(sm + OFF_LOC);
  uint32_t* ybits = reinterpret_cast<uint32_t*>(sm + OFF_YB);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + OFF_MISC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + OFF_MISC + 8);
  auto bar = [&](int i) { return sbase + OFF_BAR + i * 8; };
  constexpr int N_DW = HAS_BIAS ? F + 16 : F;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int T = static_cast<int>((a.B + BT - 1) / BT);

  // ---------------- one-time setup
  if (tid == 0) {
    for (int i = 0; i < NXS; ++i) { mbar_init(bar(B_XFULL + i), 1); mbar_init(bar(B_XEMPTY + i), 1); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(B_WFULL + i), 1);  mbar_init(bar(B_WEMPTY + i), 1);
      mbar_init(bar(B_ZFULL + i), 1);  mbar_init(bar(B_ZEMPTY + i), 8);
      mbar_init(bar(B_YFULL + i), 8);  mbar_init(bar(B_YEMPTY + i), 1);
      mbar_init(bar(B_DXFULL + i), 1); mbar_init(bar(B_DXEMPTY + i), 4);
      mbar_init(bar(B_MEMPTY + i), 12);   // all 12 epilogue warps are done with the group's index/bias rows
    }
    mbar_init(bar(B_DWFULL), 1);
    mbar_init(bar(B_DWEMPTY), 4);
    mbar_fence_init();
    *abort_flag = 0;
  }
  // rows F..FR-1 of every X block: row F = ones (bias gradient column), the rest zeros; written once
  for (int i = tid; i < NXS * 2 * 16 * 8; i += NTHREADS) {
    const int chunk = i & 7, row = (i >> 3) & 15, blk = i >> 7;       // blk in [0, NXS*2)
    const uint32_t v = (row == 0) ? 0x3F803F80u : 0u;
    *reinterpret_cast<uint4*>(sm + OFF_X + blk * XBLK + (F + row) * 128 + chunk * 16) = make_uint4(v, v, v, v);
  }
  fence_proxy_async();
  if (warp == 2) {
    tmem_alloc(smem_u32(tmem_slot), TM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  const int n_my_groups = (a.NG > static_cast<int>(blockIdx.x)) ? (a.NG - 1 - static_cast<int>(blockIdx.x)) / static_cast<int>(gridDim.x) + 1 : 0;

  if (warp == 0) {
    // ================================================================ producer
    uint32_t pend[2] = {0u, 0u};   // full-barriers of the two most recent items, not yet signalled
    int npend = 0;
    auto flush_all = [&]() {
      cp_async_wait<0>();
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) { if (npend > 0) mbar_arrive(pend[0]); if (npend > 1) mbar_arrive(pend[1]); }
      npend = 0;
    };
    auto wait_empty = [&](uint32_t b, uint32_t parity) {
      // never sleep on an empty-slot barrier while earlier items still await their "full" signal
      const bool ready = __all_sync(0xffffffffu, mbar_try_wait(b, parity));     // warp-uniform decision
      if (!ready) { if (npend) flush_all(); mbar_wait(b, parity, abort_flag, a.err, 1, WAIT_LIMIT); __syncwarp(); }
    };
    auto item_done = [&](uint32_t full_bar) {
      cp_async_commit();
      if (npend == 2) {           // the oldest pending item has landed once at most 2 groups are in flight
        cp_async_wait<2>();
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(pend[0]);
        pend[0] = pend[1];
        npend = 1;
      }
      pend[npend++] = full_bar;
    };
    int it = 0;
    for (int gi = 0; gi < n_my_groups; ++gi) {
      const int g = blockIdx.x + gi * gridDim.x;
      const int ws = gi & 1;
      const int64_t l0 = static_cast<int64_t>(g) * G;
      const int rows_real = static_cast<int>(imin64(G, a.L - l0));
      // ---- W item: weights tile, index row, bias row
      wait_empty(bar(B_WEMPTY + ws), ((gi >> 1) & 1) ^ 1);
      wait_empty(bar(B_MEMPTY + ws), ((gi >> 1) & 1) ^ 1);
      {
        const int32_t* lrow = a.loc + static_cast<int64_t>(g) * F;
        loc_s[ws * F + lane] = min(max(__ldg(lrow + lane), 0), a.D - 1);
        loc_s[ws * F + lane + 32] = min(max(__ldg(lrow + lane + 32), 0), a.D - 1);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int c = lane * 4 + i;
          bias_s[ws * G + c] = (HAS_BIAS && c < rows_real) ? __bfloat162float(u.bias[l0 + c]) : 0.f;
        }
        const uint32_t wb = sbase + OFF_W + ws * WSTAGE;
#pragma unroll 4
        for (int i = 0; i < 32; ++i) {
          const int idx = i * 32 + lane, r = idx >> 3, c = idx & 7;
          cp_async16(wb + r * 128 + ((c ^ (r & 7)) << 4), u.w + (l0 + r) * F + c * 8, r < rows_real);
        }
        __syncwarp();
      }
      item_done(bar(B_WFULL + ws));
      // ---- X items: one per batch tile
      for (int t = 0; t < T; ++t, ++it) {
        const int xs = it % NXS;
        wait_empty(bar(B_XEMPTY + xs), ((it / NXS) & 1) ^ 1);
        const int64_t b0 = static_cast<int64_t>(t) * BT;
        const uint32_t xb = sbase + OFF_X + xs * XSTAGE;
        const int j = lane & 15;                     // 16-byte chunk along the batch: 8 rows each
        const bool valid = b0 + j * 8 < a.B;
        const uint32_t dcol = (j >> 3) * XBLK;
#pragma unroll 4
        for (int i = 0; i < 32; ++i) {
          const int k = i * 2 + (lane >> 4);
          const __nv_bfloat16* src = a.xt + static_cast<int64_t>(loc_s[ws * F + k]) * a.B + b0 + j * 8;
          cp_async16(xb + dcol + k * 128 + (((j & 7) ^ (k & 7)) << 4), valid ? src : a.xt, valid);
        }
        item_done(bar(B_XFULL + xs));
      }
    }
    flush_all();
  } else if (warp == 1) {
    // ================================================================ MMA issuer (one thread)
    if (lane == 0) {
      constexpr uint32_t ID_FWD = make_idesc(128, G, 1, 0);
      constexpr uint32_t ID_BWX = make_idesc(128, F, 0, 1);
      constexpr uint32_t ID_BWW = make_idesc(128, N_DW, 1, 0);
      int it = 0;
      auto backward = [&](int j, int t, int ws, int gi) {
        const int ys = j & 1;
        mbar_wait(bar(B_YFULL + ys), (j >> 1) & 1, abort_flag, a.err, 2, WAIT_LIMIT);
        mbar_wait(bar(B_DXEMPTY + ys), ((j >> 1) & 1) ^ 1, abort_flag, a.err, 3, WAIT_LIMIT);
        if (t == 0) mbar_wait(bar(B_DWEMPTY), (gi & 1) ^ 1, abort_flag, a.err, 4, WAIT_LIMIT);
        tc_fence_after();
        const uint32_t yb = sbase + OFF_Y + ys * YSTAGE, wb = sbase + OFF_W + ws * WSTAGE, xb = sbase + OFF_X + (j % NXS) * XSTAGE;
#pragma unroll
        for (int ks = 0; ks < G / 16; ++ks)      // dXg[b,k] += Y[b, l-chunk] * W[l-chunk, k]
          umma_bf16(tmem + TM_DX + ys * F, make_sdesc(yb + (ks >> 2) * YBLK + (ks & 3) * 32, 16, 1024),
                    make_sdesc(wb + ks * 2048, WSTAGE, 1024), ID_BWX, ks > 0);
        tc_commit(bar(B_DXFULL + ys));
#pragma unroll
        for (int ks = 0; ks < BT / 16; ++ks)     // dW[l,k] += Y[b-chunk, l]^T * X[k, b-chunk]
          umma_bf16(tmem + TM_DW, make_sdesc(yb + ks * 2048, YBLK, 1024),
                    make_sdesc(xb + (ks >> 2) * XBLK + (ks & 3) * 32, 16, 1024), ID_BWW, (t > 0) || (ks > 0));
        tc_commit(bar(B_YEMPTY + ys));
        tc_commit(bar(B_XEMPTY + (j % NXS)));
      };
      for (int gi = 0; gi < n_my_groups; ++gi) {
        const int ws = gi & 1;
        mbar_wait(bar(B_WFULL + ws), (gi >> 1) & 1, abort_flag, a.err, 5, WAIT_LIMIT);
        for (int t = 0; t < T; ++t, ++it) {
          const int xs = it % NXS, zs = it & 1;
          mbar_wait(bar(B_XFULL + xs), (it / NXS) & 1, abort_flag, a.err, 6, WAIT_LIMIT);
          mbar_wait(bar(B_ZEMPTY + zs), ((it >> 1) & 1) ^ 1, abort_flag, a.err, 7, WAIT_LIMIT);
          tc_fence_after();
          const uint32_t xb = sbase + OFF_X + xs * XSTAGE, wb = sbase + OFF_W + ws * WSTAGE;
#pragma unroll
          for (int ks = 0; ks < F / 16; ++ks)    // Z[b,l] += X[k-chunk, b]^T * W[l, k-chunk]
            umma_bf16(tmem + TM_Z + zs * G, make_sdesc(xb + ks * 2048, XBLK, 1024), make_sdesc(wb + ks * 32, 16, 1024), ID_FWD, ks > 0);
          tc_commit(bar(B_ZFULL + zs));
          if (t > 0) backward(it - 1, t - 1, ws, gi);
        }
        backward(it - 1, T - 1, ws, gi);
        tc_commit(bar(B_WEMPTY + ws));
        tc_commit(bar(B_DWFULL));
      }
    }
  } else if (warp >= 4 && warp < 12) {
    // ================================================================ epilogue A: Z -> dY
    const int ea = warp - 4, q = ea & 3, h = ea >> 2;
    const int row = q * 32 + lane;               // batch row inside the tile == TMEM lane
    const int et = tid - 128;                    // 0..255
    float loss_acc = 0.f;
    int it = 0;
    for (int gi = 0; gi < n_my_groups; ++gi) {
      const int g = blockIdx.x + gi * gridDim.x;
      const int ws = gi & 1;
      const int rows_real = static_cast<int>(imin64(G, a.L - static_cast<int64_t>(g) * G));
      const int t_beg = __ldg(a.tgt_ptr + g), t_end = __ldg(a.tgt_ptr + g + 1);
      const bool has_t = t_end > t_beg;
      mbar_wait(bar(B_WFULL + ws), (gi >> 1) & 1, abort_flag, a.err, 8, WAIT_LIMIT);   // bias_s of this group is in place
      for (int t = 0; t < T; ++t, ++it) {
        const int zs = it & 1;
        const int64_t b0 = static_cast<int64_t>(t) * BT;
        uint32_t ym[2] = {0u, 0u};
        if (has_t) {
          uint32_t* yb = ybits + (it & 1) * BT * 4;
          yb[et * 2] = 0u; yb[et * 2 + 1] = 0u;
          named_bar_sync(1, 256);
          for (int i = t_beg + et; i < t_end; i += 256) {
            const uint32_t e = __ldg(a.tgt_ent + i);
            const int64_t rb = static_cast<int64_t>(e >> 8) - b0;
            const int c = e & 0xFF;
            if (rb >= 0 && rb < BT && c < G) atomicOr(&yb[rb * 4 + (c >> 5)], 1u << (c & 31));
          }
          named_bar_sync(1, 256);
          ym[0] = yb[row * 4 + h * 2]; ym[1] = yb[row * 4 + h * 2 + 1];
        }
        const bool row_valid = b0 + row < a.B;
        const float gs = row_valid ? a.grad_scale : 0.f;
        mbar_wait(bar(B_ZFULL + zs), (it >> 1) & 1, abort_flag, a.err, 9, WAIT_LIMIT);
        mbar_wait(bar(B_YEMPTY + zs), ((it >> 1) & 1) ^ 1, abort_flag, a.err, 10, WAIT_LIMIT);
        tc_fence_after();
        uint8_t* ytile = sm + OFF_Y + zs * YSTAGE + h * YBLK + row * 128;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t r[32];
          tmem_ld32(tmem + (static_cast<uint32_t>(q * 32) << 16) + TM_Z + zs * G + h * 64 + c * 32, r);
          tmem_ld_wait();
          if (c == 1) {                              // this warp's part of the Z stage is now in registers
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(B_ZEMPTY + zs));
          }
          const int colbase = h * 64 + c * 32;
          const float* bs = bias_s + ws * G + colbase;
          const uint32_t ymask = ym[c];
          const bool ragged = colbase + 32 > rows_real;
#pragma unroll
          for (int e8 = 0; e8 < 32; e8 += 8) {
            uint32_t pk[4];
#pragma unroll
            for (int p = 0; p < 4; ++p) {
              float gq[2];
#pragma unroll
              for (int x = 0; x < 2; ++x) {
                const int e = e8 + 2 * p + x;
                const float zv = round_to_bf16_f(__uint_as_float(r[e]) + bs[e]);
                float la = 0.f;
                float gl = loss_grad<LOSS, WITH_LOSS>(zv, (ymask >> e) & 1u, la);
                if (ragged && colbase + e >= rows_real) { gl = 0.f; la = 0.f; }
                if (WITH_LOSS) loss_acc += row_valid ? la : 0.f;
                gq[x] = gl * gs;
              }
              pk[p] = pack_bf16x2(gq[0], gq[1]);
            }
            if (a.z_dump != nullptr && row_valid) {
#pragma unroll
              for (int e = e8; e < e8 + 8; ++e)
                if (colbase + e < rows_real)
                  a.z_dump[(b0 + row) * a.ldz + static_cast<int64_t>(g) * G + colbase + e] =
                      __float2bfloat16_rn(__uint_as_float(r[e]) + bs[e]);
            }
            const int chunk = (c * 32 + e8) >> 3;    // 16-byte chunk inside the 128-byte row of this block
            *reinterpret_cast<uint4*>(ytile + ((chunk ^ (row & 7)) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
          }
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(B_YFULL + zs));
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(B_MEMPTY + ws));
    }
    if (WITH_LOSS) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) loss_acc += __shfl_xor_sync(0xffffffffu, loss_acc, o);
      if (lane == 0 && !*abort_flag) atomicAdd(a.loss, loss_acc * a.grad_scale);
    }
  } else if (warp >= 12) {
    // ================================================================ epilogue B: dXg scatter, weight update
    const int q = warp & 3;
    const int row = q * 32 + lane;               // TMEM lane: batch row (dXg) or label row (dW)
    const int bt = tid - 384;                    // 0..127
    float* stg = reinterpret_cast<float*>(sm + OFF_STG);
    int it = 0;
    for (int gi = 0; gi < n_my_groups; ++gi) {
      const int g = blockIdx.x + gi * gridDim.x;
      const int ws = gi & 1;
      const int64_t l0 = static_cast<int64_t>(g) * G;
      const int rows_real = static_cast<int>(imin64(G, a.L - l0));
      mbar_wait(bar(B_WFULL + ws), (gi >> 1) & 1, abort_flag, a.err, 11, WAIT_LIMIT);
      const int my_loc = loc_s[ws * F + (bt & (F - 1))];
      for (int t = 0; t < T; ++t, ++it) {
        const int ds = it & 1;
        const int64_t b0 = static_cast<int64_t>(t) * BT;
        mbar_wait(bar(B_DXFULL + ds), (it >> 1) & 1, abort_flag, a.err, 12, WAIT_LIMIT);
        tc_fence_after();
        uint32_t r0[32], r1[32];
        const uint32_t ta = tmem + (static_cast<uint32_t>(q * 32) << 16) + TM_DX + ds * F;
        tmem_ld32(ta, r0);
        tmem_ld32(ta + 32, r1);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(B_DXEMPTY + ds));
        if (bt < F) bulk_wait_read<0>();           // the previous tile's reduce has finished reading the staging tile
        named_bar_sync(2, 128);
#pragma unroll
        for (int k = 0; k < 32; ++k) { stg[k * BT + row] = __uint_as_float(r0[k]); stg[(k + 32) * BT + row] = __uint_as_float(r1[k]); }
        fence_proxy_async();
        named_bar_sync(2, 128);
        if (bt < F && !*abort_flag) {
          const uint32_t nvalid = static_cast<uint32_t>(imin64(BT, a.B - b0));
          bulk_reduce_add_f32(a.dxt + static_cast<int64_t>(my_loc) * a.B + b0, smem_u32(stg + bt * BT), nvalid * 4u);
          bulk_commit();
        }
      }
      // ---- weight / bias update from the dW accumulator
      mbar_wait(bar(B_DWFULL), gi & 1, abort_flag, a.err, 13, WAIT_LIMIT);
      tc_fence_after();
      uint32_t r0[32], r1[32], rb[16];
      const uint32_t ta = tmem + (static_cast<uint32_t>(q * 32) << 16) + TM_DW;
      tmem_ld32(ta, r0);
      tmem_ld32(ta + 32, r1);
      if (HAS_BIAS) tmem_ld16(ta + 64, rb);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(B_DWEMPTY));
      if (row < rows_real && !*abort_flag) {
        const int64_t l = l0 + row, gl = u.label0 + l;
        __nv_bfloat16* wrow = u.w + l * F;
#pragma unroll
        for (int c8 = 0; c8 < F / 8; ++c8) {
          uint4 wv = *reinterpret_cast<const uint4*>(wrow + c8 * 8);
          uint32_t* wp = reinterpret_cast<uint32_t*>(&wv);
          uint4 rp = make_uint4(0, 0, 0, 0);
          const bool sr = u.flags & HASTE_F_SR, packed = u.flags & HASTE_F_RNG_PACKED;
          if (sr && packed) rp = rand_packed8(u.seed, u.step, gl, c8);
#pragma unroll
          for (int x = 0; x < 8; ++x) {
            const int k = c8 * 8 + x;
            const float acc = __uint_as_float(k < 32 ? r0[k & 31] : r1[k & 31]);
            const float gr = round_to_bf16_f(acc);          // the gradient as the unfused kernel would store it
            if (a.dw_dump != nullptr) a.dw_dump[l * F + k] = __float2bfloat16_rn(acc);
            uint32_t r16 = 0;
            if (sr) r16 = packed ? unpack16(rp, x) : rand16_reference(u.seed, gl * F + k);
            const uint16_t wb = (wp[x >> 1] >> (16 * (x & 1))) & 0xFFFFu;
            const uint16_t nb = sgd_update_bits(wb, gr, nullptr, u.lr, u.wd, u.mu, u.flags, r16);
            wp[x >> 1] = (x & 1) ? ((wp[x >> 1] & 0xFFFFu) | (uint32_t(nb) << 16)) : ((wp[x >> 1] & 0xFFFF0000u) | nb);
          }
          *reinterpret_cast<uint4*>(wrow + c8 * 8) = wv;
        }
        if (HAS_BIAS) {
          const float gb = round_to_bf16_f(__uint_as_float(rb[0]));
          if (a.db_dump != nullptr) a.db_dump[l] = __float2bfloat16_rn(__uint_as_float(rb[0]));
          uint32_t r16 = 0;
          if (u.flags & HASTE_F_SR)
            r16 = rand16(u.flags, u.seed ^ ((u.flags & HASTE_F_RNG_PACKED) ? 0x62696173ull : 0ull), u.step, gl, 0, 1);
          u.bias[l] = __ushort_as_bfloat16(sgd_update_bits(__bfloat16_as_ushort(u.bias[l]), gb, nullptr, u.lr, u.wd, u.mu, u.flags, r16));
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(B_MEMPTY + ws));
    }
    if (bt < F) bulk_wait<0>();
  }

  // ---------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 2) tmem_dealloc(tmem, TM_COLS);
}

static int* g_err_host = nullptr;   // pinned, device-mapped: written by a kernel whose wait gave up
static int* g_err_dev = nullptr;

static int ensure_err_flag() {
  if (g_err_host != nullptr) return HASTE_OK;
  cudaError_t e = cudaHostAlloc(reinterpret_cast<void**>(&g_err_host), sizeof(int), cudaHostAllocMapped | cudaHostAllocPortable);
  if (e != cudaSuccess) return fail(HASTE_ERR_LAUNCH, "cudaHostAlloc(error flag): %s", cudaGetErrorString(e));
  *g_err_host = 0;
  e = cudaHostGetDevicePointer(reinterpret_cast<void**>(&g_err_dev), g_err_host, 0);
  if (e != cudaSuccess) return fail(HASTE_ERR_LAUNCH, "cudaHostGetDevicePointer: %s", cudaGetErrorString(e));
  return HASTE_OK;
}

}  // namespace s100

bool train_step_sm100_supported(int64_t B, int64_t F, int64_t G, const UpdateArgs& u) {
  return G == s100::G && F == s100::F && (B % 8) == 0 && u.mom_w == nullptr && u.mom_b == nullptr;
}

int launch_train_step_sm100(const int32_t* loc, const void* xt, const int32_t* tgt_ptr, const uint32_t* tgt_ent, float* dxt, float* loss,
                            const UpdateArgs& u, int64_t B, int64_t D, int64_t F, int64_t L, int64_t G, int loss_kind, float grad_scale,
                            cudaStream_t st, const StepDump* dump) {
  using namespace s100;
  if (int rc = ensure_err_flag()) return rc;
  if (*g_err_host != 0) {
    const int code = *g_err_host;
    *g_err_host = 0;
    return fail(HASTE_ERR_TIMEOUT, "an earlier fused train step gave up waiting on an on-chip barrier (wait id %d); its outputs are invalid", code);
  }
  StepArgs a;
  a.loc = loc; a.xt = static_cast<const __nv_bfloat16*>(xt); a.tgt_ptr = tgt_ptr; a.tgt_ent = tgt_ent; a.dxt = dxt; a.loss = loss;
  a.err = g_err_dev; a.B = B; a.L = L; a.D = static_cast<int>(D); a.NG = static_cast<int>((L + G - 1) / G); a.grad_scale = grad_scale;
  a.z_dump = dump ? static_cast<__nv_bfloat16*>(dump->z) : nullptr; a.ldz = dump ? dump->ldz : 0;
  a.dw_dump = dump ? static_cast<__nv_bfloat16*>(dump->dw) : nullptr; a.db_dump = dump ? static_cast<__nv_bfloat16*>(dump->dbias) : nullptr;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = a.NG < sms ? a.NG : sms;
  const bool wl = (u.flags & HASTE_F_LOSS) && loss != nullptr;
  const bool hb = u.bias != nullptr;
#define HASTE_S100_LAUNCH(LK, WL, HB)                                                                              \
  {                                                                                                                \
    auto k = ffi_train_step_sm100_kernel<LK, WL, HB>;                                                              \
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);               \
    if (e != cudaSuccess) return fail(HASTE_ERR_LAUNCH, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));         \
    k<<<grid, NTHREADS, SMEM_BYTES, st>>>(a, u);                                                                    \
  }
  if (loss_kind == HASTE_LOSS_BCE) {
    if (wl) { if (hb) HASTE_S100_LAUNCH(HASTE_LOSS_BCE, true, true) else HASTE_S100_LAUNCH(HASTE_LOSS_BCE, true, false) }
    else    { if (hb) HASTE_S100_LAUNCH(HASTE_LOSS_BCE, false, true) else HASTE_S100_LAUNCH(HASTE_LOSS_BCE, false, false) }
  } else {
    if (wl) { if (hb) HASTE_S100_LAUNCH(HASTE_LOSS_SQHINGE, true, true) else HASTE_S100_LAUNCH(HASTE_LOSS_SQHINGE, true, false) }
    else    { if (hb) HASTE_S100_LAUNCH(HASTE_LOSS_SQHINGE, false, true) else HASTE_S100_LAUNCH(HASTE_LOSS_SQHINGE, false, false) }
  }
#undef HASTE_S100_LAUNCH
  return check_launch("ffi_train_step_sm100_kernel");
}

}  // namespace haste
