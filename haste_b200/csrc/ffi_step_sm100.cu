// Fused FFI train step on the 5th-generation tensor cores (tcgen05 + TMEM), group size 128, fan-in 64.
//
// One persistent CTA per SM walks label groups g = blockIdx.x, += gridDim.x (the incomplete last round goes to the
// highest-numbered CTAs).  Per group and per 128-row
// batch tile three UMMA products run out of the same three shared-memory tiles (none is ever transposed or
// re-gathered; the 128-byte-swizzled "row block" layout serves both operand majors):
//     X tile [F rows = slots][128 batch]   gathered rows of xt           (+ one row of ones: bias gradient)
//     W tile [G rows = labels][F]          the group's weights
//     Y tile [128 batch][G]                dLoss/dlogit for the tile, written by the epilogue warps
//   forward            Z [b,l]  (TMEM, 128 cols)  = X^T(MN-major A) * W (K-major B),          K = F
//   backward-features  dXg[b,k] (TMEM,  64 cols)  = Y (K-major A)   * W (MN-major B),        K = G
//   backward-weights   dW [l,k] (TMEM, 64+16 cols, accumulated over the batch tiles)
//                                                 = Y^T(MN-major A) * X (K-major B),          K = 128
// Warp roles (512 threads): warps 0,2,3 producers (cp.async gather of X tiles through a 6-stage ring, W double
// buffered; load items are dealt round-robin so three are in flight), warp 1 issues every tcgen05.mma,
// warps 4-11 turn Z into dY (bias, bf16 rounding, loss gradient, target bits) and store it swizzled,
// warps 12-15 drain dXg (TMEM -> registers -> coalesced red.global.add into dxt rows) and at the end of a
// group apply SGD + weight decay + stochastic rounding to the weights and bias straight from the dW
// accumulator.  Logits, dY and dW never reach global memory.
// All hand-offs are mbarriers with bounded waits; a wait that gives up raises a CTA-wide abort flag, every
// role drains its loops without touching global memory, TMEM is freed and the host sees HASTE_ERR_TIMEOUT.
#include "common.cuh"
#include "launchers.h"
#include "sm100.cuh"
#include <stdlib.h>

namespace haste {
namespace s100 {
// out-of-line Philox for the reference random stream: that path is slow anyway and must not bloat the epilogue code
__device__ __noinline__ static uint32_t rand16_reference_call(uint64_t seed, int64_t flat) { return rand16_reference(seed, flat); }
// likewise one shared copy of the packed-stream generator and of the bias draw for the update warps
__device__ __noinline__ static uint4 rand_packed8_call(uint64_t seed, uint32_t step, int64_t row, int col8) { return rand_packed8(seed, step, row, col8); }
__device__ __noinline__ static uint32_t rand16_call(uint32_t flags, uint64_t seed, uint32_t step, int64_t row) { return rand16(flags, seed, step, row, 0, 1); }

using namespace sm100;

constexpr int G = 128, F = 64, BT = 128;
constexpr int FR = F + 16;                    // rows of an X block: F gathered rows, one row of ones, 15 zero rows
constexpr int NXS = 6;                        // X ring stages
constexpr int NYS = 2;                        // dY ring stages
constexpr int XBLK = FR * 128;                // one 64-batch block of an X stage (bytes)
constexpr int XSTAGE = 2 * XBLK;
constexpr int WSTAGE = G * 128;
constexpr int YBLK = BT * 128;
constexpr int YSTAGE = 2 * YBLK;
constexpr int OFF_X = 0;
constexpr int OFF_W = OFF_X + NXS * XSTAGE;
constexpr int OFF_Y = OFF_W + 2 * WSTAGE;
constexpr int OFF_BIAS = OFF_Y + NYS * YSTAGE;         // float [2][G]
constexpr int OFF_LOC = OFF_BIAS + 2 * G * 4;        // int   [2][F]
constexpr int OFF_YB = OFF_LOC + 2 * F * 4;          // u32   [2][BT][4]  target bits
constexpr int OFF_BAR = OFF_YB + 2 * BT * 4 * 4;     // mbarriers
constexpr int OFF_MISC = OFF_BAR + 32 * 8;           // tmem base address, abort flag
constexpr int SMEM_BYTES = OFF_MISC + 64 + 1024;     // + slack for the 1024-byte alignment of the base
static_assert(SMEM_BYTES <= 232448, "shared memory budget");

// barrier indices
constexpr int B_XFULL = 0, B_XEMPTY = NXS, B_WFULL = 2 * NXS, B_WEMPTY = B_WFULL + 2, B_ZFULL = B_WEMPTY + 2,
              B_ZEMPTY = B_ZFULL + 2, B_YFULL = B_ZEMPTY + 2, B_YEMPTY = B_YFULL + NYS, B_DXFULL = B_YEMPTY + NYS,
              B_DXEMPTY = B_DXFULL + 2, B_DWFULL = B_DXEMPTY + 2, B_DWEMPTY = B_DWFULL + 1, B_MEMPTY = B_DWEMPTY + 1,
              NBAR = B_MEMPTY + 2;
static_assert(NBAR <= 32, "barrier space");

// TMEM columns
// Z double-buffered (2 x 128), dXg double-buffered (2 x 64), dW single (64 + 16)
constexpr uint32_t TM_Z = 0, TM_DX = 256, TM_DW = 384, TM_COLS = 512;
constexpr int N_EB = 8;                          // epilogue-B warps: 4 TMEM lane quarters x 2 slot halves
constexpr int N_EA_SET = 8;                      // epilogue-A warps working on one tile: 4 TMEM lane quarters x 2 column halves
constexpr int N_SETS = 1;                        // sets of epilogue-A warps; set s takes the tiles whose Z stage is s
constexpr int N_EA = N_EA_SET * N_SETS;
constexpr int BX_LAG = N_SETS;                   // backward-features runs this many tiles behind the forward product
constexpr int N_UP = 8;                          // update warps: 4 TMEM lane quarters x 2 slot halves
constexpr int NTHREADS = (4 + N_EA + N_EB + N_UP) * 32;   // 4 control warps + epilogue-A + epilogue-B + update warps
static_assert(NTHREADS <= 1024, "thread budget");
constexpr int EA_COLS = G * 4 / N_EA_SET;        // label columns of a tile handled by one epilogue-A warp (32 or 64)
constexpr int UP_SLOTS = F * 4 / N_UP;           // slots updated by one update warp
static_assert((N_EA_SET == 8 || N_EA_SET == 16) && (N_SETS == 1 || N_SETS == 2), "epilogue A: 8 or 16 warps per tile, one or two sets");
constexpr long long WAIT_LIMIT = 4000000000ll;   // clock cycles (~2 s) before a wait gives up

#ifdef HASTE_TRACE
// development build only: per-role event timeline of CTA 0
__device__ unsigned long long g_trace[7][2048];     // (clock << 16) | event, zero = unused
#define TR(role, ev)                                                        \
  do {                                                                      \
    if (blockIdx.x == 0 && tr_n < 2048) { g_trace[role][tr_n++] = (static_cast<unsigned long long>(clock64()) << 16) | static_cast<unsigned>(ev); } \
  } while (0)
#else
#define TR(role, ev) do {} while (0)
#endif

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

// Two fp32 -> one bf16x2 word with max(0, .) applied to both halves (one conversion instruction).
__device__ __forceinline__ uint32_t pack_bf16x2_relu(float lo, float hi) {
  uint32_t d;
  asm("cvt.rn.relu.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}
// v rounded to bf16 (nearest even), returned as fp32: converting (v, 0) to a bf16x2 word puts bf16(v) in the
// upper half over a zero lower half, which is the fp32 image of the rounded value — no unpacking needed.
__device__ __forceinline__ float round_bf16_as_f32(float v) {
  uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(v), "f"(0.f));
  return __uint_as_float(d);
}

template <int LOSS, bool WITH_LOSS, bool HAS_BIAS, bool DEBUG>
__global__ void __launch_bounds__(NTHREADS, 1) ffi_train_step_sm100_kernel(StepArgs a, UpdateArgs u) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const uint32_t sbase = smem_u32(sm);
  float* bias_s = reinterpret_cast<float*>(sm + OFF_BIAS);
  uint32_t* loc_s = reinterpret_cast<uint32_t*>(sm + OFF_LOC);   // per slot: element offset loc * B of its dxt row
  uint32_t* ybits = reinterpret_cast<uint32_t*>(sm + OFF_YB);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + OFF_MISC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + OFF_MISC + 8);
  auto bar = [&](int i) { return sbase + OFF_BAR + i * 8; };
  constexpr int N_DW = HAS_BIAS ? F + 16 : F;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int T = static_cast<int>((a.B + BT - 1) / BT);
  // CTAs walk the batch tiles in rotated order so that, at any moment, the dX reductions of different SMs
  // are spread over the whole dxt array instead of all landing in the same 128 batch columns
  const int rot = static_cast<int>(blockIdx.x % static_cast<unsigned>(T));
  auto tile_b0 = [&](int t) { int tt = t + rot; if (tt >= T) tt -= T; return static_cast<int64_t>(tt) * BT; };

  // ---------------- one-time setup
  if (tid == 0) {
    for (int i = 0; i < NXS; ++i) { mbar_init(bar(B_XFULL + i), 1); mbar_init(bar(B_XEMPTY + i), 1); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(B_WFULL + i), 1);  mbar_init(bar(B_WEMPTY + i), 1);
      mbar_init(bar(B_ZFULL + i), 1);  mbar_init(bar(B_ZEMPTY + i), N_EA_SET);
      mbar_init(bar(B_DXFULL + i), 1); mbar_init(bar(B_DXEMPTY + i), N_EB);
      mbar_init(bar(B_MEMPTY + i), N_EA + N_EB + N_UP);   // every epilogue warp is done with the group's index/bias rows and W tile
    }
    for (int i = 0; i < NYS; ++i) { mbar_init(bar(B_YFULL + i), N_EA_SET); mbar_init(bar(B_YEMPTY + i), 2); }   // both backward issuers commit
    mbar_init(bar(B_DWFULL), 1);
    mbar_init(bar(B_DWEMPTY), N_UP);
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
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), TM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  int tr_n = 0;   // trace cursor of this thread (development builds)
  (void)tr_n;
  // Groups are dealt round-robin; the incomplete last round goes to the highest-numbered CTAs.  The head of a
  // long-tailed label distribution sits in the first groups, whose tiles are the expensive ones (positives, target
  // bitmap): the CTAs that own them then have one group less to do.
  const int n_cta = static_cast<int>(gridDim.x), cta = static_cast<int>(blockIdx.x);
  const int full_rounds = a.NG / n_cta, rem_groups = a.NG - full_rounds * n_cta;
  const int n_my_groups = full_rounds + (cta >= n_cta - rem_groups ? 1 : 0);
  auto group_of = [&](int gi) { return gi < full_rounds ? cta + gi * n_cta : full_rounds * n_cta + (cta - (n_cta - rem_groups)); };

  if (warp == 0 || warp == 2) {
    // ================================================================ producers
    // The sequence of load items (per group: the W item, then one X item per batch tile) is dealt round-robin to
    // the two producer warps; each handles one item at a time: wait for the slot, issue the copies, wait for
    // them to land, make them visible to the tensor core's proxy, signal "full".
    const int p = warp >> 1;
    int item = 0, it = 0;
    auto land = [&](uint32_t full_bar) {
      cp_async_commit();
      cp_async_wait<0>();
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(full_bar);
    };
    for (int gi = 0; gi < n_my_groups; ++gi) {
      const int g = group_of(gi);
      const int ws = gi & 1;
      const int64_t l0 = static_cast<int64_t>(g) * G;
      const int rows_real = static_cast<int>(imin64(G, a.L - l0));
      const int32_t* lrow = a.loc + static_cast<int64_t>(g) * F;
      const int loc_lo = min(max(__ldg(lrow + lane), 0), a.D - 1);        // clamped: never addresses outside xt / dxt
      const int loc_hi = min(max(__ldg(lrow + lane + 32), 0), a.D - 1);
      if ((item & 1) == p) {
        // ---- W item: weights tile, index row, bias row
        mbar_wait(bar(B_WEMPTY + ws), ((gi >> 1) & 1) ^ 1, abort_flag, a.err, 1, WAIT_LIMIT, 100);
        mbar_wait(bar(B_MEMPTY + ws), ((gi >> 1) & 1) ^ 1, abort_flag, a.err, 1, WAIT_LIMIT, 100);
        __syncwarp();
        loc_s[ws * F + lane] = static_cast<uint32_t>(loc_lo) * static_cast<uint32_t>(a.B);        // D * B < 2^32 is a launch condition
        loc_s[ws * F + lane + 32] = static_cast<uint32_t>(loc_hi) * static_cast<uint32_t>(a.B);
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
        if (lane == 0) TR(p * 4, 100 + gi);
        land(bar(B_WFULL + ws));
        if (lane == 0) TR(p * 4, 500 + gi);
      }
      ++item;
      // ---- X items: one per batch tile
      for (int t = 0; t < T; ++t, ++it, ++item) {
        if ((item & 1) != p) continue;
        const int xs = it % NXS;
        mbar_wait(bar(B_XEMPTY + xs), ((it / NXS) & 1) ^ 1, abort_flag, a.err, 1, WAIT_LIMIT, 100);
        __syncwarp();
        const int64_t b0 = tile_b0(t);
        const uint32_t xb = sbase + OFF_X + xs * XSTAGE;
        const int j = lane & 15;                     // 16-byte chunk along the batch: 8 rows each
        const bool valid = b0 + j * 8 < a.B;
        const uint32_t dcol = (j >> 3) * XBLK + ((j & 7) << 4);
#pragma unroll 4
        for (int i = 0; i < 32; ++i) {
          const int k = i * 2 + (lane >> 4);
          const int lk = __shfl_sync(0xffffffffu, (i < 16) ? loc_lo : loc_hi, k & 31);
          const __nv_bfloat16* src = a.xt + static_cast<int64_t>(lk) * a.B + b0 + j * 8;
          cp_async16(xb + ((dcol + k * 128) ^ ((k & 7) << 4)), valid ? src : a.xt, valid);
        }
        if (lane == 0) TR(p * 4, 1000 + it);
        land(bar(B_XFULL + xs));
        if (lane == 0) TR(p * 4, 5000 + it);
      }
    }
  } else if (warp == 1 || warp == 3) {
    // ================================================================ MMA issuers (one thread each)
    // Feeding the tensor pipe from a single thread costs more cycles per tcgen05.mma than the small (N = 64..128)
    // products take to execute, so the work is split: warp 1 issues forward + backward-features, warp 3 issues
    // backward-weights.  Both hang off the same mbarriers; the pipe executes in arrival order.
    {
      constexpr uint32_t ID_FWD = make_idesc(128, G, 1, 0);
      constexpr uint32_t ID_BWX = make_idesc(128, F, 0, 1);
      constexpr uint32_t ID_BWW = make_idesc(128, N_DW, 1, 0);
      // Descriptors are built once.  Per MMA only the start-address field (low word, 16-byte units) moves, by
      // compile-time constants; it never carries out of its 14-bit field because every operand lies inside the
      // CTA's shared memory window.
      const uint64_t D_XA = make_sdesc(sbase + OFF_X, XBLK, 1024);    // X tile as MN-major A   (forward)
      const uint64_t D_XB = make_sdesc(sbase + OFF_X, 16, 1024);      // X tile as K-major  B   (backward-weights)
      const uint64_t D_WB = make_sdesc(sbase + OFF_W, 16, 1024);      // W tile as K-major  B   (forward)
      const uint64_t D_WM = make_sdesc(sbase + OFF_W, WSTAGE, 1024);  // W tile as MN-major B   (backward-features)
      const uint64_t D_YA = make_sdesc(sbase + OFF_Y, 16, 1024);      // Y tile as K-major  A   (backward-features)
      const uint64_t D_YM = make_sdesc(sbase + OFF_Y, YBLK, 1024);    // Y tile as MN-major A   (backward-weights)
      if (warp == 1) {
        // ---------------- forward + backward-features
        const uint32_t xa_lo = static_cast<uint32_t>(D_XA), xa_hi = static_cast<uint32_t>(D_XA >> 32);
        const uint32_t wb_lo = static_cast<uint32_t>(D_WB), wb_hi = static_cast<uint32_t>(D_WB >> 32);
        const uint32_t wm_lo = static_cast<uint32_t>(D_WM), wm_hi = static_cast<uint32_t>(D_WM >> 32);
        const uint32_t ya_lo = static_cast<uint32_t>(D_YA), ya_hi = static_cast<uint32_t>(D_YA >> 32);
        const uint32_t id_fwd = ID_FWD, id_bwx = ID_BWX;
        // Order of issue: forward(it) first, then backward-features of tile it - BX_LAG.  Both become possible at
        // the same moment (epilogue A finished a tile); the forward product goes first because an epilogue-A
        // set is waiting for it, while nothing waits for the backward product's dY stage (three stages).
        int it = 0, xs = 0, xph = 0;
        int j = 0, jy = 0, jyph = 0, j_t = 0, j_g = 0;     // next backward-features tile: dY stage and phase, position in its group
        auto backward_x = [&]() {
          const int ds = j & 1, ws = j_g & 1;
          mbar_wait(bar(B_YFULL + jy), jyph, abort_flag, a.err, 2, WAIT_LIMIT);
          mbar_wait(bar(B_DXEMPTY + ds), ((j >> 1) & 1) ^ 1, abort_flag, a.err, 3, WAIT_LIMIT);
          tc_fence_after();
          if (lane == 0) TR(1, 2000 + j);
          const uint32_t ya = ya_lo + static_cast<uint32_t>(jy) * (YSTAGE >> 4), wm = wm_lo + (ws ? (WSTAGE >> 4) : 0u);
          const uint32_t tdx = tmem + TM_DX + (ds ? F : 0);
          // dXg[b,k] = sum over label chunks of Y[b, l-chunk] * W[l-chunk, k]
          const bool last_of_group = j_t + 1 == T;
          if (elect_one()) {
            umma_bf16_lohi<false>(tdx, ya, ya_hi, wm, wm_hi, id_bwx);
#pragma unroll
            for (int ks = 1; ks < G / 16; ++ks)
              umma_bf16_lohi<true>(tdx, ya + (((ks >> 2) * YBLK + (ks & 3) * 32) >> 4), ya_hi, wm + ((ks * 2048) >> 4), wm_hi, id_bwx);
            tc_commit(bar(B_DXFULL + ds));
            tc_commit(bar(B_YEMPTY + jy));
            if (last_of_group) tc_commit(bar(B_WEMPTY + ws));   // every product that reads this group's W tile has been issued
          }
          __syncwarp();
          if (lane == 0) TR(1, 3000 + j);
          if (++jy == NYS) { jy = 0; jyph ^= 1; }
          ++j;
          if (++j_t == T) { j_t = 0; ++j_g; }
        };
        for (int gi = 0; gi < n_my_groups; ++gi) {
          const int ws = gi & 1;
          // the W stage of this group was last used by group gi - 2: its products must all be issued before the
          // stage can be refilled (matters only when a group has fewer tiles than the lag)
          while (j < it && j_g + 2 <= gi) backward_x();
          mbar_wait(bar(B_WFULL + ws), (gi >> 1) & 1, abort_flag, a.err, 5, WAIT_LIMIT);
          for (int t = 0; t < T; ++t, ++it) {
            const int zs = it & 1;
            mbar_wait(bar(B_XFULL + xs), xph, abort_flag, a.err, 6, WAIT_LIMIT);
            mbar_wait(bar(B_ZEMPTY + zs), ((it >> 1) & 1) ^ 1, abort_flag, a.err, 7, WAIT_LIMIT);
            tc_fence_after();
            if (lane == 0) TR(1, 1000 + it);
            const uint32_t xa = xa_lo + static_cast<uint32_t>(xs) * (XSTAGE >> 4), wb = wb_lo + (ws ? (WSTAGE >> 4) : 0u);
            const uint32_t tz = tmem + TM_Z + (zs ? G : 0);
            // Z[b,l] = sum over slot chunks of X[k-chunk, b]^T * W[l, k-chunk]
            if (elect_one()) {
              umma_bf16_lohi<false>(tz, xa, xa_hi, wb, wb_hi, id_fwd);
#pragma unroll
              for (int ks = 1; ks < F / 16; ++ks)
                umma_bf16_lohi<true>(tz, xa + ((ks * 2048) >> 4), xa_hi, wb + ((ks * 32) >> 4), wb_hi, id_fwd);
              tc_commit(bar(B_ZFULL + zs));
            }
            __syncwarp();
            if (++xs == NXS) { xs = 0; xph ^= 1; }
            if (it >= BX_LAG) backward_x();
          }
        }
        while (j < it) backward_x();
      } else {
        // ---------------- backward-weights
        const uint32_t xb_lo = static_cast<uint32_t>(D_XB), xb_hi = static_cast<uint32_t>(D_XB >> 32);
        const uint32_t ym_lo = static_cast<uint32_t>(D_YM), ym_hi = static_cast<uint32_t>(D_YM >> 32);
        const uint32_t id_bww = ID_BWW;
        int j = 0, xs = 0, jy = 0, jyph = 0;
        for (int gi = 0; gi < n_my_groups; ++gi) {
          const uint32_t tdw = tmem + TM_DW;
          mbar_wait(bar(B_DWEMPTY), (gi & 1) ^ 1, abort_flag, a.err, 4, WAIT_LIMIT);
          for (int t = 0; t < T; ++t, ++j) {
            // Y(t) complete implies forward(t) complete, so the tile's X slot is loaded as well
            mbar_wait(bar(B_YFULL + jy), jyph, abort_flag, a.err, 14, WAIT_LIMIT);
            tc_fence_after();
            if (lane == 0) TR(5, 1000 + j);
            const uint32_t ym = ym_lo + static_cast<uint32_t>(jy) * (YSTAGE >> 4), xb = xb_lo + static_cast<uint32_t>(xs) * (XSTAGE >> 4);
            // dW[l,k] += sum over batch chunks of Y[b-chunk, l]^T * X[k, b-chunk]
            if (elect_one()) {
              umma_bf16_lohi_rt(tdw, ym, ym_hi, xb, xb_hi, id_bww, t > 0);
#pragma unroll
              for (int ks = 1; ks < BT / 16; ++ks)
                umma_bf16_lohi<true>(tdw, ym + ((ks * 2048) >> 4), ym_hi, xb + (((ks >> 2) * XBLK + (ks & 3) * 32) >> 4), xb_hi, id_bww);
              tc_commit(bar(B_YEMPTY + jy));
              tc_commit(bar(B_XEMPTY + xs));
              if (t + 1 == T) tc_commit(bar(B_DWFULL));
            }
            __syncwarp();
            if (++jy == NYS) { jy = 0; jyph ^= 1; }
            if (lane == 0) TR(5, 2000 + j);
            if (++xs == NXS) xs = 0;
          }
        }
      }
    }
  } else if (warp >= 4 && warp < 4 + N_EA) {
    // ================================================================ epilogue A: Z -> dY
    // With two sets, a set works on every other tile: the waits, fences and TMEM latencies of one set's tile are
    // covered by the other set's arithmetic.
    const int ea = warp - 4, set = ea / N_EA_SET, es = ea % N_EA_SET;
    const int q = es & 3, h = es >> 2;           // TMEM lane quarter, column range (EA_COLS labels each)
    const int row = q * 32 + lane;               // batch row inside the tile == TMEM lane
    const int et = tid - 128 - set * N_EA_SET * 32;   // thread index inside the set
    float loss_acc = 0.f;
    const float inv_4gs2_sq = 0.0625f / (a.grad_scale * a.grad_scale);   // undoes the (4 s)^2 carried by the fast loss sum
    int it = 0, ys = 0, yph = 0;                 // global tile counter, its dY stage and phase
    auto next_tile = [&]() { ++it; if (++ys == NYS) { ys = 0; yph ^= 1; } };
    for (int gi = 0; gi < n_my_groups; ++gi) {
      const int g = group_of(gi);
      const int ws = gi & 1;
      const int rows_real = static_cast<int>(imin64(G, a.L - static_cast<int64_t>(g) * G));
      const int t_beg = __ldg(a.tgt_ptr + g), t_end = __ldg(a.tgt_ptr + g + 1);
      const bool has_t = t_end > t_beg;
      mbar_wait(bar(B_WFULL + ws), (gi >> 1) & 1, abort_flag, a.err, 8, WAIT_LIMIT);   // bias_s of this group is in place
      for (int t = 0; t < T; ++t, next_tile()) {
        if (N_SETS > 1 && (it & 1) != set) continue;     // the other set's tile
        const int zs = it & 1;
        const int64_t b0 = tile_b0(t);
        uint64_t ym = 0ull;                              // target bits of this thread's row, EA_COLS label columns
        if (has_t && t_end - t_beg <= 8) {
          // Few targets in this group (the common case): each thread picks the bits of its own row and 32 label
          // columns straight from the entry list — no shared bitmap, no barrier between the epilogue warps.
          const uint32_t rowkey = static_cast<uint32_t>(b0 + row);
          for (int i = t_beg; i < t_end; ++i) {
            const uint32_t e = __ldg(a.tgt_ent + i);
            const uint32_t c = (e & 0xFFu) - static_cast<uint32_t>(h * EA_COLS);
            if ((e >> 8) == rowkey && c < static_cast<uint32_t>(EA_COLS)) ym |= 1ull << c;
          }
        } else if (has_t) {
          uint32_t* yb = ybits + (it & 1) * BT * 4;
          for (int i = et; i < BT * 4; i += N_EA_SET * 32) yb[i] = 0u;
          named_bar_sync(1 + set, N_EA_SET * 32);
          // head groups of a long-tailed label distribution hold thousands of entries: eight independent loads in
          // flight per thread, so that the scan runs at L2 throughput rather than one L2 latency per entry
          for (int i0 = t_beg + et; i0 < t_end; i0 += 8 * N_EA_SET * 32) {
            uint32_t e8[8];
#pragma unroll
            for (int x = 0; x < 8; ++x) {
              const int i = i0 + x * N_EA_SET * 32;
              e8[x] = i < t_end ? __ldg(a.tgt_ent + i) : 0xFFFFFFFFu;       // row 2^24 - 1: outside every tile
            }
#pragma unroll
            for (int x = 0; x < 8; ++x) {
              const int64_t rb = static_cast<int64_t>(e8[x] >> 8) - b0;
              const int c = e8[x] & 0xFF;
              if (rb >= 0 && rb < BT && c < G) atomicOr(&yb[rb * 4 + (c >> 5)], 1u << (c & 31));
            }
          }
          named_bar_sync(1 + set, N_EA_SET * 32);
          if (EA_COLS == 32) ym = yb[row * 4 + h];
          else ym = static_cast<uint64_t>(yb[row * 4 + h * 2]) | (static_cast<uint64_t>(yb[row * 4 + h * 2 + 1]) << 32);
        }
        const bool row_valid = b0 + row < a.B;
        const float gs = row_valid ? a.grad_scale : 0.f;
        mbar_wait(bar(B_ZFULL + zs), (it >> 1) & 1, abort_flag, a.err, 9, WAIT_LIMIT);
        if (es == 0 && lane == 0) TR(2 + 4 * set, 1000 + it);
        mbar_wait(bar(B_YEMPTY + ys), yph ^ 1, abort_flag, a.err, 10, WAIT_LIMIT);
        tc_fence_after();
        if (es == 0 && lane == 0) TR(2 + 4 * set, 2000 + it);
        const int col0 = h * EA_COLS;                              // first label column of this warp
        uint8_t* ytile = sm + OFF_Y + ys * YSTAGE + (col0 >> 6) * YBLK + row * 128;
        const uint32_t ta = tmem + (static_cast<uint32_t>(q * 32) << 16) + TM_Z + zs * G + col0;
        const float4* bs4 = reinterpret_cast<const float4*>(bias_s + ws * G + col0);
        const float gs2 = 2.f * gs;
        const float inv_gs2_sq = row_valid ? inv_4gs2_sq : 0.f;
        const bool ragged = col0 + EA_COLS > rows_real;     // only the last group of the layer can be ragged
        float tile_loss = 0.f, fast_loss = 0.f;        // fast_loss: hinge (4s)^2-scaled squares, or BCE raw log2 terms
        const float hgs = 0.5f * gs;
        // 16 label columns per iteration.  Nearly every chunk has no positive label in the warp's 32 rows and no
        // ragged edge: one warp vote per chunk sends those down a branch with no per-element tests (which would cost
        // about a quarter of the epilogue's instructions); the rest take the general branch with target bits and a
        // column-valid mask.
#pragma unroll 1
        for (int c16 = 0; c16 < EA_COLS; c16 += 16) {
          uint32_t r[16];
          __syncwarp();
          if (es == 0 && lane == 0) TR(2 + 4 * set, 7000 + c16);
          tmem_ld16(ta + c16, r);
          tmem_ld_wait();
          if (es == 0 && lane == 0) TR(2 + 4 * set, 8000 + c16);
          const uint32_t ym16 = static_cast<uint32_t>(ym >> c16) & 0xFFFFu;
          const bool general = DEBUG || ragged || __any_sync(0xffffffffu, ym16 != 0u);
          if (!general) {
#pragma unroll
            for (int e8 = 0; e8 < 16; e8 += 8) {
              const float4 ba = bs4[(c16 + e8) >> 2], bb = bs4[((c16 + e8) >> 2) + 1];
              float z[8];
              z[0] = __uint_as_float(r[e8 + 0]) + ba.x; z[1] = __uint_as_float(r[e8 + 1]) + ba.y;
              z[2] = __uint_as_float(r[e8 + 2]) + ba.z; z[3] = __uint_as_float(r[e8 + 3]) + ba.w;
              z[4] = __uint_as_float(r[e8 + 4]) + bb.x; z[5] = __uint_as_float(r[e8 + 5]) + bb.y;
              z[6] = __uint_as_float(r[e8 + 6]) + bb.z; z[7] = __uint_as_float(r[e8 + 7]) + bb.w;
              uint4 pk;
              if (LOSS == HASTE_LOSS_SQHINGE) {
                // dLoss/dz = 2 s max(0, 1 + z) with s = grad_scale, evaluated as max(0, fma(2s, z, 2s)); 1 + z is
                // exact in fp32 for a bf16 z (down to |z| ~ 2^-16), so this is the same single rounding as
                // (1 + z) * 2s.  The max is left to the bf16 conversion.  The loss term max(0,1+z)^2 is accumulated
                // as (x + |x|)^2 = (2 max(0,x))^2 and rescaled by 1/(4s)^2 once per tile.
                float x[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  x[i] = fmaf(gs2, round_bf16_as_f32(z[i]), gs2);   // logits are rounded to bf16 first, as the unfused forward stores them
                  if (WITH_LOSS) { const float m2 = x[i] + fabsf(x[i]); fast_loss = fmaf(m2, m2, fast_loss); }
                }
                pk = make_uint4(pack_bf16x2_relu(x[0], x[1]), pack_bf16x2_relu(x[2], x[3]), pack_bf16x2_relu(x[4], x[5]), pack_bf16x2_relu(x[6], x[7]));
              } else {
                // dLoss/dz = s sigmoid(z) = s/2 + s/2 tanh(z/2) (one MUFU op, one fma); loss term softplus(z) =
                // max(z,0) - ln 2 * log2(0.5 + 0.5 |tanh(z/2)|), whose logarithm argument stays in [0.5, 1]; the
                // log2 values are summed raw and scaled by -ln 2 once per tile.
                float x[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  const float zr = round_bf16_as_f32(z[i]);
                  float th;
                  asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(0.5f * zr));
                  x[i] = fmaf(hgs, th, hgs);
                  if (WITH_LOSS) { tile_loss += fmaxf(zr, 0.f); fast_loss += __log2f(fmaf(0.5f, fabsf(th), 0.5f)); }
                }
                pk = make_uint4(pack_bf16x2(x[0], x[1]), pack_bf16x2(x[2], x[3]), pack_bf16x2(x[4], x[5]), pack_bf16x2(x[6], x[7]));
              }
              const int chunk = ((col0 & 63) + c16 + e8) >> 3;     // 16-byte chunk inside the 128-byte row of this block
              *reinterpret_cast<uint4*>(ytile + ((chunk ^ (row & 7)) << 4)) = pk;
            }
          } else {
            const int nvalid = rows_real - (col0 + c16);           // columns of this chunk that are real labels
#pragma unroll
            for (int e8 = 0; e8 < 16; e8 += 8) {
              const float4 ba = bs4[(c16 + e8) >> 2], bb = bs4[((c16 + e8) >> 2) + 1];
              const float bias8[8] = {ba.x, ba.y, ba.z, ba.w, bb.x, bb.y, bb.z, bb.w};
              float x[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const float zr = round_bf16_as_f32(__uint_as_float(r[e8 + i]) + bias8[i]);
                const uint32_t pos = (ym16 >> (e8 + i)) & 1u;
                float gl, la;
                if (LOSS == HASTE_LOSS_SQHINGE) {
                  // squared hinge with target sign s: dLoss/dz = -2 s max(0, 1 - s z); ns = -s is built from the target bit
                  const float ns = __uint_as_float(0x3F800000u | (pos << 31));
                  const float m = fmaxf(fmaf(ns, zr, 1.f), 0.f);
                  gl = (ns * m) * gs2;
                  la = m * m;
                } else {
                  // dLoss/dz = sigmoid(z) - y, loss = max(z,0) - y z - ln(0.5 + 0.5 |tanh(z/2)|)
                  const float y = static_cast<float>(pos);
                  float th;
                  asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(0.5f * zr));
                  gl = (fmaf(0.5f, th, 0.5f) - y) * gs;
                  la = fmaxf(zr, 0.f) - y * zr - 0.69314718f * __log2f(fmaf(0.5f, fabsf(th), 0.5f));
                }
                if (e8 + i >= nvalid) { gl = 0.f; la = 0.f; }
                if (WITH_LOSS) tile_loss += la;
                x[i] = gl;
                if (DEBUG) {
                  if (a.z_dump != nullptr && row_valid && e8 + i < nvalid)
                    reinterpret_cast<uint16_t*>(a.z_dump)[(b0 + row) * a.ldz + static_cast<int64_t>(g) * G + col0 + c16 + e8 + i] =
                        static_cast<uint16_t>(__float_as_uint(zr) >> 16);
                }
              }
              const int chunk = ((col0 & 63) + c16 + e8) >> 3;
              *reinterpret_cast<uint4*>(ytile + ((chunk ^ (row & 7)) << 4)) =
                  make_uint4(pack_bf16x2(x[0], x[1]), pack_bf16x2(x[2], x[3]), pack_bf16x2(x[4], x[5]), pack_bf16x2(x[6], x[7]));
            }
          }
        }
        tc_fence_before();                             // this warp's half of the Z stage has been read
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(B_ZEMPTY + zs));
        if (WITH_LOSS && row_valid) loss_acc += tile_loss + fast_loss * (LOSS == HASTE_LOSS_SQHINGE ? inv_gs2_sq : -0.69314718f);
        if (es == 0 && lane == 0) TR(2 + 4 * set, 2700 + it);
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(B_YFULL + ys));
        if (es == 0 && lane == 0) TR(2 + 4 * set, 3000 + it);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(B_MEMPTY + ws));    // this warp no longer needs the group's bias row
    }
    if (WITH_LOSS) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) loss_acc += __shfl_xor_sync(0xffffffffu, loss_acc, o);
      if (lane == 0 && !*abort_flag) atomicAdd(a.loss, loss_acc * a.grad_scale);
    }
  } else if (warp >= 4 + N_EA && warp < 4 + N_EA + N_EB) {
    // ================================================================ epilogue B: dXg scatter
    const int q = warp & 3;
    const int row = q * 32 + lane;               // TMEM lane == batch row inside the tile
    const int bt = tid - (4 + N_EA) * 32;        // 0..127
    const int kh = (warp - (4 + N_EA)) >> 2;     // which half of the 64 slots this warp scatters
    int it = 0;
    for (int gi = 0; gi < n_my_groups; ++gi) {
      const int ws = gi & 1;
      mbar_wait(bar(B_WFULL + ws), (gi >> 1) & 1, abort_flag, a.err, 11, WAIT_LIMIT);   // loc_s of this group is in place
      const uint4* loc4 = reinterpret_cast<const uint4*>(loc_s + ws * F);
      for (int t = 0; t < T; ++t, ++it) {
        const int64_t b0 = tile_b0(t);
        const int ds = it & 1;
        mbar_wait(bar(B_DXFULL + ds), (it >> 1) & 1, abort_flag, a.err, 12, WAIT_LIMIT);
        tc_fence_after();
        if (bt == 0) TR(3, 1000 + it);
        const uint32_t ta = tmem + (static_cast<uint32_t>(q * 32) << 16) + TM_DX + (ds ? F : 0) + kh * 32;
        uint32_t r0[32];
        tmem_ld32(ta, r0);
        tmem_ld_wait();
        tc_fence_before();                         // this warp's half of the dXg tile is in registers: hand it back at once
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(B_DXEMPTY + ds));
        // dXg[b,k] of this thread's batch row goes to dxt[loc[k], b]: for a fixed k the warp's 32 lanes hit 32
        // consecutive floats, so each red below is one 128-byte transaction
        if ((b0 + row < a.B) && !*abort_flag) {
          float* dbase = a.dxt + b0 + row;
#pragma unroll
          for (int k4 = 0; k4 < 32; k4 += 4) {
            const uint4 lc = loc4[kh * 8 + (k4 >> 2)];      // 32-bit row offsets: one widening add per address
            atomicAdd(dbase + lc.x, __uint_as_float(r0[k4 + 0]));
            atomicAdd(dbase + lc.y, __uint_as_float(r0[k4 + 1]));
            atomicAdd(dbase + lc.z, __uint_as_float(r0[k4 + 2]));
            atomicAdd(dbase + lc.w, __uint_as_float(r0[k4 + 3]));
          }
        }
        if (bt == 0) TR(3, 2000 + it);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(B_MEMPTY + ws));    // this warp no longer needs the group's index row
    }
  } else {
    // ================================================================ update warps: SGD + stochastic rounding
    // Weight / bias update of each finished group from its dW accumulator: warp (q, kh) owns label rows
    // q*32..q*32+31 and slots kh*32..kh*32+31.  The accumulator slice is read, rounded to bf16 (as the unfused
    // kernel would store the gradient) and handed back to the tensor core at once; the old weights and bias are
    // copied out of the group's W tile / bias row in shared memory and the stage is released; only then does the
    // slow part (Philox, update arithmetic, stores) run, holding nothing the pipeline needs.
    const int q = warp & 3;
    const int row = q * 32 + lane;               // label row inside the group == TMEM lane
    const int kh = (warp - (4 + N_EA + N_EB)) >> 2;
    static_assert(UP_SLOTS == 32, "two 16-slot pieces per update warp");
    for (int gu = 0; gu < n_my_groups; ++gu) {
      const int gg = group_of(gu);
      const int wsu = gu & 1;
      const int64_t l0 = static_cast<int64_t>(gg) * G;
      const int rows_real_u = static_cast<int>(imin64(G, a.L - l0));
      mbar_wait(bar(B_WFULL + wsu), (gu >> 1) & 1, abort_flag, a.err, 15, WAIT_LIMIT);   // W tile and bias row are in place
      if (warp == 4 + N_EA + N_EB && lane == 0) TR(6, 4000 + gu);
      mbar_wait(bar(B_DWFULL), gu & 1, abort_flag, a.err, 13, WAIT_LIMIT);
      if (warp == 4 + N_EA + N_EB && lane == 0) TR(6, 4500 + gu);
      tc_fence_after();
      const uint32_t tdw = tmem + (static_cast<uint32_t>(q * 32) << 16) + TM_DW;
      uint32_t gw[16];                            // this thread's 32 gradients, bf16 pairs
      float gb = 0.f;
      {
        uint32_t r_lo[16], r_hi[16], rb[8];
        __syncwarp();
        tmem_ld16(tdw + kh * UP_SLOTS, r_lo);
        tmem_ld16(tdw + kh * UP_SLOTS + 16, r_hi);
        if (HAS_BIAS && kh == 0) tmem_ld8(tdw + F, rb);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(B_DWEMPTY));
#pragma unroll
        for (int x = 0; x < 8; ++x) {
          gw[x] = pack_bf16x2(__uint_as_float(r_lo[2 * x]), __uint_as_float(r_lo[2 * x + 1]));
          gw[8 + x] = pack_bf16x2(__uint_as_float(r_hi[2 * x]), __uint_as_float(r_hi[2 * x + 1]));
        }
        if (HAS_BIAS && kh == 0) gb = round_to_bf16_f(__uint_as_float(rb[0]));
      }
      uint32_t ww[16];                            // the same 32 old weights
      {
        const uint8_t* wsm = sm + OFF_W + wsu * WSTAGE + row * 128;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const uint4 wv = *reinterpret_cast<const uint4*>(wsm + (((kh * 4 + c) ^ (row & 7)) << 4));
          ww[4 * c] = wv.x; ww[4 * c + 1] = wv.y; ww[4 * c + 2] = wv.z; ww[4 * c + 3] = wv.w;
        }
      }
      // the old bias comes from the group's bias row (the fp32 image of the bf16 value: exact)
      const uint16_t b_old = (HAS_BIAS && kh == 0) ? __bfloat16_as_ushort(__float2bfloat16_rn(bias_s[wsu * G + row])) : uint16_t(0);
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(B_MEMPTY + wsu));   // this warp no longer needs the group's W tile / bias row
      if (row < rows_real_u && !*abort_flag) {
        const int64_t l = l0 + row, gl = u.label0 + l;
        const bool sr = u.flags & HASTE_F_SR, packed = u.flags & HASTE_F_RNG_PACKED, contract = u.flags & HASTE_F_CONTRACT;
        __nv_bfloat16* wrow = u.w + l * F;
        if (DEBUG) {
          if (a.dw_dump != nullptr) {
#pragma unroll
            for (int x = 0; x < 16; ++x) reinterpret_cast<uint32_t*>(a.dw_dump + l * F + kh * UP_SLOTS)[x] = gw[x];
          }
        }
#pragma unroll 1
        for (int pc = 0; pc < 2; ++pc) {          // two pieces of 16 slots (two Philox calls each in the packed stream)
          const int cq = kh * 2 + pc;
          uint32_t g8[8], w8[8];
#pragma unroll
          for (int x = 0; x < 8; ++x) { g8[x] = pc ? gw[8 + x] : gw[x]; w8[x] = pc ? ww[8 + x] : ww[x]; }
          uint32_t rnd[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};           // 16 x 16 random bits, two per word
          if (sr) {
            if (packed) {
              const uint4 rp0 = rand_packed8_call(u.seed, u.step, gl, cq * 2), rp1 = rand_packed8_call(u.seed, u.step, gl, cq * 2 + 1);
              rnd[0] = rp0.x; rnd[1] = rp0.y; rnd[2] = rp0.z; rnd[3] = rp0.w;
              rnd[4] = rp1.x; rnd[5] = rp1.y; rnd[6] = rp1.z; rnd[7] = rp1.w;
            } else {
#pragma unroll
              for (int x = 0; x < 16; x += 2)
                rnd[x >> 1] = rand16_reference_call(u.seed, gl * F + cq * 16 + x) | (rand16_reference_call(u.seed, gl * F + cq * 16 + x + 1) << 16);
            }
          }
          uint32_t ob[8];
          if (sr && contract) {
            // the configuration every benchmark and the reference's compiled kernel use, without per-element flag
            // tests: w' = fma(-lr, fma(wd, w, g), w), then add 16 random bits and keep the high half
#pragma unroll
            for (int p = 0; p < 8; ++p) {
              const float g0 = __uint_as_float(g8[p] << 16), g1 = __uint_as_float(g8[p] & 0xFFFF0000u);
              const float w0 = __uint_as_float(w8[p] << 16), w1 = __uint_as_float(w8[p] & 0xFFFF0000u);
              const float n0 = __fmaf_rn(-u.lr, __fmaf_rn(u.wd, w0, g0), w0), n1 = __fmaf_rn(-u.lr, __fmaf_rn(u.wd, w1, g1), w1);
              const uint32_t rr = rnd[p];
              const uint32_t s0 = __float_as_uint(n0) + (rr & 0xFFFFu), s1 = __float_as_uint(n1) + (rr >> 16);
              ob[p] = __byte_perm(s0, s1, 0x7632);              // high halves: s0 -> low 16 bits, s1 -> high 16 bits
            }
          } else
#pragma unroll
          for (int p = 0; p < 8; ++p) {
            const float g0 = __uint_as_float(g8[p] << 16), g1 = __uint_as_float(g8[p] & 0xFFFF0000u);
            const float w0 = __uint_as_float(w8[p] << 16), w1 = __uint_as_float(w8[p] & 0xFFFF0000u);
            float n0, n1;
            if (contract) { n0 = sgd_math<true>(w0, g0, nullptr, u.lr, u.wd, 0.f); n1 = sgd_math<true>(w1, g1, nullptr, u.lr, u.wd, 0.f); }
            else          { n0 = sgd_math<false>(w0, g0, nullptr, u.lr, u.wd, 0.f); n1 = sgd_math<false>(w1, g1, nullptr, u.lr, u.wd, 0.f); }
            const uint32_t rr = rnd[p];
            const uint32_t o0 = sr ? ((__float_as_uint(n0) + (rr & 0xFFFFu)) >> 16) : rn_bf16_bits(n0);
            const uint32_t o1 = sr ? ((__float_as_uint(n1) + (rr >> 16)) >> 16) : rn_bf16_bits(n1);
            ob[p] = (o0 & 0xFFFFu) | (o1 << 16);
          }
          *reinterpret_cast<uint4*>(wrow + cq * 16) = make_uint4(ob[0], ob[1], ob[2], ob[3]);
          *reinterpret_cast<uint4*>(wrow + cq * 16 + 8) = make_uint4(ob[4], ob[5], ob[6], ob[7]);
        }
        if (HAS_BIAS && kh == 0) {
          if (DEBUG) if (a.db_dump != nullptr) a.db_dump[l] = __float2bfloat16_rn(gb);
          uint32_t r16 = 0;
          if (sr) r16 = rand16_call(u.flags, u.seed ^ (packed ? 0x62696173ull : 0ull), u.step, gl);
          u.bias[l] = __ushort_as_bfloat16(sgd_update_bits(b_old, gb, nullptr, u.lr, u.wd, u.mu, u.flags, r16));
        }
      }
      if (warp == 4 + N_EA + N_EB && lane == 0) TR(6, 6000 + gu);
    }
  }

  // ---------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, TM_COLS);
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

bool train_step_sm100_supported(int64_t B, int64_t D, int64_t F, int64_t G, const UpdateArgs& u) {
  return G == s100::G && F == s100::F && (B % 8) == 0 && D * B < (int64_t(1) << 32) && u.mom_w == nullptr && u.mom_b == nullptr;
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
#define HASTE_S100_LAUNCH(LK, WL, HB, DBG)                                                                         \
  {                                                                                                                \
    auto k = ffi_train_step_sm100_kernel<LK, WL, HB, DBG>;                                                         \
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);               \
    if (e != cudaSuccess) return fail(HASTE_ERR_LAUNCH, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));         \
    k<<<grid, NTHREADS, SMEM_BYTES, st>>>(a, u);                                                                    \
  }
#define HASTE_S100_BY_LOSS(WL, HB, DBG)                                                                            \
  { if (loss_kind == HASTE_LOSS_BCE) HASTE_S100_LAUNCH(HASTE_LOSS_BCE, WL, HB, DBG) else HASTE_S100_LAUNCH(HASTE_LOSS_SQHINGE, WL, HB, DBG) }
  if (dump != nullptr) {
    // the debug variants always accumulate the loss
    if (loss == nullptr) return fail(HASTE_ERR_BAD_ARG, "debug step needs a loss pointer");
    if (hb) HASTE_S100_BY_LOSS(true, true, true) else HASTE_S100_BY_LOSS(true, false, true)
  } else if (wl) {
    if (hb) HASTE_S100_BY_LOSS(true, true, false) else HASTE_S100_BY_LOSS(true, false, false)
  } else {
    if (hb) HASTE_S100_BY_LOSS(false, true, false) else HASTE_S100_BY_LOSS(false, false, false)
  }
#undef HASTE_S100_BY_LOSS
#undef HASTE_S100_LAUNCH
  return check_launch("ffi_train_step_sm100_kernel");
}

}  // namespace haste

#ifdef HASTE_TRACE
extern "C" int haste_dbg_trace_dump(long long* out, int* counts) {
  cudaDeviceSynchronize();
  (void)counts;
  cudaMemcpyFromSymbol(out, haste::s100::g_trace, sizeof(long long) * 7 * 2048);
  void* p = nullptr;
  cudaGetSymbolAddress(&p, haste::s100::g_trace);
  cudaMemset(p, 0, sizeof(long long) * 7 * 2048);
  return 0;
}
#endif
