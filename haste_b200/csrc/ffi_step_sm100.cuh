// Fused FFI train step on the 5th-generation tensor cores (tcgen05 + TMEM), as a template over the two layer
// shapes the benchmark configurations use: (group size 128, fan-in 64) and (group size 64, fan-in 128).
//
// One persistent CTA per SM walks label groups g = blockIdx.x, += gridDim.x (the incomplete last round goes to the
// highest-numbered CTAs).  Per group and per 128-row batch tile three UMMA products run out of the same three
// shared-memory tiles (none is ever transposed or re-gathered; the 128-byte-swizzled "row block" layout serves both
// operand majors):
//     X tile [F + 16 rows = slots][128 batch]  rows of xt gathered by TMA (tile::gather4); row F holds ones
//     W tile [G rows = labels][F]               the group's weights, loaded by TMA through a 2-D tensor map
//     B tile [G rows][16]                       (no swizzle) the group's bias in column 0, zeros elsewhere
//     Y tile [128 batch][G]                     dLoss/dlogit for the tile, written by the loss-epilogue warps
//   forward            Z [b,l]  (TMEM, G cols)   = X^T (MN-major A) * [W | B] (K-major B), K = F + 16: the ones row
//                                                  times the bias column adds the bias inside the product
//   backward-features  dXg[b,k] (TMEM, F cols)   = Y (K-major A) * W (MN-major B),          K = G
//   backward-weights   dW [l,k] (TMEM, F+16 cols, accumulated over the batch tiles; M = G)
//                                                = Y^T (MN-major A) * X (K-major B),         K = 128; column F of the
//                                                  result (the ones row) is the bias gradient
// Warp roles: 4 producer warps (warp 0 loads the W tile through a tensor map; all four gather X tiles with TMA
// tile::gather4, one instruction per lane and tile — the gather rate grows with the number of issuing warps),
// warp 1 issues forward + backward-features, warp 3 issues backward-weights, 8 loss-epilogue warps turn Z into dY
// (bf16 rounding of the logit, loss gradient, target bits) and store it swizzled, 4 (F=64) or 8 (F=128) scatter
// warps drain dXg (TMEM -> registers -> coalesced red.global.add into dxt rows), 8 update warps apply SGD + weight
// decay (+ momentum) + stochastic rounding to the weights and bias straight from the dW accumulator.  Logits, dY
// and dW never reach global memory.
// All hand-offs are mbarriers with bounded waits; a wait that gives up raises a CTA-wide abort flag, every role
// drains its loops without touching global memory, TMEM is freed and the host sees HASTE_ERR_TIMEOUT.
#pragma once
#include "common.cuh"
#include "launchers.h"
#include "runtime.h"
#include "sm100.cuh"

namespace haste {
namespace s100 {
// out-of-line Philox for the reference random stream: that path is slow anyway and must not bloat the update code
__device__ __noinline__ static uint32_t rand16_reference_call(uint64_t seed, int64_t flat) { return rand16_reference(seed, flat); }
// the packed-stream generator is inlined into the update loop (measured: 4 % of the kernel against a call)
__device__ __forceinline__ static uint4 rand_packed8_call(uint64_t seed, uint32_t step, int64_t row, int col8) { return rand_packed8(seed, step, row, col8); }
__device__ __noinline__ static uint32_t rand16_call(uint32_t flags, uint64_t seed, uint32_t step, int64_t row) { return rand16(flags, seed, step, row, 0, 1); }

using namespace sm100;

template <int G_, int F_>
struct Cfg {
  static constexpr int G = G_, F = F_, BT = 128;
  static_assert((G == 128 && F == 64) || (G == 64 && F == 128), "shapes with a tcgen05 fused step");
  static constexpr int FR = F + 16;                   // rows of an X block: F gathered rows, one row of ones, 15 zero rows
  static constexpr int NXS = (F == 64) ? 5 : 4;       // X ring stages
  static constexpr int NYS = 2;                       // dY ring stages
  static constexpr int NDX = (F == 64) ? 2 : 1;       // dXg accumulator stages in TMEM
  static constexpr int XBLK = FR * 128;               // one 64-batch block of an X stage (bytes)
  static constexpr int XSTAGE = 2 * XBLK;
  static constexpr int NWB = F / 64;                  // 64-slot blocks of a W stage
  static constexpr int WBLK = G * 128;
  static constexpr int WSTAGE = NWB * WBLK;
  static constexpr int NYB = G / 64;                  // 64-label blocks of a dY stage
  static constexpr int YBLK = BT * 128;
  static constexpr int YSTAGE = NYB * YBLK;
  static constexpr int BTILE = G * 32;                // bias tile: G rows x 16 bf16, no swizzle
  static constexpr int OFF_X = 0;
  static constexpr int OFF_W = OFF_X + NXS * XSTAGE;
  static constexpr int OFF_Y = OFF_W + 2 * WSTAGE;
  static constexpr int OFF_BT = OFF_Y + NYS * YSTAGE;
  static constexpr int OFF_LOC = OFF_BT + 2 * BTILE;           // u32 [2][F]: element offset loc * B of each slot's dxt row
  static constexpr int OFF_LOCR = OFF_LOC + 2 * F * 4;         // int [4][F]: each producer warp's copy of the group's (clamped) indices, for the gather
  static constexpr int OFF_YB = OFF_LOCR + 4 * F * 4;          // u32 [2][BT][G/32]: target bits
  static constexpr int OFF_BAR = OFF_YB + 2 * BT * (G / 32) * 4;
  static constexpr int OFF_MISC = OFF_BAR + 32 * 8;            // tmem base address, abort flag
  static constexpr int SMEM_BYTES = OFF_MISC + 64 + 1024;      // + slack for the 1024-byte alignment of the base
  static_assert(SMEM_BYTES <= 232448, "shared memory budget");
  static_assert(XSTAGE % 1024 == 0 && WBLK % 1024 == 0 && YBLK % 1024 == 0 && OFF_BT % 128 == 0, "tile alignment");

  // barrier indices
  static constexpr int B_XFULL = 0, B_XEMPTY = NXS, B_WFULL = 2 * NXS, B_WEMPTY = B_WFULL + 2, B_ZFULL = B_WEMPTY + 2,
                       B_ZEMPTY = B_ZFULL + 2, B_YFULL = B_ZEMPTY + 2, B_YEMPTY = B_YFULL + NYS, B_DXFULL = B_YEMPTY + NYS,
                       B_DXEMPTY = B_DXFULL + NDX, B_DWFULL = B_DXEMPTY + NDX, B_DWEMPTY = B_DWFULL + 1, B_MEMPTY = B_DWEMPTY + 1,
                       B_FIN = B_MEMPTY + 2, NBAR = B_FIN + 2;   // B_FIN: one per issuer warp, "all my products have completed"
  static_assert(NBAR <= 32, "barrier space");

  // TMEM columns: Z double-buffered, dXg NDX stages, dW single (F + 16)
  static constexpr uint32_t TM_Z = 0, TM_DX = 2 * G, TM_DW = TM_DX + NDX * F, TM_COLS = 512;
  static_assert(TM_DW + FR <= TM_COLS, "TMEM budget");

  static constexpr int N_EA = 8;                      // loss-epilogue warps: 4 TMEM lane quarters x 2 column halves
  static constexpr int EBS = 64;                      // slots per scatter warp
  static constexpr int N_EB = 4 * (F / EBS);          // scatter warps: 4 TMEM lane quarters x 64-slot chunks
  static constexpr int N_UP = 8;                      // update warps: 4 TMEM lane quarters x 2 slot halves
  static constexpr int W_EA = 4, W_EB = W_EA + N_EA, W_UP = W_EB + N_EB;
  static constexpr int NPW = 4;                       // producer warps: warp 0, warp 2, then extra warps after the update warps
  static_assert(NPW >= 1 && NPW <= NXS, "a producer must not run more than one phase ahead on any stage barrier");
  static constexpr int W_XP = W_UP + N_UP;            // first extra producer warp
  static constexpr int NTHREADS = (W_XP + (NPW > 2 ? NPW - 2 : 0)) * 32;
  static_assert(NTHREADS <= 1024, "thread budget");
  static constexpr int EA_COLS = G * 4 / N_EA;        // label columns of a tile handled by one loss-epilogue warp
  static constexpr int UPS = F / 2;                   // slots updated by one update warp
  static constexpr int ROWS_PER_Q = G / 4;            // label rows of the dW accumulator in one TMEM lane quarter (32, or 16 for M = 64)
};

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
  long long wait_limit;
  int stall_tile;      // debug builds: the first loss-epilogue warp withholds its "dY ready" arrival at this tile (-1 = never)
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
__device__ __forceinline__ float tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int G_, int F_, int LOSS, bool WITH_LOSS, bool MOM, bool DEBUG>
__global__ void __launch_bounds__(Cfg<G_, F_>::NTHREADS, 1)
ffi_train_step_sm100_kernel(StepArgs a, UpdateArgs u, const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w) {
  using C = Cfg<G_, F_>;
  constexpr int G = C::G, F = C::F, BT = C::BT, FR = C::FR, NXS = C::NXS, NYS = C::NYS, NDX = C::NDX;
  constexpr int XBLK = C::XBLK, XSTAGE = C::XSTAGE, WBLK = C::WBLK, WSTAGE = C::WSTAGE, YBLK = C::YBLK, YSTAGE = C::YSTAGE;
  constexpr int N_EA = C::N_EA, N_EB = C::N_EB, N_UP = C::N_UP, EA_COLS = C::EA_COLS, UPS = C::UPS;
  constexpr int YBW = G / 32;                          // 32-bit words of target bits per batch row

  extern __shared__ uint8_t smem_raw[];
  uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const uint32_t sbase = smem_u32(sm);
  uint32_t* loc_s = reinterpret_cast<uint32_t*>(sm + C::OFF_LOC);
  uint32_t* ybits = reinterpret_cast<uint32_t*>(sm + C::OFF_YB);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + C::OFF_MISC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + C::OFF_MISC + 8);
  auto bar = [&](int i) { return sbase + C::OFF_BAR + i * 8; };
  const long long WL = a.wait_limit;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int T = static_cast<int>((a.B + BT - 1) / BT);
  // Every group's batch tiles are walked in the same order, t = 0 .. T-1: the order in which the tiles enter a group's
  // dW accumulator — and with it the last bit of the fp32 sum — must not depend on the rank or CTA the group lands on.
  // (An earlier build rotated the order by CTA index to spread the dX reductions of neighbouring SMs over dxt; a shard
  // boundary at an odd group index then showed 3 of 306,304 weights differing from the unsharded run.  Rotations by
  // the global group index with period 2, 4 or 8 all measured within 1 % of no rotation, which is what is left.)
  auto tile_b0 = [&](int t) { return t * BT; };
  const bool has_bias = u.bias != nullptr;

  // ---------------- one-time setup
  if (tid == 0) {
    for (int i = 0; i < NXS; ++i) { mbar_init(bar(C::B_XFULL + i), 1); mbar_init(bar(C::B_XEMPTY + i), 1); }   // X stage: one arrival that announces the gathered bytes
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(C::B_WFULL + i), 1);  mbar_init(bar(C::B_WEMPTY + i), 1);
      mbar_init(bar(C::B_ZFULL + i), 1);  mbar_init(bar(C::B_ZEMPTY + i), N_EA);
      mbar_init(bar(C::B_MEMPTY + i), N_EA + N_EB + N_UP);   // every epilogue warp is done with the group's index row, bias and W tile
    }
    for (int i = 0; i < NDX; ++i) { mbar_init(bar(C::B_DXFULL + i), 1); mbar_init(bar(C::B_DXEMPTY + i), N_EB); }
    for (int i = 0; i < NYS; ++i) { mbar_init(bar(C::B_YFULL + i), N_EA); mbar_init(bar(C::B_YEMPTY + i), 2); }   // both backward issuers commit
    mbar_init(bar(C::B_DWFULL), 1);
    mbar_init(bar(C::B_DWEMPTY), N_UP);
    mbar_init(bar(C::B_FIN), 1);
    mbar_init(bar(C::B_FIN + 1), 1);
    mbar_fence_init();
    *abort_flag = 0;
  }
  // rows F..FR-1 of every X block: row F = ones (bias column of the forward product, bias-gradient column of
  // backward-weights), the rest zeros; written once.  The bias tiles start as zeros.
  for (int i = tid; i < NXS * 2 * 16 * 8; i += C::NTHREADS) {
    const int chunk = i & 7, row = (i >> 3) & 15, blk = i >> 7;       // blk in [0, NXS*2)
    const uint32_t v = (row == 0) ? 0x3F803F80u : 0u;
    *reinterpret_cast<uint4*>(sm + C::OFF_X + blk * XBLK + (F + row) * 128 + chunk * 16) = make_uint4(v, v, v, v);
  }
  for (int i = tid; i < 2 * C::BTILE / 16; i += C::NTHREADS) *reinterpret_cast<uint4*>(sm + C::OFF_BT + i * 16) = make_uint4(0u, 0u, 0u, 0u);
  fence_proxy_async();
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), C::TM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  // Everything above touched only this CTA's shared memory and TMEM, so it may run while the preparation kernel that
  // precedes the step in the stream is still finishing; from here on the step reads what that kernel wrote.
  grid_dependency_wait();

  // Groups are dealt round-robin; the incomplete last round goes to the highest-numbered CTAs.  The head of a
  // long-tailed label distribution sits in the first groups, whose tiles are the expensive ones (positives, target
  // bitmap): the CTAs that own them then have one group less to do.
  const int n_cta = static_cast<int>(gridDim.x), cta = static_cast<int>(blockIdx.x);
  const int full_rounds = a.NG / n_cta, rem_groups = a.NG - full_rounds * n_cta;
  const int n_my_groups = full_rounds + (cta >= n_cta - rem_groups ? 1 : 0);
  auto group_of = [&](int gi) { return gi < full_rounds ? cta + gi * n_cta : full_rounds * n_cta + (cta - (n_cta - rem_groups)); };

  const int prod_id = warp == 0 ? 0 : (warp == 2 ? 1 : (warp >= C::W_XP ? 2 + warp - C::W_XP : -1));
  if (prod_id >= 0 && prod_id < C::NPW) {
    // ================================================================ producers
    // Per group: the index row (as dxt row offsets for the scatter warps) and the bias column go to shared memory
    // with ordinary stores, the W tile comes through the tensor map.  Per batch tile: F index rows of xt, 256 bytes
    // each, as F/4 TMA gather4 loads per 64-batch block (four index rows per instruction, landing at their swizzled
    // positions); lane 0 arms the stage's barrier with the byte count, then every lane issues its share.
    // The W item of every group belongs to producer 0; the X items (one per batch tile) are dealt round-robin.
    int it = 0;                  // X items so far (all producers count all of them)
    int w_armed = 0;             // W stages armed so far
    int my_last = -1;            // last X item this warp actually issued
    for (int gi = 0; gi < n_my_groups; ++gi) {
      const int g = group_of(gi);
      const int ws = gi & 1;
      const int64_t l0 = static_cast<int64_t>(g) * G;
      const int rows_real = static_cast<int>(imin64(G, a.L - l0));
      const int32_t* lrow = a.loc + static_cast<int64_t>(g) * F;
      int locv[F / 32];
#pragma unroll
      for (int j = 0; j < F / 32; ++j) locv[j] = min(max(__ldg(lrow + lane + 32 * j), 0), a.D - 1);   // clamped: never addresses outside xt / dxt
      if (prod_id == 0) {
      uint16_t bv[G / 32];
#pragma unroll
      for (int j = 0; j < G / 32; ++j) {
        const int c = lane + 32 * j;
        bv[j] = (has_bias && c < rows_real) ? __bfloat16_as_ushort(u.bias[l0 + c]) : uint16_t(0);
      }
      bool ok = mbar_wait(bar(C::B_WEMPTY + ws), ((gi >> 1) & 1) ^ 1, abort_flag, a.err, 1, WL, 100);
      ok = mbar_wait(bar(C::B_MEMPTY + ws), ((gi >> 1) & 1) ^ 1, abort_flag, a.err, 1, WL, 100) && ok;
      __syncwarp();
#pragma unroll
      for (int j = 0; j < F / 32; ++j) {
        loc_s[ws * F + lane + 32 * j] = static_cast<uint32_t>(locv[j]) * static_cast<uint32_t>(a.B);   // D * B < 2^32 is a launch condition
      }
#pragma unroll
      for (int j = 0; j < G / 32; ++j) {
        const int c = lane + 32 * j;
        *reinterpret_cast<uint16_t*>(sm + C::OFF_BT + ws * C::BTILE + (c >> 3) * 256 + (c & 7) * 16) = bv[j];
      }
      fence_proxy_async();
      __syncwarp();
      if (ok && !*abort_flag) {
        if (lane == 0) {
          mbar_arrive_expect_tx(bar(C::B_WFULL + ws), WSTAGE);
#pragma unroll
          for (int kb = 0; kb < C::NWB; ++kb)
            tma_load_2d(sbase + C::OFF_W + ws * WSTAGE + kb * WBLK, &tm_w, kb * 64, static_cast<int>(l0), bar(C::B_WFULL + ws));
        }
        ++w_armed;
      }
      __syncwarp();
      }
      // this warp's own copy of the index row, read back four slots at a time for the gathers
      int* locr = reinterpret_cast<int*>(sm + C::OFF_LOCR) + prod_id * F;
      __syncwarp();
#pragma unroll
      for (int j = 0; j < F / 32; ++j) locr[lane + 32 * j] = locv[j];
      __syncwarp();
      const int4* lr4 = reinterpret_cast<const int4*>(locr);
      for (int t = 0; t < T; ++t, ++it) {
        if (it % C::NPW != prod_id) continue;
        const int xs = it % NXS;
        const bool okx = mbar_wait(bar(C::B_XEMPTY + xs), ((it / NXS) & 1) ^ 1, abort_flag, a.err, 2, WL, 100);
        __syncwarp();
        if (!okx || *abort_flag) continue;
        const int b0 = tile_b0(t);
        const uint32_t xb = sbase + C::OFF_X + xs * XSTAGE;
        if (lane == 0) mbar_arrive_expect_tx(bar(C::B_XFULL + xs), F * 256);
        __syncwarp();
#pragma unroll
        for (int i = lane; i < 2 * (F / 4); i += 32) {        // one gather4 per four slots and 64-batch block
          const int blk = i / (F / 4), r4 = i % (F / 4);
          const int4 lr = lr4[r4];
          tma_gather4(xb + blk * XBLK + r4 * 512, &tm_x, b0 + blk * 64, lr.x, lr.y, lr.z, lr.w, bar(C::B_XFULL + xs));
        }
        my_last = it;
      }
    }
    // Every copy this warp started has to land before the CTA may exit (normally the consumers have long seen them;
    // after an abort nobody else waits any more).
    // (only the most recent use of each stage: an older phase of the same barrier can no longer be waited for)
    for (int j = max(0, it - NXS); j < it; ++j)
      if (j % C::NPW == prod_id && j <= my_last) mbar_wait_final(bar(C::B_XFULL + j % NXS), (j / NXS) & 1, WL);
    for (int j = max(0, w_armed - 2); j < w_armed; ++j) mbar_wait_final(bar(C::B_WFULL + (j & 1)), (j >> 1) & 1, WL);
  } else if (warp == 1 || warp == 3) {
    // ================================================================ MMA issuers (one elected lane each)
    // Feeding the tensor pipe from a single thread costs more cycles per tcgen05.mma than the small (N = 64..144)
    // products take to execute, so the work is split: warp 1 issues forward + backward-features, warp 3 issues
    // backward-weights.  Both hang off the same mbarriers; the pipe executes in arrival order.
    constexpr uint32_t ID_FWD = make_idesc(128, G, 1, 0);
    constexpr uint32_t ID_BWX = make_idesc(128, F, 0, 1);
    constexpr uint32_t ID_BWW = make_idesc(G, FR, 1, 0);
    // Descriptors are built once.  Per MMA only the start-address field (low word, 16-byte units) moves, by
    // compile-time constants; it never carries out of its 14-bit field because every operand lies inside the
    // CTA's shared memory window.
    const uint64_t D_XA = make_sdesc(sbase + C::OFF_X, XBLK, 1024);            // X tile as MN-major A   (forward)
    const uint64_t D_XB = make_sdesc(sbase + C::OFF_X, 16, 1024);              // X tile as K-major  B   (backward-weights)
    const uint64_t D_WB = make_sdesc(sbase + C::OFF_W, 16, 1024);              // W tile as K-major  B   (forward)
    const uint64_t D_BB = make_sdesc_noswizzle(sbase + C::OFF_BT, 128, 256);   // bias tile as K-major B (forward, last K step)
    const uint64_t D_WM = make_sdesc(sbase + C::OFF_W, WBLK, 1024);            // W tile as MN-major B   (backward-features)
    const uint64_t D_YA = make_sdesc(sbase + C::OFF_Y, 16, 1024);              // Y tile as K-major  A   (backward-features)
    const uint64_t D_YM = make_sdesc(sbase + C::OFF_Y, YBLK, 1024);            // Y tile as MN-major A   (backward-weights)
    if (warp == 1) {
      // ---------------- forward + backward-features
      const uint32_t xa_lo = static_cast<uint32_t>(D_XA), xa_hi = static_cast<uint32_t>(D_XA >> 32);
      const uint32_t wb_lo = static_cast<uint32_t>(D_WB), wb_hi = static_cast<uint32_t>(D_WB >> 32);
      const uint32_t bb_lo = static_cast<uint32_t>(D_BB), bb_hi = static_cast<uint32_t>(D_BB >> 32);
      const uint32_t wm_lo = static_cast<uint32_t>(D_WM), wm_hi = static_cast<uint32_t>(D_WM >> 32);
      const uint32_t ya_lo = static_cast<uint32_t>(D_YA), ya_hi = static_cast<uint32_t>(D_YA >> 32);
      const uint32_t id_fwd = ID_FWD, id_bwx = ID_BWX;
      // Order of issue: forward(it) first, then backward-features of tile it - 1.  Both become possible at the same
      // moment (the loss epilogue finished a tile); the forward product goes first because the epilogue warps are
      // waiting for it, while nothing waits for the backward product's dY stage yet.
      int it = 0, xs = 0, xph = 0;
      int j = 0, jy = 0, jyph = 0, j_t = 0, j_g = 0;     // next backward-features tile: dY stage and phase, position in its group
      auto backward_x = [&]() {
        const int ds = j % NDX, ws = j_g & 1;
        bool ok = mbar_wait(bar(C::B_YFULL + jy), jyph, abort_flag, a.err, 3, WL);
        ok = mbar_wait(bar(C::B_DXEMPTY + ds), ((j / NDX) & 1) ^ 1, abort_flag, a.err, 4, WL) && ok;
        tc_fence_after();
        const uint32_t ya = ya_lo + static_cast<uint32_t>(jy) * (YSTAGE >> 4), wm = wm_lo + (ws ? (WSTAGE >> 4) : 0u);
        const uint32_t tdx = tmem + C::TM_DX + ds * F;
        // dXg[b,k] = sum over label chunks of Y[b, l-chunk] * W[l-chunk, k]
        const bool last_of_group = j_t + 1 == T;
        if (ok && elect_one()) {          // after an abort nothing more is issued
          umma_bf16_lohi<false>(tdx, ya, ya_hi, wm, wm_hi, id_bwx);
#pragma unroll
          for (int ks = 1; ks < G / 16; ++ks)
            umma_bf16_lohi<true>(tdx, ya + (((ks >> 2) * YBLK + (ks & 3) * 32) >> 4), ya_hi, wm + ((ks * 2048) >> 4), wm_hi, id_bwx);
          tc_commit(bar(C::B_DXFULL + ds));
          tc_commit(bar(C::B_YEMPTY + jy));
          if (last_of_group) tc_commit(bar(C::B_WEMPTY + ws));   // every product that reads this group's W tile has been issued
        }
        __syncwarp();
        if (++jy == NYS) { jy = 0; jyph ^= 1; }
        ++j;
        if (++j_t == T) { j_t = 0; ++j_g; }
      };
      for (int gi = 0; gi < n_my_groups; ++gi) {
        const int ws = gi & 1;
        // the W stage of this group was last used by group gi - 2: its products must all be issued before the
        // stage can be refilled (matters only when a group has a single tile)
        while (j < it && j_g + 2 <= gi) backward_x();
        const bool okw = mbar_wait(bar(C::B_WFULL + ws), (gi >> 1) & 1, abort_flag, a.err, 5, WL);
        for (int t = 0; t < T; ++t, ++it) {
          const int zs = it & 1;
          bool ok = mbar_wait(bar(C::B_XFULL + xs), xph, abort_flag, a.err, 6, WL) && okw;
          ok = mbar_wait(bar(C::B_ZEMPTY + zs), ((it >> 1) & 1) ^ 1, abort_flag, a.err, 7, WL) && ok;
          tc_fence_after();
          const uint32_t xa = xa_lo + static_cast<uint32_t>(xs) * (XSTAGE >> 4), wb = wb_lo + (ws ? (WSTAGE >> 4) : 0u);
          const uint32_t bb = bb_lo + (ws ? (C::BTILE >> 4) : 0u);
          const uint32_t tz = tmem + C::TM_Z + zs * G;
          // Z[b,l] = sum over slot chunks of X[k-chunk, b]^T * W[l, k-chunk], then ones^T * bias
          if (ok && elect_one()) {
            umma_bf16_lohi<false>(tz, xa, xa_hi, wb, wb_hi, id_fwd);
#pragma unroll
            for (int ks = 1; ks < F / 16; ++ks)
              umma_bf16_lohi<true>(tz, xa + ((ks * 2048) >> 4), xa_hi, wb + (((ks >> 2) * WBLK + (ks & 3) * 32) >> 4), wb_hi, id_fwd);
            umma_bf16_lohi<true>(tz, xa + (((F / 16) * 2048) >> 4), xa_hi, bb, bb_hi, id_fwd);
            tc_commit(bar(C::B_ZFULL + zs));
          }
          __syncwarp();
          if (++xs == NXS) { xs = 0; xph ^= 1; }
          if (it >= 1) backward_x();
        }
      }
      while (j < it) backward_x();
      // every product this warp issued has completed before the CTA tears down its TMEM
      if (elect_one()) tc_commit(bar(C::B_FIN));
      __syncwarp();
      mbar_wait_final(bar(C::B_FIN), 0, WL);
    } else {
      // ---------------- backward-weights
      const uint32_t xb_lo = static_cast<uint32_t>(D_XB), xb_hi = static_cast<uint32_t>(D_XB >> 32);
      const uint32_t ym_lo = static_cast<uint32_t>(D_YM), ym_hi = static_cast<uint32_t>(D_YM >> 32);
      const uint32_t id_bww = ID_BWW;
      int j = 0, xs = 0, jy = 0, jyph = 0;
      for (int gi = 0; gi < n_my_groups; ++gi) {
        const uint32_t tdw = tmem + C::TM_DW;
        const bool okd = mbar_wait(bar(C::B_DWEMPTY), (gi & 1) ^ 1, abort_flag, a.err, 8, WL);
        for (int t = 0; t < T; ++t, ++j) {
          // Y(t) complete implies forward(t) complete, so the tile's X stage is loaded as well
          const bool ok = mbar_wait(bar(C::B_YFULL + jy), jyph, abort_flag, a.err, 9, WL) && okd;
          tc_fence_after();
          const uint32_t ym = ym_lo + static_cast<uint32_t>(jy) * (YSTAGE >> 4), xb = xb_lo + static_cast<uint32_t>(xs) * (XSTAGE >> 4);
          // dW[l,k] += sum over batch chunks of Y[b-chunk, l]^T * X[k, b-chunk]
          if (ok && elect_one()) {
            umma_bf16_lohi_rt(tdw, ym, ym_hi, xb, xb_hi, id_bww, t > 0);
#pragma unroll
            for (int ks = 1; ks < BT / 16; ++ks)
              umma_bf16_lohi<true>(tdw, ym + ((ks * 2048) >> 4), ym_hi, xb + (((ks >> 2) * XBLK + (ks & 3) * 32) >> 4), xb_hi, id_bww);
            tc_commit(bar(C::B_YEMPTY + jy));
            tc_commit(bar(C::B_XEMPTY + xs));
            if (t + 1 == T) tc_commit(bar(C::B_DWFULL));
          }
          __syncwarp();
          if (++jy == NYS) { jy = 0; jyph ^= 1; }
          if (++xs == NXS) xs = 0;
        }
      }
      if (elect_one()) tc_commit(bar(C::B_FIN + 1));
      __syncwarp();
      mbar_wait_final(bar(C::B_FIN + 1), 0, WL);
    }
  } else if (warp >= C::W_EA && warp < C::W_EB) {
    // ================================================================ loss epilogue: Z -> dY
    const int ea = warp - C::W_EA;
    const int q = ea & 3, h = ea >> 2;           // TMEM lane quarter, column range (EA_COLS labels each)
    const int row = q * 32 + lane;               // batch row inside the tile == TMEM lane
    const int et = tid - C::W_EA * 32;           // thread index inside the role
    float loss_acc = 0.f;
    const float inv_4gs2_sq = 0.0625f / (a.grad_scale * a.grad_scale);   // undoes the (4 s)^2 carried by the fast loss sum
    int it = 0, ys = 0, yph = 0;                 // global tile counter, its dY stage and phase
    for (int gi = 0; gi < n_my_groups; ++gi) {
      const int g = group_of(gi);
      const int ws = gi & 1;
      const int rows_real = static_cast<int>(imin64(G, a.L - static_cast<int64_t>(g) * G));
      const int t_beg = __ldg(a.tgt_ptr + g), t_end = __ldg(a.tgt_ptr + g + 1);
      const bool has_t = t_end > t_beg;
      for (int t = 0; t < T; ++t) {
        const int zs = it & 1;
        const int b0 = tile_b0(t);
        uint64_t ym = 0ull;                              // target bits of this thread's row, EA_COLS label columns
        if (has_t && t_end - t_beg <= 8) {
          // Few targets in this group (the common case): each thread picks the bits of its own row and its label
          // columns straight from the entry list — no shared bitmap, no barrier between the epilogue warps.
          const uint32_t rowkey = static_cast<uint32_t>(b0 + row);
          for (int i = t_beg; i < t_end; ++i) {
            const uint32_t e = __ldg(a.tgt_ent + i);
            const uint32_t c = (e & 0xFFu) - static_cast<uint32_t>(h * EA_COLS);
            if ((e >> 8) == rowkey && c < static_cast<uint32_t>(EA_COLS)) ym |= 1ull << c;
          }
        } else if (has_t) {
          uint32_t* yb = ybits + (it & 1) * BT * YBW;
          for (int i = et; i < BT * YBW; i += N_EA * 32) yb[i] = 0u;
          named_bar_sync(1, N_EA * 32);
          // head groups of a long-tailed label distribution hold thousands of entries: eight independent loads in
          // flight per thread, so that the scan runs at L2 throughput rather than one L2 latency per entry
          for (int i0 = t_beg + et; i0 < t_end; i0 += 8 * N_EA * 32) {
            uint32_t e8[8];
#pragma unroll
            for (int x = 0; x < 8; ++x) {
              const int i = i0 + x * N_EA * 32;
              e8[x] = i < t_end ? __ldg(a.tgt_ent + i) : 0xFFFFFFFFu;       // row 2^24 - 1: outside every tile
            }
#pragma unroll
            for (int x = 0; x < 8; ++x) {
              const int rb = static_cast<int>(e8[x] >> 8) - b0;
              const int c = e8[x] & 0xFF;
              if (rb >= 0 && rb < BT && c < G) atomicOr(&yb[rb * YBW + (c >> 5)], 1u << (c & 31));
            }
          }
          named_bar_sync(1, N_EA * 32);
          if (EA_COLS == 32) ym = yb[row * YBW + h];
          else ym = static_cast<uint64_t>(yb[row * YBW + h * 2]) | (static_cast<uint64_t>(yb[row * YBW + h * 2 + 1]) << 32);
        }
        const bool row_valid = b0 + row < a.B;
        const float gs = row_valid ? a.grad_scale : 0.f;
        mbar_wait(bar(C::B_ZFULL + zs), (it >> 1) & 1, abort_flag, a.err, 10, WL);
        mbar_wait(bar(C::B_YEMPTY + ys), yph ^ 1, abort_flag, a.err, 11, WL);
        tc_fence_after();
        const int col0 = h * EA_COLS;                              // first label column of this warp
        uint8_t* yrow = sm + C::OFF_Y + ys * YSTAGE + row * 128;
        const uint32_t ta = tmem + (static_cast<uint32_t>(q * 32) << 16) + C::TM_Z + zs * G + col0;
        const float gs2 = 2.f * gs;
        const float inv_gs2_sq = row_valid ? inv_4gs2_sq : 0.f;
        const bool ragged = col0 + EA_COLS > rows_real;     // only the last group of the layer can be ragged
        float tile_loss = 0.f, fast_loss = 0.f;             // fast_loss: hinge (4s)^2-scaled squares, or BCE raw log2 terms
        const float hgs = 0.5f * gs;
        // 16 label columns per iteration.  Nearly every chunk has no positive label in the warp's 32 rows and no
        // ragged edge: one warp vote per chunk sends those down a branch with no per-element tests; the rest take
        // the general branch with target bits and a column-valid mask.
        // (not unrolled: two iterations per loop body cost 27 % of the kernel's time, four 40 %, measured; moving the
        // general branch out of line, to shrink the loop instead, changed nothing)
        constexpr int CH = 16;                             // label columns per TMEM load
#pragma unroll 1
        for (int c16 = 0; c16 < EA_COLS; c16 += CH) {
          uint32_t r[CH];
          __syncwarp();
          tmem_ld(ta + c16, r);
          tmem_ld_wait();
          const uint32_t ym16 = static_cast<uint32_t>(ym >> c16) & (CH == 32 ? 0xFFFFFFFFu : 0xFFFFu);
          const bool general = DEBUG || ragged || __any_sync(0xffffffffu, ym16 != 0u);
          uint8_t* yblk = yrow + ((col0 + c16) >> 6) * YBLK;
          const int chunk0 = ((col0 + c16) & 63) >> 3;       // 16-byte chunk inside the 128-byte row of the block
          if (!general) {
            float bce_prod = 1.f;
            float fl[4] = {0.f, 0.f, 0.f, 0.f};        // partial sums: no serial dependency through one accumulator
#pragma unroll
            for (int e8 = 0; e8 < CH; e8 += 8) {
              uint4 pk;
              float x[8];
              if (LOSS == HASTE_LOSS_SQHINGE) {
                // dLoss/dz = 2 s max(0, 1 + z) with s = grad_scale, evaluated as max(0, fma(2s, z, 2s)); 1 + z is
                // exact in fp32 for a bf16 z (down to |z| ~ 2^-16), so this is the same single rounding as
                // (1 + z) * 2s.  The max is left to the bf16 conversion.  The loss term max(0,1+z)^2 is accumulated
                // as (x + |x|)^2 = (2 max(0,x))^2 and rescaled by 1/(4s)^2 once per tile.
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  x[i] = fmaf(gs2, round_bf16_as_f32(__uint_as_float(r[e8 + i])), gs2);   // logits are rounded to bf16 first, as the unfused forward stores them
                  if (WITH_LOSS) { const float m2 = x[i] + fabsf(x[i]); fl[i & 3] = fmaf(m2, m2, fl[i & 3]); }
                }
                pk = make_uint4(pack_bf16x2_relu(x[0], x[1]), pack_bf16x2_relu(x[2], x[3]), pack_bf16x2_relu(x[4], x[5]), pack_bf16x2_relu(x[6], x[7]));
              } else {
                // dLoss/dz = s sigmoid(z) = s/2 + s/2 tanh(z/2) (one MUFU op, one fma); loss term softplus(z) =
                // max(z,0) - ln(0.5 + 0.5 |tanh(z/2)|).  max(z,0) is summed as (z + |z|) / 2; the logarithm arguments
                // lie in [0.5, 1], so the 16 of a chunk are multiplied together (>= 2^-16) and one log2 is taken.
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  const float zr = round_bf16_as_f32(__uint_as_float(r[e8 + i]));
                  const float th = tanh_approx(0.5f * zr);
                  x[i] = fmaf(hgs, th, hgs);
                  if (WITH_LOSS) { fl[i & 1] += zr; fl[2 + (i & 1)] += fabsf(zr); bce_prod *= fmaf(0.5f, fabsf(th), 0.5f); }
                }
                pk = make_uint4(pack_bf16x2(x[0], x[1]), pack_bf16x2(x[2], x[3]), pack_bf16x2(x[4], x[5]), pack_bf16x2(x[6], x[7]));
              }
              *reinterpret_cast<uint4*>(yblk + (((chunk0 + (e8 >> 3)) ^ (row & 7)) << 4)) = pk;
            }
            if (WITH_LOSS) {
              if (LOSS == HASTE_LOSS_BCE) { fast_loss += __log2f(bce_prod); tile_loss += (fl[0] + fl[1]) + (fl[2] + fl[3]); }
              else fast_loss += (fl[0] + fl[1]) + (fl[2] + fl[3]);
            }
          } else {
            const int nvalid = rows_real - (col0 + c16);           // columns of this chunk that are real labels
#pragma unroll
            for (int e8 = 0; e8 < CH; e8 += 8) {
              float x[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const float zr = round_bf16_as_f32(__uint_as_float(r[e8 + i]));
                const uint32_t pos = (ym16 >> (e8 + i)) & 1u;
                float gl, la;
                if (LOSS == HASTE_LOSS_SQHINGE) {
                  // squared hinge with target sign s: dLoss/dz = -2 s max(0, 1 - s z); ns = -s is built from the target bit
                  const float ns = __uint_as_float(0x3F800000u | (pos << 31));
                  const float m = fmaxf(fmaf(ns, zr, 1.f), 0.f);
                  gl = (ns * m) * gs2;
                  la = m * m;
                } else {
                  // dLoss/dz = sigmoid(z) - y, loss = max(z,0) - y z - ln(0.5 + 0.5 |tanh(z/2)|); the factor 2 matches
                  // the (z + |z|) sums of the other branch, halved once per tile
                  const float y = static_cast<float>(pos);
                  const float th = tanh_approx(0.5f * zr);
                  gl = (fmaf(0.5f, th, 0.5f) - y) * gs;
                  la = 2.f * (fmaxf(zr, 0.f) - y * zr - 0.69314718f * __log2f(fmaf(0.5f, fabsf(th), 0.5f)));
                }
                if (e8 + i >= nvalid) { gl = 0.f; la = 0.f; }
                if (WITH_LOSS) tile_loss += la;
                x[i] = gl;
                if (DEBUG) {
                  if (a.z_dump != nullptr && row_valid && e8 + i < nvalid)
                    reinterpret_cast<uint16_t*>(a.z_dump)[(static_cast<int64_t>(b0) + row) * a.ldz + static_cast<int64_t>(g) * G + col0 + c16 + e8 + i] =
                        static_cast<uint16_t>(__float_as_uint(zr) >> 16);
                }
              }
              *reinterpret_cast<uint4*>(yblk + (((chunk0 + (e8 >> 3)) ^ (row & 7)) << 4)) =
                  make_uint4(pack_bf16x2(x[0], x[1]), pack_bf16x2(x[2], x[3]), pack_bf16x2(x[4], x[5]), pack_bf16x2(x[6], x[7]));
            }
          }
        }
        tc_fence_before();                             // this warp's part of the Z stage has been read
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(C::B_ZEMPTY + zs));
        if (WITH_LOSS && row_valid) {
          // hinge: tile_loss holds plain squares, fast_loss (4s)^2-scaled ones; BCE: tile_loss holds twice the
          // max(z,0)-type terms, fast_loss raw log2 sums
          if (LOSS == HASTE_LOSS_SQHINGE) loss_acc += tile_loss + fast_loss * inv_gs2_sq;
          else loss_acc += 0.5f * tile_loss - 0.69314718f * fast_loss;
        }
        fence_proxy_async();
        __syncwarp();
        const bool stall = DEBUG && ea == 0 && it == a.stall_tile;   // test hook: leave the dY stage one arrival short
        if (lane == 0 && !stall) mbar_arrive(bar(C::B_YFULL + ys));
        ++it;
        if (++ys == NYS) { ys = 0; yph ^= 1; }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(C::B_MEMPTY + ws));    // this warp no longer needs anything of the group
    }
    if (WITH_LOSS) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) loss_acc += __shfl_xor_sync(0xffffffffu, loss_acc, o);
      if (lane == 0 && !*abort_flag) atomicAdd(a.loss, loss_acc * a.grad_scale);
    }
  } else if (warp >= C::W_EB && warp < C::W_UP) {
    // ================================================================ scatter: dXg -> dxt
    const int e = warp - C::W_EB;
    const int q = warp & 3;
    const int row = q * 32 + lane;               // TMEM lane == batch row inside the tile
    const int kc = e >> 2;                       // which EBS-slot chunk this warp scatters
    int it = 0;
    for (int gi = 0; gi < n_my_groups; ++gi) {
      const int ws = gi & 1;
      mbar_wait(bar(C::B_WFULL + ws), (gi >> 1) & 1, abort_flag, a.err, 12, WL);   // loc_s of this group is in place
      const uint4* loc4 = reinterpret_cast<const uint4*>(loc_s + ws * F + kc * C::EBS);
      for (int t = 0; t < T; ++t, ++it) {
        const int b0 = tile_b0(t);
        const int ds = it % NDX;
        mbar_wait(bar(C::B_DXFULL + ds), (it / NDX) & 1, abort_flag, a.err, 13, WL);
        tc_fence_after();
        const uint32_t ta = tmem + (static_cast<uint32_t>(q * 32) << 16) + C::TM_DX + ds * F + kc * C::EBS;
        // dXg[b,k] of this thread's batch row goes to dxt[loc[k], b]: for a fixed k the warp's 32 lanes hit 32
        // consecutive floats, so each red below is one 128-byte transaction.  Two halves of 32 slots, so that only
        // 32 accumulator values are live at a time; the stage goes back to the tensor core after the second load.
        const bool do_red = (b0 + row < a.B) && !*abort_flag;
        float* dbase = a.dxt + b0 + row;
#pragma unroll
        for (int half = 0; half < C::EBS / 32; ++half) {
          uint32_t r0[32];
          tmem_ld32(ta + half * 32, r0);
          tmem_ld_wait();
          if (half == C::EBS / 32 - 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(C::B_DXEMPTY + ds));
          }
          if (do_red) {
#pragma unroll
            for (int k4 = 0; k4 < 32; k4 += 4) {
              const uint4 lc = loc4[half * 8 + (k4 >> 2)];      // 32-bit row offsets: one widening add per address
              atomicAdd(dbase + lc.x, __uint_as_float(r0[k4 + 0]));
              atomicAdd(dbase + lc.y, __uint_as_float(r0[k4 + 1]));
              atomicAdd(dbase + lc.z, __uint_as_float(r0[k4 + 2]));
              atomicAdd(dbase + lc.w, __uint_as_float(r0[k4 + 3]));
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(C::B_MEMPTY + ws));    // this warp no longer needs the group's index row
    }
  } else if (warp >= C::W_UP && warp < C::W_XP) {
    // ================================================================ update warps: SGD + stochastic rounding
    // Weight / bias update of each finished group from its dW accumulator: warp (q, kh) owns the label rows of TMEM
    // lane quarter q (32 rows for G = 128; 16 for G = 64, where an M = 64 accumulator occupies lanes 0-15 of each
    // quarter) and slots kh*UPS .. kh*UPS+UPS-1.  The accumulator slice is read, rounded to bf16 (as the unfused
    // kernel would store the gradient) and handed back to the tensor core at once; the old weights come out of the
    // group's W tile in shared memory.
    const int e = warp - C::W_UP;
    const int q = warp & 3;
    const int kh = e >> 2;
    // G = 64: only lanes 0-15 of a TMEM lane quarter hold accumulator rows, so lane l and lane l+16 share label row
    // l: lane l keeps the lower 8 slots of every 16-slot piece, lane l+16 gets the upper 8 by shuffle — the whole
    // warp works and a lane's 8 slots are exactly one Philox call, one 16-byte chunk of W and one 16-byte store.
    constexpr bool SPLIT = C::ROWS_PER_Q == 16;
    constexpr int NSL = SPLIT ? 8 : 16;            // slots per lane and piece
    const int lrow = SPLIT ? (lane & 15) : lane;
    const int half = SPLIT ? (lane >> 4) : 0;
    const int row = q * C::ROWS_PER_Q + lrow;      // label row inside the group
    constexpr int NPC = UPS / 16;                  // pieces of 16 slots
    for (int gu = 0; gu < n_my_groups; ++gu) {
      const int gg = group_of(gu);
      const int wsu = gu & 1;
      const int64_t l0 = static_cast<int64_t>(gg) * G;
      const int rows_real_u = static_cast<int>(imin64(G, a.L - l0));
      mbar_wait(bar(C::B_WFULL + wsu), (gu >> 1) & 1, abort_flag, a.err, 14, WL);   // W tile and bias column are in place
      mbar_wait(bar(C::B_DWFULL), gu & 1, abort_flag, a.err, 15, WL);
      tc_fence_after();
      const uint32_t tdw = tmem + (static_cast<uint32_t>(q * 32) << 16) + C::TM_DW;
      uint32_t gw[UPS / 2];                       // this TMEM lane's gradients, bf16 pairs (garbage in lanes 16-31 when SPLIT)
      float gb = 0.f;
      {
        __syncwarp();
#pragma unroll
        for (int pc = 0; pc < NPC; ++pc) {
          uint32_t rr[16];
          tmem_ld16(tdw + kh * UPS + pc * 16, rr);
          tmem_ld_wait();
#pragma unroll
          for (int x = 0; x < 8; ++x) gw[pc * 8 + x] = pack_bf16x2(__uint_as_float(rr[2 * x]), __uint_as_float(rr[2 * x + 1]));
        }
        if (kh == 0) {
          uint32_t rb[8];
          tmem_ld8(tdw + F, rb);
          tmem_ld_wait();
          gb = round_to_bf16_f(__uint_as_float(rb[0]));
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(C::B_DWEMPTY));
      }
      const bool do_row = row < rows_real_u && !*abort_flag;
      const unsigned row_mask = __ballot_sync(0xffffffffu, do_row);      // lanes l and l+16 always agree
      const int64_t l = l0 + row, gl = u.label0 + l;
      const bool sr = u.flags & HASTE_F_SR, packed = u.flags & HASTE_F_RNG_PACKED, contract = u.flags & HASTE_F_CONTRACT;
      // the old bias comes from the group's bias column in shared memory
      const uint16_t b_old = (has_bias && kh == 0 && half == 0)
                                 ? *reinterpret_cast<const uint16_t*>(sm + C::OFF_BT + wsu * C::BTILE + (row >> 3) * 256 + (row & 7) * 16)
                                 : uint16_t(0);
      if (do_row) {
        __nv_bfloat16* wrow = u.w + l * F;
#pragma unroll 1
        for (int pc = 0; pc < NPC; ++pc) {          // pieces of 16 slots
          uint32_t p8[8];
#pragma unroll
          for (int x = 0; x < 8; ++x) p8[x] = gw[x];
#pragma unroll
          for (int p2 = 1; p2 < NPC; ++p2)       // register select (a dynamic index would put gw in local memory)
            if (p2 == pc) {
#pragma unroll
              for (int x = 0; x < 8; ++x) p8[x] = gw[p2 * 8 + x];
            }
          uint32_t g8[NSL / 2], w8[NSL / 2];
          if (SPLIT) {
#pragma unroll
            for (int x = 0; x < 4; ++x) {
              const uint32_t up = __shfl_sync(row_mask, p8[4 + x], lane & 15);     // upper 8 slots of the piece, from the lane that read TMEM
              g8[x] = half ? up : p8[x];
            }
          } else {
#pragma unroll
            for (int x = 0; x < NSL / 2; ++x) g8[x] = p8[x];
          }
          const int s0 = kh * UPS + pc * 16 + half * 8;        // first slot of this lane's part of the piece
          {
            // the old weights: one (SPLIT) or two 16-byte chunks of the row in the W tile
            const uint8_t* wsm = sm + C::OFF_W + wsu * WSTAGE + (s0 >> 6) * WBLK + row * 128;
            const int c0 = (s0 & 63) >> 3;
            const uint4 wa = *reinterpret_cast<const uint4*>(wsm + ((c0 ^ (row & 7)) << 4));
            w8[0] = wa.x; w8[1] = wa.y; w8[2] = wa.z; w8[3] = wa.w;
            if (!SPLIT) {
              const uint4 wb = *reinterpret_cast<const uint4*>(wsm + (((c0 + 1) ^ (row & 7)) << 4));
              w8[NSL / 2 - 4] = wb.x; w8[NSL / 2 - 3] = wb.y; w8[NSL / 2 - 2] = wb.z; w8[NSL / 2 - 1] = wb.w;
            }
          }
          if (DEBUG) {
            if (a.dw_dump != nullptr) {
#pragma unroll
              for (int x = 0; x < NSL / 2; ++x) reinterpret_cast<uint32_t*>(a.dw_dump + l * F + s0)[x] = g8[x];
            }
          }
          uint32_t rnd[NSL / 2];           // NSL x 16 random bits, two per word
#pragma unroll
          for (int x = 0; x < NSL / 2; ++x) rnd[x] = 0u;
          if (sr) {
            if (packed) {
              const uint4 rp0 = rand_packed8_call(u.seed, u.step, gl, s0 >> 3);
              rnd[0] = rp0.x; rnd[1] = rp0.y; rnd[2] = rp0.z; rnd[3] = rp0.w;
              if (!SPLIT) {
                const uint4 rp1 = rand_packed8_call(u.seed, u.step, gl, (s0 >> 3) + 1);
                rnd[NSL / 2 - 4] = rp1.x; rnd[NSL / 2 - 3] = rp1.y; rnd[NSL / 2 - 2] = rp1.z; rnd[NSL / 2 - 1] = rp1.w;
              }
            } else {
#pragma unroll
              for (int x = 0; x < NSL; x += 2)
                rnd[x >> 1] = rand16_reference_call(u.seed, gl * F + s0 + x) | (rand16_reference_call(u.seed, gl * F + s0 + x + 1) << 16);
            }
          }
          uint32_t ob[NSL / 2];
          if (!MOM && sr && contract) {
            // the configuration every benchmark and the reference's compiled kernel use, without per-element flag
            // tests: w' = fma(-lr, fma(wd, w, g), w), then add 16 random bits and keep the high half
#pragma unroll
            for (int p = 0; p < NSL / 2; ++p) {
              const float g0 = __uint_as_float(g8[p] << 16), g1 = __uint_as_float(g8[p] & 0xFFFF0000u);
              const float w0 = __uint_as_float(w8[p] << 16), w1 = __uint_as_float(w8[p] & 0xFFFF0000u);
              const float n0 = __fmaf_rn(-u.lr, __fmaf_rn(u.wd, w0, g0), w0), n1 = __fmaf_rn(-u.lr, __fmaf_rn(u.wd, w1, g1), w1);
              const uint32_t rr = rnd[p];
              const uint32_t s0b = __float_as_uint(n0) + (rr & 0xFFFFu), s1b = __float_as_uint(n1) + (rr >> 16);
              ob[p] = __byte_perm(s0b, s1b, 0x7632);              // high halves: s0b -> low 16 bits, s1b -> high 16 bits
            }
          } else {
            float mv[NSL];
            float* mrow = MOM ? u.mom_w + l * F + s0 : nullptr;
            if (MOM) {
#pragma unroll
              for (int x = 0; x < NSL / 4; ++x) {
                const float4 m4 = reinterpret_cast<const float4*>(mrow)[x];
                mv[4 * x] = m4.x; mv[4 * x + 1] = m4.y; mv[4 * x + 2] = m4.z; mv[4 * x + 3] = m4.w;
              }
            }
#pragma unroll
            for (int p = 0; p < NSL / 2; ++p) {
              const float g0 = __uint_as_float(g8[p] << 16), g1 = __uint_as_float(g8[p] & 0xFFFF0000u);
              const float w0 = __uint_as_float(w8[p] << 16), w1 = __uint_as_float(w8[p] & 0xFFFF0000u);
              float n0, n1;
              if (contract) { n0 = sgd_math<true>(w0, g0, MOM ? &mv[2 * p] : nullptr, u.lr, u.wd, u.mu); n1 = sgd_math<true>(w1, g1, MOM ? &mv[2 * p + 1] : nullptr, u.lr, u.wd, u.mu); }
              else          { n0 = sgd_math<false>(w0, g0, MOM ? &mv[2 * p] : nullptr, u.lr, u.wd, u.mu); n1 = sgd_math<false>(w1, g1, MOM ? &mv[2 * p + 1] : nullptr, u.lr, u.wd, u.mu); }
              const uint32_t rr = rnd[p];
              const uint32_t o0 = sr ? ((__float_as_uint(n0) + (rr & 0xFFFFu)) >> 16) : rn_bf16_bits(n0);
              const uint32_t o1 = sr ? ((__float_as_uint(n1) + (rr >> 16)) >> 16) : rn_bf16_bits(n1);
              ob[p] = (o0 & 0xFFFFu) | (o1 << 16);
            }
            if (MOM) {
#pragma unroll
              for (int x = 0; x < NSL / 4; ++x) reinterpret_cast<float4*>(mrow)[x] = make_float4(mv[4 * x], mv[4 * x + 1], mv[4 * x + 2], mv[4 * x + 3]);
            }
          }
          *reinterpret_cast<uint4*>(wrow + s0) = make_uint4(ob[0], ob[1], ob[2], ob[3]);
          if (!SPLIT) *reinterpret_cast<uint4*>(wrow + s0 + 8) = make_uint4(ob[NSL / 2 - 4], ob[NSL / 2 - 3], ob[NSL / 2 - 2], ob[NSL / 2 - 1]);
        }
        if (has_bias && kh == 0 && half == 0) {
          if (DEBUG) if (a.db_dump != nullptr) a.db_dump[l] = __float2bfloat16_rn(gb);
          uint32_t r16 = 0;
          if (sr) r16 = rand16_call(u.flags, u.seed ^ (packed ? 0x62696173ull : 0ull), u.step, gl);
          u.bias[l] = __ushort_as_bfloat16(sgd_update_bits(b_old, gb, (MOM && u.mom_b != nullptr) ? u.mom_b + l : nullptr, u.lr, u.wd, u.mu, u.flags, r16));
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(C::B_MEMPTY + wsu));   // this warp no longer needs the group's W tile / bias column
    }
  }

  // ---------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, C::TM_COLS);
}

// Launch one shape.  `dump` selects the debug instantiation (always accumulates the loss).
template <int G_, int F_>
int launch_step_shape(const int32_t* loc, const void* xt, const int32_t* tgt_ptr, const uint32_t* tgt_ent, float* dxt, float* loss,
                      const UpdateArgs& u, int64_t B, int64_t D, int64_t L, int loss_kind, float grad_scale, int max_ctas, cudaStream_t st,
                      const StepDump* dump) {
  using C = Cfg<G_, F_>;
  if (int rc = report_pending_status("fused train step")) return rc;
  StepArgs a;
  a.loc = loc; a.xt = static_cast<const __nv_bfloat16*>(xt); a.tgt_ptr = tgt_ptr; a.tgt_ent = tgt_ent; a.dxt = dxt; a.loss = loss;
  if (int rc = device_status_word(&a.err)) return rc;
  a.B = B; a.L = L; a.D = static_cast<int>(D); a.NG = static_cast<int>((L + G_ - 1) / G_); a.grad_scale = grad_scale;
  a.wait_limit = wait_limit_cycles();
  a.stall_tile = dump ? take_stall_tile() : -1;
  a.z_dump = dump ? static_cast<__nv_bfloat16*>(dump->z) : nullptr; a.ldz = dump ? dump->ldz : 0;
  a.dw_dump = dump ? static_cast<__nv_bfloat16*>(dump->dw) : nullptr; a.db_dump = dump ? static_cast<__nv_bfloat16*>(dump->dbias) : nullptr;
  CUtensorMap tm_x, tm_w;
  // xt [D][B]: one box = 64 batch columns of one row (gather4 stacks four rows); W [L][F]: one box = 64 slots x G labels
  if (int rc = make_tmap_bf16_2d(&tm_x, xt, static_cast<uint64_t>(B), static_cast<uint64_t>(D), static_cast<uint64_t>(B) * 2, 64, 1)) return rc;
  if (int rc = make_tmap_bf16_2d(&tm_w, u.w, static_cast<uint64_t>(F_), static_cast<uint64_t>(L), static_cast<uint64_t>(F_) * 2, 64, G_)) return rc;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (max_ctas > 0 && max_ctas < sms) sms = max_ctas;
  const int grid = a.NG < sms ? a.NG : sms;
  const bool wl = (u.flags & HASTE_F_LOSS) && loss != nullptr;
  const bool mom = u.mom_w != nullptr;
#define HASTE_S100_LAUNCH(LK, WLOSS, MOMF, DBG)                                                                     \
  {                                                                                                                \
    auto k = ffi_train_step_sm100_kernel<G_, F_, LK, WLOSS, MOMF, DBG>;                                             \
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);            \
    if (e != cudaSuccess) return fail(HASTE_ERR_LAUNCH, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));         \
    cudaLaunchConfig_t cfg = {};                                                                                   \
    cfg.gridDim = dim3(static_cast<unsigned>(grid)); cfg.blockDim = dim3(C::NTHREADS);                              \
    cfg.dynamicSmemBytes = C::SMEM_BYTES; cfg.stream = st;                                                          \
    cudaLaunchAttribute attr[1];                                                                                    \
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;                                                \
    attr[0].val.programmaticStreamSerializationAllowed = 1;   /* the prologue overlaps the preceding kernel's tail */ \
    cfg.attrs = attr; cfg.numAttrs = dependent_launch_enabled() ? 1 : 0;                                            \
    e = cudaLaunchKernelEx(&cfg, k, a, u, tm_x, tm_w);                                                              \
    if (e != cudaSuccess) return fail(HASTE_ERR_LAUNCH, "cudaLaunchKernelEx: %s", cudaGetErrorString(e));           \
  }
#define HASTE_S100_BY_LOSS(WLOSS, MOMF, DBG)                                                                       \
  { if (loss_kind == HASTE_LOSS_BCE) HASTE_S100_LAUNCH(HASTE_LOSS_BCE, WLOSS, MOMF, DBG) else HASTE_S100_LAUNCH(HASTE_LOSS_SQHINGE, WLOSS, MOMF, DBG) }
  if (dump != nullptr) {
    if (loss == nullptr) return fail(HASTE_ERR_BAD_ARG, "debug step needs a loss pointer");
    if (mom) return fail(HASTE_ERR_UNSUPPORTED, "debug step: momentum is not supported");
    HASTE_S100_BY_LOSS(true, false, true)
  } else if (wl) {
    if (mom) HASTE_S100_BY_LOSS(true, true, false) else HASTE_S100_BY_LOSS(true, false, false)
  } else {
    if (mom) HASTE_S100_BY_LOSS(false, true, false) else HASTE_S100_BY_LOSS(false, false, false)
  }
#undef HASTE_S100_BY_LOSS
#undef HASTE_S100_LAUNCH
  return check_launch("ffi_train_step_sm100_kernel");
}

}  // namespace s100
}  // namespace haste
