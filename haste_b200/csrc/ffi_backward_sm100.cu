// Unfused backward of the FFI layer on tcgen05 / TMEM, for the layer shapes (group size 128, fan-in 64) and
// (group size 64, fan-in 128): one pass over dY [B, ldy] produces both gradients of the autograd surface,
//     dxt[loc[g,k], b] += sum_{l in g} w[l,k] * dy[b,l]          (fp32, reduced into dxt with red.global.add)
//     dw [l, k]         = sum_b dy[b,l] * xt[loc[g,k], b]          (bf16, round to nearest)
//     dbias[l]          = sum_b dy[b,l]                            (bf16; via a row of ones under the X tile)
// so dY is read from HBM once instead of once per gradient.  HBM-bound by that read (2*B*L bytes).
//
// Persistent, one CTA per SM.  Same operand layouts as the fused train step: per 128-row batch tile the Y tile
// (a dY slice), the X tile and the W tile sit in 128-byte-swizzled shared memory; backward-features takes Y as
// K-major A and W as MN-major B, backward-weights takes Y as MN-major A and X as K-major B.
//
// The rows of dY need no alignment.  An autograd gradient is a contiguous [B, L] tensor and L is odd in most
// real label sets, so a row's slice for one group starts at any even byte offset.  The eight "Y warps" copy
// the 16-byte-aligned chunks that cover each row slice (cp.async, G/8 + 1 chunks per row) to the slice's own place
// in the Y tile, then shift every row left by its misalignment inside shared memory (two 16-byte reads, four
// funnel shifts, one 16-byte write per chunk) before they hand the tile to the tensor core.  Rows whose index
// is equal modulo 8 share the misalignment, so each warp takes one such class and the shift is warp-uniform.
// Columns at and beyond L are zeroed in the same pass (their neighbours in memory belong to the next row).
//
// Warp roles (24 or 25 warps): warps 0, 2 (and 24) gather X tiles with TMA tile::gather4 (warp 0 also loads the W tile
// through a tensor map), warp 1 issues backward-features, warp 3 backward-weights, warps 4-11 drain dXg (TMEM ->
// registers -> coalesced red.global.add.f32), warps 12-15 turn the dW accumulator into bf16 rows of dw / dbias at
// the end of each group, warps 16-23 are the Y warps.  All waits are bounded (see mbar_wait).
#include "common.cuh"
#include "launchers.h"
#include "runtime.h"
#include "sm100.cuh"

namespace haste {
namespace b100 {
using namespace sm100;

template <int G_, int F_>
struct Cfg {
  static constexpr int G = G_, F = F_, BT = 128;
  static_assert((G == 128 && F == 64) || (G == 64 && F == 128), "shapes with a tcgen05 backward");
  static constexpr int FR = F + 16;                   // X block rows: F gathered rows, one row of ones, 15 zero rows
  // Shared memory goes to the dY ring first: dY streams from HBM (several microseconds from request to arrival under
  // load, and a tile that has arrived still has to be shifted), the X rows come out of L2.
  static constexpr int NXS = (F == 64) ? 2 : 3;       // X ring stages
  static constexpr int NYS = 4;                       // dY ring stages
  static constexpr int NDX = 2;                       // dXg accumulator stages
  static constexpr int NDW = (F == 64) ? 2 : 1;       // dW accumulator stages
  static constexpr int XBLK = FR * 128, XSTAGE = 2 * XBLK;
  static constexpr int NWB = F / 64, WBLK = G * 128, WSTAGE = NWB * WBLK;
  static constexpr int NYB = G / 64, YBLK = BT * 128, YSTAGE = NYB * YBLK;
  static constexpr int NCH = G / 8;                   // 16-byte chunks of a row slice
  static constexpr int YSIDE = BT * 16;               // one more aligned chunk per row (the tail of a misaligned slice)
  static constexpr int OFF_X = 0;
  static constexpr int OFF_W = OFF_X + NXS * XSTAGE;
  static constexpr int OFF_Y = OFF_W + 2 * WSTAGE;
  static constexpr int OFF_YSIDE = OFF_Y + NYS * YSTAGE;
  static constexpr int OFF_LOC = OFF_YSIDE + NYS * YSIDE;      // u32 [2][F]: element offset loc * B of each slot's dxt row
  static constexpr int OFF_LOCR = OFF_LOC + 2 * F * 4;         // int [4][F]: each producer warp's copy of the group's indices
  static constexpr int OFF_BAR = OFF_LOCR + 4 * F * 4;
  static constexpr int OFF_MISC = OFF_BAR + 40 * 8;
  static constexpr int SMEM_BYTES = OFF_MISC + 64 + 1024;
  static_assert(SMEM_BYTES <= 232448, "shared memory budget");
  static_assert(XSTAGE % 1024 == 0 && WBLK % 1024 == 0 && YBLK % 1024 == 0, "tile alignment");
  static constexpr int B_XFULL = 0, B_XEMPTY = NXS, B_YFULL = 2 * NXS, B_YEMPTY = B_YFULL + NYS, B_WFULL = B_YEMPTY + NYS,
                       B_WEMPTY = B_WFULL + 2, B_DXFULL = B_WEMPTY + 2, B_DXEMPTY = B_DXFULL + NDX, B_DWFULL = B_DXEMPTY + NDX,
                       B_DWEMPTY = B_DWFULL + NDW, B_LEMPTY = B_DWEMPTY + NDW, B_FIN = B_LEMPTY + 2, NBAR = B_FIN + 2;
  static_assert(NBAR <= 40, "barrier space");
  static constexpr int N_EB = 8;                      // scatter warps: 4 TMEM lane quarters x 2 slot halves
  static constexpr int EBS = F / 2;                   // slots per scatter warp
  static constexpr int N_EC = 4;                      // dW writer warps: one per TMEM lane quarter
  static constexpr int N_Y = 8;                       // Y warps: one per row class (row index modulo 8)
  static constexpr int NPW = NXS;                     // X producer warps: 0, 2 and (at three stages) one after the Y warps
  static_assert(NPW <= NXS, "a producer must not run more than one phase ahead on any stage barrier");
  static constexpr int W_EB = 4, W_EC = W_EB + N_EB, W_Y = W_EC + N_EC, W_XP = W_Y + N_Y;
  static constexpr int NTHREADS = (W_XP + NPW - 2) * 32;
  static constexpr uint32_t TM_DX = 0, TM_DW = NDX * F, TM_COLS = 512;
  static_assert(TM_DW + NDW * FR <= TM_COLS, "TMEM budget");
  static constexpr int ROWS_PER_Q = G / 4;            // label rows of the dW accumulator in one TMEM lane quarter
};

struct BwdArgs {
  const int32_t* loc;
  const __nv_bfloat16* dy;
  float* dxt;
  __nv_bfloat16* dw;
  __nv_bfloat16* dbias;
  int* err;
  int64_t B, L, ldy;
  int D, NG;
  long long wait_limit;
};

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// DX / DW: which gradients this instantiation produces (the roles of the other one are compiled out: its issuer, its
// operand loads, its epilogue warps).  UPD (with DW): the dW writer warps apply SGD + weight decay (+ momentum) +
// stochastic rounding to the weights and bias in global memory instead of storing the gradient.
template <int G_, int F_, bool DX, bool DW, bool UPD>
__global__ void __launch_bounds__(Cfg<G_, F_>::NTHREADS, 1)
ffi_backward_sm100_kernel(BwdArgs a, UpdateArgs u, const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w) {
  static_assert(DX || DW, "nothing to compute");
  static_assert(!UPD || DW, "the update consumes the weight gradient");
  using C = Cfg<G_, F_>;
  constexpr int G = C::G, F = C::F, BT = C::BT, FR = C::FR, NXS = C::NXS, NYS = C::NYS, NDX = C::NDX, NDW = C::NDW;
  constexpr int XBLK = C::XBLK, XSTAGE = C::XSTAGE, WBLK = C::WBLK, WSTAGE = C::WSTAGE, YBLK = C::YBLK, YSTAGE = C::YSTAGE, NCH = C::NCH;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const uint32_t sbase = smem_u32(sm);
  uint32_t* loc_s = reinterpret_cast<uint32_t*>(sm + C::OFF_LOC);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + C::OFF_MISC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + C::OFF_MISC + 8);
  auto bar = [&](int i) { return sbase + C::OFF_BAR + i * 8; };
  const long long WL = a.wait_limit;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int T = static_cast<int>((a.B + BT - 1) / BT);

  if (tid == 0) {
    for (int i = 0; i < NXS; ++i) { mbar_init(bar(C::B_XFULL + i), 1); mbar_init(bar(C::B_XEMPTY + i), 1); }
    for (int i = 0; i < NYS; ++i) { mbar_init(bar(C::B_YFULL + i), C::N_Y); mbar_init(bar(C::B_YEMPTY + i), (DX ? 1 : 0) + (DW ? 1 : 0)); }   // every issuer commits
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(C::B_WFULL + i), 1);  mbar_init(bar(C::B_WEMPTY + i), 1);
      mbar_init(bar(C::B_LEMPTY + i), C::N_EB);      // the scatter warps are done with the group's index row
      mbar_init(bar(C::B_FIN + i), 1);
    }
    for (int i = 0; i < NDX; ++i) { mbar_init(bar(C::B_DXFULL + i), 1); mbar_init(bar(C::B_DXEMPTY + i), C::N_EB); }
    for (int i = 0; i < NDW; ++i) { mbar_init(bar(C::B_DWFULL + i), 1); mbar_init(bar(C::B_DWEMPTY + i), C::N_EC); }
    mbar_fence_init();
    *abort_flag = 0;
  }
  // rows F..FR-1 of every X block: row F = ones (bias-gradient column), the rest zeros; written once
  for (int i = tid; i < NXS * 2 * 16 * 8; i += C::NTHREADS) {
    const int chunk = i & 7, row = (i >> 3) & 15, blk = i >> 7;
    const uint32_t v = (row == 0) ? 0x3F803F80u : 0u;
    *reinterpret_cast<uint4*>(sm + C::OFF_X + blk * XBLK + (F + row) * 128 + chunk * 16) = make_uint4(v, v, v, v);
  }
  fence_proxy_async();
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), C::TM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const int n_my_groups = (a.NG > static_cast<int>(blockIdx.x)) ? (a.NG - 1 - static_cast<int>(blockIdx.x)) / static_cast<int>(gridDim.x) + 1 : 0;
  auto group_of = [&](int gi) { return static_cast<int>(blockIdx.x) + gi * static_cast<int>(gridDim.x); };

  const int prod_id = warp == 0 ? 0 : (warp == 2 ? 1 : (warp >= C::W_XP ? 2 + warp - C::W_XP : -1));
  if (prod_id >= 0) {
    // ================================================================ X / W producers
    // Per group: producer 0 writes the index row (as dxt row offsets for the scatter warps) and loads the W tile
    // through the tensor map.  Per batch tile: F index rows of xt, 256 bytes each, as TMA gather4 loads (four index
    // rows per instruction, landing at their swizzled positions), dealt round-robin over the four warps.
    int it = 0, w_armed = 0, my_last = -1;
    for (int gi = 0; gi < n_my_groups; ++gi) {
      const int g = group_of(gi);
      const int ws = gi & 1;
      const int64_t l0 = static_cast<int64_t>(g) * G;
      const int32_t* lrow = a.loc + static_cast<int64_t>(g) * F;
      int locv[F / 32];
#pragma unroll
      for (int j = 0; j < F / 32; ++j) locv[j] = min(max(__ldg(lrow + lane + 32 * j), 0), a.D - 1);   // clamped: never addresses outside xt / dxt
      if (DX && prod_id == 0) {
        bool ok = mbar_wait(bar(C::B_WEMPTY + ws), ((gi >> 1) & 1) ^ 1, abort_flag, a.err, 31, WL, 100);
        ok = mbar_wait(bar(C::B_LEMPTY + ws), ((gi >> 1) & 1) ^ 1, abort_flag, a.err, 31, WL, 100) && ok;
        __syncwarp();
#pragma unroll
        for (int j = 0; j < F / 32; ++j)
          loc_s[ws * F + lane + 32 * j] = static_cast<uint32_t>(locv[j]) * static_cast<uint32_t>(a.B);   // D * B < 2^32 is a launch condition
        __syncwarp();
        if (ok && !*abort_flag) {
          if (lane == 0) {
            // the arrival also releases the index row written above to the warps that wait for this barrier
            mbar_arrive_expect_tx(bar(C::B_WFULL + ws), WSTAGE);
#pragma unroll
            for (int kb = 0; kb < C::NWB; ++kb)
              tma_load_2d(sbase + C::OFF_W + ws * WSTAGE + kb * WBLK, &tm_w, kb * 64, static_cast<int>(l0), bar(C::B_WFULL + ws));
          }
          ++w_armed;
        }
        __syncwarp();
      }
      int* locr = reinterpret_cast<int*>(sm + C::OFF_LOCR) + prod_id * F;
      __syncwarp();
#pragma unroll
      for (int j = 0; j < F / 32; ++j) locr[lane + 32 * j] = locv[j];
      __syncwarp();
      const int4* lr4 = reinterpret_cast<const int4*>(locr);
      for (int t = 0; DW && t < T; ++t, ++it) {          // X is an operand of backward-weights only
        if (it % C::NPW != prod_id) continue;
        const int xs = it % NXS;
        const bool okx = mbar_wait(bar(C::B_XEMPTY + xs), ((it / NXS) & 1) ^ 1, abort_flag, a.err, 32, WL, 100);
        __syncwarp();
        if (!okx || *abort_flag) continue;
        const int b0 = t * BT;
        const uint32_t xb = sbase + C::OFF_X + xs * XSTAGE;
        if (lane == 0) mbar_arrive_expect_tx(bar(C::B_XFULL + xs), F * 256);
        __syncwarp();
#pragma unroll
        for (int i = lane; i < 2 * (F / 4); i += 32) {
          const int blk = i / (F / 4), r4 = i % (F / 4);
          const int4 lr = lr4[r4];
          tma_gather4(xb + blk * XBLK + r4 * 512, &tm_x, b0 + blk * 64, lr.x, lr.y, lr.z, lr.w, bar(C::B_XFULL + xs));
        }
        my_last = it;
      }
    }
    // every copy this warp started has to land before the CTA may exit (only the most recent use of each stage)
    for (int j = max(0, it - NXS); j < it; ++j)
      if (j % C::NPW == prod_id && j <= my_last) mbar_wait_final(bar(C::B_XFULL + j % NXS), (j / NXS) & 1, WL);
    for (int j = max(0, w_armed - 2); j < w_armed; ++j) mbar_wait_final(bar(C::B_WFULL + (j & 1)), (j >> 1) & 1, WL);
  } else if (warp >= C::W_Y && warp < C::W_XP) {
    // ================================================================ Y warps: dY slice -> aligned, swizzled Y tile
    // Warp k owns the rows r = k, k + 8, ... of every tile.  Copies run LAG tiles ahead of the shifting.
    const int k = warp - C::W_Y;
    constexpr int LAG = NYS - 1;                       // tiles between the start of a copy and its hand-over
    constexpr int PER_ROW = NCH + 1;
    constexpr int N_CP = 16 * PER_ROW;                 // copies per warp and tile
    const uintptr_t dy_base = reinterpret_cast<uintptr_t>(a.dy);
    const uintptr_t dy_end = dy_base + 2ull * static_cast<uint64_t>((a.B - 1) * a.ldy + a.L);   // first byte after the last gradient
    const int n_items = n_my_groups * T;
    const int rr = lane >> 3, c = lane & 7;            // shifting: lane = (row within a set of four, chunk within a 64-label block)
    int gi_i = 0, t_i = 0;                             // issue position
    int gi_p = 0, t_p = 0;                             // shift position
    // Order inside an iteration: first hand over the tile whose copies have landed (shift, then arrive), only then
    // wait for a free stage and start the next copies — a tile that is ready never waits for the tensor core to
    // finish an older one.
    for (int it = 0; it < n_items + LAG; ++it) {
      if (it >= LAG) {
        cp_async_wait<LAG - 1>();                      // this lane's copies of tile it - LAG have landed (groups 0 .. it-1 are committed)
        __syncwarp();                                  // ... and so have the other lanes'
        const int jt = it - LAG, ys = jt % NYS;
        const int64_t l0 = static_cast<int64_t>(group_of(gi_p)) * G;
        const int64_t b0 = static_cast<int64_t>(t_p) * BT;
        // all rows of this warp start at the same offset inside a 16-byte granule
        const uint32_t sh = static_cast<uint32_t>((dy_base + 2ull * static_cast<uint64_t>((b0 + k) * a.ldy + l0)) & 15u);
        const bool mask_cols = l0 + G > a.L;
        if ((sh != 0 || mask_cols) && !*abort_flag) {
          const uint32_t wo = sh >> 2, hb = (sh & 2u) << 3;     // whole words, then 0 or 16 bits
          uint8_t* yb = sm + C::OFF_Y + ys * YSTAGE;
          const uint8_t* yside = sm + C::OFF_YSIDE + ys * C::YSIDE;
          // (Unrolling this over the four row sets, so that their shared-memory latencies overlap, made the whole
          // kernel slower in measurement — aligned inputs included — and is therefore not done.)
#pragma unroll 1
          for (int set = 0; set < 4; ++set) {
            const int r = k + 8 * (4 * set + rr);
#pragma unroll
            for (int blk = 0; blk < C::NYB; ++blk) {           // ascending: chunk 8 is read (as a neighbour) before it is rewritten
              const int cj = blk * 8 + c;
              uint8_t* p = yb + blk * YBLK + r * 128 + ((c ^ (r & 7)) << 4);
              const uint8_t* pn = (cj + 1 == NCH) ? yside + r * 16
                                                  : yb + ((cj + 1) >> 3) * YBLK + r * 128 + ((((cj + 1) & 7) ^ (r & 7)) << 4);
              const uint4 v0 = *reinterpret_cast<const uint4*>(p);
              const uint4 v1 = *reinterpret_cast<const uint4*>(pn);
              __syncwarp();                            // every lane has read its neighbour's chunk before anyone rewrites one
              uint32_t w0, w1, w2, w3, w4;
              switch (wo) {                            // warp-uniform
                case 0: w0 = v0.x; w1 = v0.y; w2 = v0.z; w3 = v0.w; w4 = v1.x; break;
                case 1: w0 = v0.y; w1 = v0.z; w2 = v0.w; w3 = v1.x; w4 = v1.y; break;
                case 2: w0 = v0.z; w1 = v0.w; w2 = v1.x; w3 = v1.y; w4 = v1.z; break;
                default: w0 = v0.w; w1 = v1.x; w2 = v1.y; w3 = v1.z; w4 = v1.w; break;
              }
              uint4 o = make_uint4(__funnelshift_r(w0, w1, hb), __funnelshift_r(w1, w2, hb), __funnelshift_r(w2, w3, hb),
                                   __funnelshift_r(w3, w4, hb));
              if (mask_cols) {
                const int nv = static_cast<int>(a.L - l0) - 8 * cj;      // valid labels of this chunk
                if (nv < 8) {
                  o.x = nv >= 2 ? o.x : (nv == 1 ? (o.x & 0xFFFFu) : 0u);
                  o.y = nv >= 4 ? o.y : (nv == 3 ? (o.y & 0xFFFFu) : 0u);
                  o.z = nv >= 6 ? o.z : (nv == 5 ? (o.z & 0xFFFFu) : 0u);
                  o.w = nv == 7 ? (o.w & 0xFFFFu) : 0u;
                }
              }
              *reinterpret_cast<uint4*>(p) = o;
            }
          }
        }
        fence_proxy_async();                           // the tile as the tensor core will read it
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(C::B_YFULL + ys));
        if (++t_p == T) { t_p = 0; ++gi_p; }
      }
      if (it < n_items) {
        const int ys = it % NYS;
        const bool ok = mbar_wait(bar(C::B_YEMPTY + ys), ((it / NYS) & 1) ^ 1, abort_flag, a.err, 33, WL, 100);
        __syncwarp();
        if (ok && !*abort_flag) {
          const int64_t l0 = static_cast<int64_t>(group_of(gi_i)) * G;
          const int64_t b0 = static_cast<int64_t>(t_i) * BT;
          const uint32_t yb = sbase + C::OFF_Y + ys * YSTAGE, yside = sbase + C::OFF_YSIDE + ys * C::YSIDE;
#pragma unroll
          for (int j = 0; j < (N_CP + 31) / 32; ++j) {
            const int idx = lane + 32 * j;
            if (idx < N_CP) {
              const int ri = idx / PER_ROW, ch = idx % PER_ROW;
              const int r = k + 8 * ri;
              const int64_t b = b0 + r;
              const uintptr_t row_addr = dy_base + 2ull * static_cast<uint64_t>(b * a.ldy + l0);
              const uintptr_t src = (row_addr & ~static_cast<uintptr_t>(15)) + 16u * ch;
              // a chunk is read when it holds at least one byte of the tensor (it lies in the same 16-byte granule as
              // that byte); everything else is zero-filled
              const bool valid = b < a.B && src + 16 > dy_base && src < dy_end && (ch < NCH || (row_addr & 15) != 0);
              const uint32_t dst = ch < NCH ? yb + (ch >> 3) * YBLK + r * 128 + (((ch & 7) ^ (r & 7)) << 4) : yside + r * 16;
              cp_async16(dst, valid ? reinterpret_cast<const void*>(src) : reinterpret_cast<const void*>(dy_base & ~static_cast<uintptr_t>(15)), valid);
            }
          }
        }
        if (++t_i == T) { t_i = 0; ++gi_i; }
      }
      cp_async_commit();
    }
    cp_async_wait<0>();
  } else if (warp == 1 || warp == 3) {
    // ================================================================ MMA issuers (one elected lane each)
    constexpr uint32_t ID_BWX = make_idesc(128, F, 0, 1);
    constexpr uint32_t ID_BWW = make_idesc(G, FR, 1, 0);
    const uint64_t D_XB = make_sdesc(sbase + C::OFF_X, 16, 1024);      // X tile as K-major  B   (backward-weights)
    const uint64_t D_WM = make_sdesc(sbase + C::OFF_W, WBLK, 1024);    // W tile as MN-major B   (backward-features)
    const uint64_t D_YA = make_sdesc(sbase + C::OFF_Y, 16, 1024);      // Y tile as K-major  A   (backward-features)
    const uint64_t D_YM = make_sdesc(sbase + C::OFF_Y, YBLK, 1024);    // Y tile as MN-major A   (backward-weights)
    if (warp == 1 && DX) {
      const uint32_t wm_lo = static_cast<uint32_t>(D_WM), wm_hi = static_cast<uint32_t>(D_WM >> 32);
      const uint32_t ya_lo = static_cast<uint32_t>(D_YA), ya_hi = static_cast<uint32_t>(D_YA >> 32);
      const uint32_t id_bwx = ID_BWX;
      int it = 0, ys = 0, yph = 0;
      for (int gi = 0; gi < n_my_groups; ++gi) {
        const int ws = gi & 1;
        const bool okw = mbar_wait(bar(C::B_WFULL + ws), (gi >> 1) & 1, abort_flag, a.err, 34, WL);
        for (int t = 0; t < T; ++t, ++it) {
          const int ds = it % NDX;
          bool ok = mbar_wait(bar(C::B_YFULL + ys), yph, abort_flag, a.err, 35, WL) && okw;
          ok = mbar_wait(bar(C::B_DXEMPTY + ds), ((it / NDX) & 1) ^ 1, abort_flag, a.err, 36, WL) && ok;
          tc_fence_after();
          const uint32_t ya = ya_lo + static_cast<uint32_t>(ys) * (YSTAGE >> 4), wm = wm_lo + (ws ? (WSTAGE >> 4) : 0u);
          const uint32_t tdx = tmem + C::TM_DX + ds * F;
          // dXg[b,k] = sum over label chunks of Y[b, l-chunk] * W[l-chunk, k]
          if (ok && elect_one()) {
            umma_bf16_lohi<false>(tdx, ya, ya_hi, wm, wm_hi, id_bwx);
#pragma unroll
            for (int ks = 1; ks < G / 16; ++ks)
              umma_bf16_lohi<true>(tdx, ya + (((ks >> 2) * YBLK + (ks & 3) * 32) >> 4), ya_hi, wm + ((ks * 2048) >> 4), wm_hi, id_bwx);
            tc_commit(bar(C::B_DXFULL + ds));
            tc_commit(bar(C::B_YEMPTY + ys));
            if (t + 1 == T) tc_commit(bar(C::B_WEMPTY + ws));
          }
          __syncwarp();
          if (++ys == NYS) { ys = 0; yph ^= 1; }
        }
      }
      if (elect_one()) tc_commit(bar(C::B_FIN));
      __syncwarp();
      mbar_wait_final(bar(C::B_FIN), 0, WL);
    } else if (warp == 3 && DW) {
      const uint32_t xb_lo = static_cast<uint32_t>(D_XB), xb_hi = static_cast<uint32_t>(D_XB >> 32);
      const uint32_t ym_lo = static_cast<uint32_t>(D_YM), ym_hi = static_cast<uint32_t>(D_YM >> 32);
      const uint32_t id_bww = ID_BWW;
      int it = 0, xs = 0, xph = 0, ys = 0, yph = 0;
      for (int gi = 0; gi < n_my_groups; ++gi) {
        const int dws = gi % NDW;
        const uint32_t tdw = tmem + C::TM_DW + dws * FR;
        const bool okd = mbar_wait(bar(C::B_DWEMPTY + dws), ((gi / NDW) & 1) ^ 1, abort_flag, a.err, 37, WL);
        for (int t = 0; t < T; ++t, ++it) {
          bool ok = mbar_wait(bar(C::B_XFULL + xs), xph, abort_flag, a.err, 38, WL) && okd;
          ok = mbar_wait(bar(C::B_YFULL + ys), yph, abort_flag, a.err, 39, WL) && ok;
          tc_fence_after();
          const uint32_t ym = ym_lo + static_cast<uint32_t>(ys) * (YSTAGE >> 4), xb = xb_lo + static_cast<uint32_t>(xs) * (XSTAGE >> 4);
          // dW[l,k] += sum over batch chunks of Y[b-chunk, l]^T * X[k, b-chunk]
          if (ok && elect_one()) {
            umma_bf16_lohi_rt(tdw, ym, ym_hi, xb, xb_hi, id_bww, t > 0);
#pragma unroll
            for (int ks = 1; ks < BT / 16; ++ks)
              umma_bf16_lohi<true>(tdw, ym + ((ks * 2048) >> 4), ym_hi, xb + (((ks >> 2) * XBLK + (ks & 3) * 32) >> 4), xb_hi, id_bww);
            tc_commit(bar(C::B_YEMPTY + ys));
            tc_commit(bar(C::B_XEMPTY + xs));
            if (t + 1 == T) tc_commit(bar(C::B_DWFULL + dws));
          }
          __syncwarp();
          if (++xs == NXS) { xs = 0; xph ^= 1; }
          if (++ys == NYS) { ys = 0; yph ^= 1; }
        }
      }
      if (elect_one()) tc_commit(bar(C::B_FIN + 1));
      __syncwarp();
      mbar_wait_final(bar(C::B_FIN + 1), 0, WL);
    }
  } else if (DX && warp >= C::W_EB && warp < C::W_EC) {
    // ================================================================ scatter: dXg -> dxt
    const int q = warp & 3, kc = (warp - C::W_EB) >> 2;
    const int row = q * 32 + lane;               // TMEM lane == batch row inside the tile
    int it = 0;
    for (int gi = 0; gi < n_my_groups; ++gi) {
      const int ws = gi & 1;
      mbar_wait(bar(C::B_WFULL + ws), (gi >> 1) & 1, abort_flag, a.err, 40, WL);   // loc_s of this group is in place
      const uint4* loc4 = reinterpret_cast<const uint4*>(loc_s + ws * F + kc * C::EBS);
      for (int t = 0; t < T; ++t, ++it) {
        const int b0 = t * BT;
        const int ds = it % NDX;
        mbar_wait(bar(C::B_DXFULL + ds), (it / NDX) & 1, abort_flag, a.err, 41, WL);
        tc_fence_after();
        const uint32_t ta = tmem + (static_cast<uint32_t>(q * 32) << 16) + C::TM_DX + ds * F + kc * C::EBS;
        // for a fixed slot the warp's 32 lanes hit 32 consecutive floats of one dxt row: one 128-byte reduction
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
              const uint4 lc = loc4[half * 8 + (k4 >> 2)];
              atomicAdd(dbase + lc.x, __uint_as_float(r0[k4 + 0]));
              atomicAdd(dbase + lc.y, __uint_as_float(r0[k4 + 1]));
              atomicAdd(dbase + lc.z, __uint_as_float(r0[k4 + 2]));
              atomicAdd(dbase + lc.w, __uint_as_float(r0[k4 + 3]));
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(C::B_LEMPTY + ws));
    }
  } else if (DW && warp >= C::W_EC && warp < C::W_Y) {
    // ================================================================ dW / dbias rows out of the accumulator
    // G = 128: TMEM lane == label row, every lane takes its row's 32 columns of each piece.  G = 64: an M = 64
    // accumulator occupies lanes 0-15 of each lane quarter, so lane l and lane l + 16 share label row l: the upper 16
    // columns of every 32-column piece go to lane l + 16 by shuffle and the whole warp works.
    constexpr bool SPLIT = C::ROWS_PER_Q == 16;
    constexpr int NCL = SPLIT ? 2 : 4;              // 8-slot chunks per lane and piece
    const int q = warp & 3;
    const int half = SPLIT ? (lane >> 4) : 0;
    const int row = q * C::ROWS_PER_Q + (lane & (C::ROWS_PER_Q - 1));
    for (int gi = 0; gi < n_my_groups; ++gi) {
      const int g = group_of(gi);
      const int dws = gi % NDW;
      const int64_t l0 = static_cast<int64_t>(g) * G;
      const int rows_real = static_cast<int>(imin64(G, a.L - l0));
      mbar_wait(bar(C::B_DWFULL + dws), (gi / NDW) & 1, abort_flag, a.err, 42, WL);
      tc_fence_after();
      const uint32_t ta = tmem + (static_cast<uint32_t>(q * 32) << 16) + C::TM_DW + dws * FR;
      const bool do_row = row < rows_real && !*abort_flag;
      const int64_t l = l0 + row, gl = u.label0 + l;
      const bool fast = UPD && u.mom_w == nullptr && (u.flags & HASTE_F_SR) && (u.flags & HASTE_F_CONTRACT);
#pragma unroll
      for (int pc = 0; pc < F / 32; ++pc) {
        uint32_t r0[32];
        __syncwarp();
        tmem_ld32(ta + pc * 32, r0);
        tmem_ld_wait();
        if (SPLIT) {
#pragma unroll
          for (int x = 0; x < 16; ++x) {
            const uint32_t up = __shfl_sync(0xffffffffu, r0[16 + x], lane & 15);
            if (half) r0[x] = up;
          }
        }
        if (do_row) {
#pragma unroll
          for (int c4 = 0; c4 < NCL; ++c4) {
            const int s0 = pc * 32 + half * 16 + c4 * 8;        // first of this chunk's 8 slots
            uint4* out = reinterpret_cast<uint4*>((UPD ? u.w : a.dw) + l * F + s0);
            // the gradient as the unfused kernel would store it: rounded to bf16
            const uint4 g8 = make_uint4(pack2(__uint_as_float(r0[8 * c4]), __uint_as_float(r0[8 * c4 + 1])),
                                        pack2(__uint_as_float(r0[8 * c4 + 2]), __uint_as_float(r0[8 * c4 + 3])),
                                        pack2(__uint_as_float(r0[8 * c4 + 4]), __uint_as_float(r0[8 * c4 + 5])),
                                        pack2(__uint_as_float(r0[8 * c4 + 6]), __uint_as_float(r0[8 * c4 + 7])));
            if (!UPD) {
              *out = g8;
            } else {
              const uint4 w8 = *out;
              const uint32_t gw[4] = {g8.x, g8.y, g8.z, g8.w}, ww[4] = {w8.x, w8.y, w8.z, w8.w};
              uint32_t rnd[4] = {0u, 0u, 0u, 0u};               // 8 x 16 random bits, two per word
              if (u.flags & HASTE_F_SR) {
                if (u.flags & HASTE_F_RNG_PACKED) {
                  const uint4 rp = rand_packed8(u.seed, u.step, gl, s0 >> 3);
                  rnd[0] = rp.x; rnd[1] = rp.y; rnd[2] = rp.z; rnd[3] = rp.w;
                } else {
#pragma unroll
                  for (int x = 0; x < 4; ++x)
                    rnd[x] = rand16_reference(u.seed, gl * F + s0 + 2 * x) | (rand16_reference(u.seed, gl * F + s0 + 2 * x + 1) << 16);
                }
              }
              uint32_t ob[4];
              if (fast) {
                // no momentum, stochastic rounding, fused multiply-add: w' = fma(-lr, fma(wd, w, g), w), then add 16
                // random bits and keep the high half
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                  const float g0 = __uint_as_float(gw[x] << 16), g1 = __uint_as_float(gw[x] & 0xFFFF0000u);
                  const float w0 = __uint_as_float(ww[x] << 16), w1 = __uint_as_float(ww[x] & 0xFFFF0000u);
                  const float n0 = __fmaf_rn(-u.lr, __fmaf_rn(u.wd, w0, g0), w0), n1 = __fmaf_rn(-u.lr, __fmaf_rn(u.wd, w1, g1), w1);
                  ob[x] = __byte_perm(__float_as_uint(n0) + (rnd[x] & 0xFFFFu), __float_as_uint(n1) + (rnd[x] >> 16), 0x7632);
                }
              } else {
                float* mrow = u.mom_w != nullptr ? u.mom_w + l * F + s0 : nullptr;
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                  float m0 = 0.f, m1 = 0.f;
                  if (mrow) { m0 = mrow[2 * x]; m1 = mrow[2 * x + 1]; }
                  const uint32_t o0 = sgd_update_bits(static_cast<uint16_t>(ww[x] & 0xFFFFu), __uint_as_float(gw[x] << 16), mrow ? &m0 : nullptr,
                                                      u.lr, u.wd, u.mu, u.flags, rnd[x] & 0xFFFFu);
                  const uint32_t o1 = sgd_update_bits(static_cast<uint16_t>(ww[x] >> 16), __uint_as_float(gw[x] & 0xFFFF0000u),
                                                      mrow ? &m1 : nullptr, u.lr, u.wd, u.mu, u.flags, rnd[x] >> 16);
                  ob[x] = o0 | (o1 << 16);
                  if (mrow) { mrow[2 * x] = m0; mrow[2 * x + 1] = m1; }
                }
              }
              *out = make_uint4(ob[0], ob[1], ob[2], ob[3]);
            }
          }
        }
      }
      uint32_t rb[8];
      __syncwarp();
      tmem_ld8(ta + F, rb);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(C::B_DWEMPTY + dws));
      if (half == 0) {
        if (!UPD) {
          if (do_row && a.dbias != nullptr) a.dbias[l] = __float2bfloat16_rn(__uint_as_float(rb[0]));
        } else if (do_row && u.bias != nullptr) {
          const float gb = round_to_bf16_f(__uint_as_float(rb[0]));
          uint32_t r16 = 0;
          if (u.flags & HASTE_F_SR) r16 = rand16(u.flags, u.seed ^ ((u.flags & HASTE_F_RNG_PACKED) ? 0x62696173ull : 0ull), u.step, gl, 0, 1);
          float m = u.mom_b != nullptr ? u.mom_b[l] : 0.f;
          u.bias[l] = __ushort_as_bfloat16(sgd_update_bits(__bfloat16_as_ushort(u.bias[l]), gb, u.mom_b != nullptr ? &m : nullptr, u.lr, u.wd,
                                                           u.mu, u.flags, r16));
          if (u.mom_b != nullptr) u.mom_b[l] = m;
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, C::TM_COLS);
}

template <int G_, int F_>
static int launch_shape(const void* xt, const void* w, const int32_t* loc, const void* dy, float* dxt, void* dw, void* dbias,
                        const UpdateArgs* upd, int64_t B, int64_t D, int64_t L, int64_t ldy, cudaStream_t st) {
  using C = Cfg<G_, F_>;
  if (int rc = report_pending_status("tcgen05 backward")) return rc;
  int* err_dev = nullptr;
  if (int rc = device_status_word(&err_dev)) return rc;
  const bool want_dx = dxt != nullptr, want_dw = dw != nullptr || upd != nullptr;
  BwdArgs a;
  a.loc = loc; a.dy = static_cast<const __nv_bfloat16*>(dy); a.dxt = dxt; a.dw = static_cast<__nv_bfloat16*>(dw);
  a.dbias = static_cast<__nv_bfloat16*>(dbias); a.err = err_dev;
  a.B = B; a.L = L; a.ldy = ldy; a.D = static_cast<int>(D); a.NG = static_cast<int>((L + C::G - 1) / C::G);
  a.wait_limit = wait_limit_cycles();
  UpdateArgs u{};
  if (upd) u = *upd;
  // a gradient that is not asked for needs neither its operand nor that operand's tensor map (the kernel never uses it)
  CUtensorMap tm_x, tm_w;
  const void* w_map = want_dx ? w : xt;
  const void* x_map = want_dw ? xt : w;
  if (want_dw) { if (int rc = make_tmap_bf16_2d(&tm_x, x_map, static_cast<uint64_t>(B), static_cast<uint64_t>(D), static_cast<uint64_t>(B) * 2, 64, 1)) return rc; }
  if (want_dx) { if (int rc = make_tmap_bf16_2d(&tm_w, w_map, static_cast<uint64_t>(C::F), static_cast<uint64_t>(L), static_cast<uint64_t>(C::F) * 2, 64, C::G)) return rc; }
  if (!want_dw) tm_x = tm_w;
  if (!want_dx) tm_w = tm_x;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = a.NG < sms ? a.NG : sms;
#define HASTE_B100_LAUNCH(DXF, DWF, UPDF)                                                                     \
  {                                                                                                          \
    auto k = ffi_backward_sm100_kernel<G_, F_, DXF, DWF, UPDF>;                                              \
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);     \
    if (e != cudaSuccess) return fail(HASTE_ERR_LAUNCH, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));  \
    k<<<grid, C::NTHREADS, C::SMEM_BYTES, st>>>(a, u, tm_x, tm_w);                                           \
  }
  if (want_dx && want_dw && !upd) HASTE_B100_LAUNCH(true, true, false)
  else if (want_dx && !want_dw) HASTE_B100_LAUNCH(true, false, false)
  else if (!want_dx && want_dw && !upd) HASTE_B100_LAUNCH(false, true, false)
  else if (!want_dx && upd) HASTE_B100_LAUNCH(false, true, true)
  else return fail(HASTE_ERR_UNSUPPORTED, "tcgen05 backward: this combination of outputs has no instantiation");
#undef HASTE_B100_LAUNCH
  return check_launch("ffi_backward_sm100_kernel");
}

}  // namespace b100

// xt / w / dw may be NULL when the gradient that needs them is not asked for.
bool backward_sm100_supported(const void* xt, const void* w, const void* dy, const void* dw, int64_t B, int64_t D, int64_t F, int64_t L,
                              int64_t G) {
  // tensor maps need 16-byte aligned bases and row strides; dxt row offsets and tile coordinates are 32-bit; dy only
  // needs its natural 2-byte alignment
  return ((G == 128 && F == 64) || (G == 64 && F == 128)) && (B % 8) == 0 && aligned16(xt) && aligned16(w) && aligned16(dw) &&
         (reinterpret_cast<uintptr_t>(dy) & 1u) == 0 && D * B < (int64_t(1) << 32) && L < (int64_t(1) << 31) && B < (int64_t(1) << 31);
}

// dxt == NULL: weight gradient only; dw == NULL and upd == NULL: feature gradient only; upd != NULL (with dxt == NULL):
// backward-weights fused with the update of upd->w / upd->bias.
int launch_backward_sm100(const void* xt, const void* w, const int32_t* loc, const void* dy, float* dxt, void* dw, void* dbias,
                          const UpdateArgs* upd, int64_t B, int64_t D, int64_t F, int64_t L, int64_t G, int64_t ldy, cudaStream_t st) {
  if (G == 128 && F == 64) return b100::launch_shape<128, 64>(xt, w, loc, dy, dxt, dw, dbias, upd, B, D, L, ldy, st);
  if (G == 64 && F == 128) return b100::launch_shape<64, 128>(xt, w, loc, dy, dxt, dw, dbias, upd, B, D, L, ldy, st);
  return fail(HASTE_ERR_UNSUPPORTED, "tcgen05 backward: no kernel for group size %lld, fan-in %lld", (long long)G, (long long)F);
}

}  // namespace haste
