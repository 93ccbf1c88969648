// Forward gather-GEMM of the FFI layer on tcgen05 / TMEM, for the layer shapes (group size 128, fan-in 64) and
// (group size 64, fan-in 128):
//     z[b, l] = sum_k xt[loc[l/G, k], b] * w[l, k] + bias[l]        (bf16 in, fp32 accumulate, bf16 out)
// This is the unfused forward of the autograd surface: it has to write the [B, L] logits, so it is bound by
// that HBM write (2*B*L bytes), not by the tensor pipe.
//
// Persistent, one CTA per SM, groups g = blockIdx.x, += gridDim.x; per group the batch is walked in 128-row
// tiles.  Same shared-memory operand layout as the fused train step (128-byte-swizzled row blocks; X tile as
// MN-major A with a row of ones under the gathered rows, W tile as K-major B, the bias as one more K step).
// Everything that moves a tile is a TMA copy: the W tile through a 2-D tensor map, the X rows by tile::gather4
// from four producer warps (the gather rate grows with the number of issuing warps), and the logits leave
// through a tensor-map store from a swizzled staging tile, which also clips the ragged last group and the
// ragged last batch tile (in whole 16-byte chunks: the store's extent is the writable width rounded down to 8
// columns, and the up to 7 columns left over are written with ordinary 2-byte stores).  Warp roles (416 threads): warps 0, 2, 3, 12 produce, warp 1 issues the MMAs,
// warps 4-11 drain the accumulator: TMEM -> bf16 -> staging tile; one thread issues the store.
// All waits are bounded (see mbar_wait).
#include "common.cuh"
#include "launchers.h"
#include "runtime.h"
#include "sm100.cuh"

namespace haste {
namespace f100 {
using namespace sm100;

template <int G_, int F_>
struct Cfg {
  static constexpr int G = G_, F = F_, BT = 128;
  static_assert((G == 128 && F == 64) || (G == 64 && F == 128), "shapes with a tcgen05 forward");
  static constexpr int FR = F + 16;                   // rows of an X block: F gathered rows, one row of ones, 15 zero rows
  static constexpr int NXS = (F == 64) ? 5 : 4;       // X ring stages
  static constexpr int XBLK = FR * 128;               // one 64-batch block of an X stage (bytes)
  static constexpr int XSTAGE = 2 * XBLK;
  static constexpr int NWB = F / 64;                  // 64-slot blocks of a W stage
  static constexpr int WBLK = G * 128;
  static constexpr int WSTAGE = NWB * WBLK;
  static constexpr int NCB = G / 64;                  // 64-label blocks of a staging tile
  static constexpr int CBLK = BT * 128;
  static constexpr int CSTAGE = NCB * CBLK;
  static constexpr int BTILE = G * 32;                // bias tile: G rows x 16 bf16, no swizzle
  static constexpr int OFF_X = 0;
  static constexpr int OFF_W = OFF_X + NXS * XSTAGE;
  static constexpr int OFF_C = OFF_W + 2 * WSTAGE;
  static constexpr int OFF_BT = OFF_C + 2 * CSTAGE;
  static constexpr int OFF_LOCR = OFF_BT + 2 * BTILE;          // int [4][F]: each producer warp's copy of the group's (clamped) indices
  static constexpr int OFF_BAR = OFF_LOCR + 4 * F * 4;
  static constexpr int OFF_MISC = OFF_BAR + 32 * 8;
  static constexpr int SMEM_BYTES = OFF_MISC + 64 + 1024;
  static_assert(SMEM_BYTES <= 232448, "shared memory budget");
  static_assert(XSTAGE % 1024 == 0 && WBLK % 1024 == 0 && CBLK % 1024 == 0 && OFF_BT % 128 == 0, "tile alignment");
  static constexpr int B_XFULL = 0, B_XEMPTY = NXS, B_WFULL = 2 * NXS, B_WEMPTY = B_WFULL + 2, B_ZFULL = B_WEMPTY + 2,
                       B_ZEMPTY = B_ZFULL + 2, B_FIN = B_ZEMPTY + 2, NBAR = B_FIN + 1;
  static_assert(NBAR <= 32, "barrier space");
  static constexpr int N_EPI = 8;                     // epilogue warps: 4 TMEM lane quarters x 2 column halves
  static constexpr int EC = G / 2;                    // label columns of a tile drained by one epilogue warp
  static constexpr int NPW = 4;                       // producer warps: 0, 2, 3 and the warp after the epilogue warps
  static_assert(NPW <= NXS, "a producer must not run more than one phase ahead on any stage barrier");
  static constexpr int W_EPI = 4, W_XP = W_EPI + N_EPI;
  static constexpr int NTHREADS = (W_XP + 1) * 32;
  static constexpr uint32_t TM_COLS = 2 * G;          // two accumulator stages
};

struct FwdArgs {
  const int32_t* loc;
  const __nv_bfloat16* bias;
  __nv_bfloat16* z;
  int* err;
  int64_t B, L, ldz, zw;
  int D, NG;
  long long wait_limit;
};

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int G_, int F_>
__global__ void __launch_bounds__(Cfg<G_, F_>::NTHREADS, 1)
ffi_forward_sm100_kernel(FwdArgs a, const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w,
                         const __grid_constant__ CUtensorMap tm_z) {
  using C = Cfg<G_, F_>;
  constexpr int G = C::G, F = C::F, BT = C::BT, NXS = C::NXS, XBLK = C::XBLK, XSTAGE = C::XSTAGE, WBLK = C::WBLK, WSTAGE = C::WSTAGE;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const uint32_t sbase = smem_u32(sm);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + C::OFF_MISC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + C::OFF_MISC + 8);
  auto bar = [&](int i) { return sbase + C::OFF_BAR + i * 8; };
  const long long WL = a.wait_limit;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int T = static_cast<int>((a.B + BT - 1) / BT);

  if (tid == 0) {
    for (int i = 0; i < NXS; ++i) { mbar_init(bar(C::B_XFULL + i), 1); mbar_init(bar(C::B_XEMPTY + i), 1); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(C::B_WFULL + i), 1);  mbar_init(bar(C::B_WEMPTY + i), 1);
      mbar_init(bar(C::B_ZFULL + i), 1);  mbar_init(bar(C::B_ZEMPTY + i), C::N_EPI);
    }
    mbar_init(bar(C::B_FIN), 1);
    mbar_fence_init();
    *abort_flag = 0;
  }
  // rows F..F+15 of every X block: row F = ones (times the bias column = the bias), the rest zeros; written once
  for (int i = tid; i < NXS * 2 * 16 * 8; i += C::NTHREADS) {
    const int chunk = i & 7, row = (i >> 3) & 15, blk = i >> 7;
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
  const int n_my_groups = (a.NG > static_cast<int>(blockIdx.x)) ? (a.NG - 1 - static_cast<int>(blockIdx.x)) / static_cast<int>(gridDim.x) + 1 : 0;

  const int prod_id = warp == 0 ? 0 : (warp == 2 ? 1 : (warp == 3 ? 2 : (warp == C::W_XP ? 3 : -1)));
  if (prod_id >= 0) {
    // ================================================================ producers
    // Producer 0 also loads every group's W tile and writes its bias column; the X tiles (one per batch tile) are
    // dealt round-robin over the four warps.  Lane 0 arms the stage's barrier with the byte count, then every lane
    // issues its share of the gathers (four index rows per instruction, landing at their swizzled positions).
    int it = 0, w_armed = 0, my_last = -1;
    for (int gi = 0; gi < n_my_groups; ++gi) {
      const int g = blockIdx.x + gi * gridDim.x;
      const int ws = gi & 1;
      const int64_t l0 = static_cast<int64_t>(g) * G;
      const int rows_real = static_cast<int>(imin64(G, a.L - l0));
      const int32_t* lrow = a.loc + static_cast<int64_t>(g) * F;
      int locv[F / 32];
#pragma unroll
      for (int j = 0; j < F / 32; ++j) locv[j] = min(max(__ldg(lrow + lane + 32 * j), 0), a.D - 1);   // clamped: never addresses outside xt
      if (prod_id == 0) {
        uint16_t bv[G / 32];
#pragma unroll
        for (int j = 0; j < G / 32; ++j) {
          const int c = lane + 32 * j;
          bv[j] = (a.bias != nullptr && c < rows_real) ? __bfloat16_as_ushort(a.bias[l0 + c]) : uint16_t(0);
        }
        const bool ok = mbar_wait(bar(C::B_WEMPTY + ws), ((gi >> 1) & 1) ^ 1, abort_flag, a.err, 21, WL, 100);
        __syncwarp();
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
      int* locr = reinterpret_cast<int*>(sm + C::OFF_LOCR) + prod_id * F;
      __syncwarp();
#pragma unroll
      for (int j = 0; j < F / 32; ++j) locr[lane + 32 * j] = locv[j];
      __syncwarp();
      const int4* lr4 = reinterpret_cast<const int4*>(locr);
      for (int t = 0; t < T; ++t, ++it) {
        if (it % C::NPW != prod_id) continue;
        const int xs = it % NXS;
        const bool okx = mbar_wait(bar(C::B_XEMPTY + xs), ((it / NXS) & 1) ^ 1, abort_flag, a.err, 22, WL, 100);
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
    // every copy this warp started has to land before the CTA may exit (only the most recent use of each stage:
    // an older phase of the same barrier can no longer be waited for)
    for (int j = max(0, it - NXS); j < it; ++j)
      if (j % C::NPW == prod_id && j <= my_last) mbar_wait_final(bar(C::B_XFULL + j % NXS), (j / NXS) & 1, WL);
    for (int j = max(0, w_armed - 2); j < w_armed; ++j) mbar_wait_final(bar(C::B_WFULL + (j & 1)), (j >> 1) & 1, WL);
  } else if (warp == 1) {
    // ================================================================ MMA issuer
    // The warp runs its control flow converged; one elected lane issues the products and commits (descriptors stay
    // in uniform registers this way).
    constexpr uint32_t ID_FWD = make_idesc(128, G, 1, 0);
    const uint64_t D_XA = make_sdesc(sbase + C::OFF_X, XBLK, 1024);            // X tile as MN-major A
    const uint64_t D_WB = make_sdesc(sbase + C::OFF_W, 16, 1024);              // W tile as K-major B
    const uint64_t D_BB = make_sdesc_noswizzle(sbase + C::OFF_BT, 128, 256);   // bias tile as K-major B (last K step)
    const uint32_t xa_lo = static_cast<uint32_t>(D_XA), xa_hi = static_cast<uint32_t>(D_XA >> 32);
    const uint32_t wb_lo = static_cast<uint32_t>(D_WB), wb_hi = static_cast<uint32_t>(D_WB >> 32);
    const uint32_t bb_lo = static_cast<uint32_t>(D_BB), bb_hi = static_cast<uint32_t>(D_BB >> 32);
    const uint32_t id_fwd = ID_FWD;
    int it = 0, xs = 0, xph = 0;
    for (int gi = 0; gi < n_my_groups; ++gi) {
      const int ws = gi & 1;
      const bool okw = mbar_wait(bar(C::B_WFULL + ws), (gi >> 1) & 1, abort_flag, a.err, 23, WL);
      for (int t = 0; t < T; ++t, ++it) {
        const int zs = it & 1;
        bool ok = mbar_wait(bar(C::B_XFULL + xs), xph, abort_flag, a.err, 24, WL) && okw;
        ok = mbar_wait(bar(C::B_ZEMPTY + zs), ((it >> 1) & 1) ^ 1, abort_flag, a.err, 25, WL) && ok;
        tc_fence_after();
        const uint32_t xa = xa_lo + static_cast<uint32_t>(xs) * (XSTAGE >> 4), wb = wb_lo + (ws ? (WSTAGE >> 4) : 0u);
        const uint32_t bb = bb_lo + (ws ? (C::BTILE >> 4) : 0u);
        const uint32_t tz = tmem + zs * G;
        if (ok && elect_one()) {          // after an abort nothing more is issued
          umma_bf16_lohi<false>(tz, xa, xa_hi, wb, wb_hi, id_fwd);
#pragma unroll
          for (int ks = 1; ks < F / 16; ++ks)
            umma_bf16_lohi<true>(tz, xa + ((ks * 2048) >> 4), xa_hi, wb + (((ks >> 2) * WBLK + (ks & 3) * 32) >> 4), wb_hi, id_fwd);
          umma_bf16_lohi<true>(tz, xa + (((F / 16) * 2048) >> 4), xa_hi, bb, bb_hi, id_fwd);
          tc_commit(bar(C::B_ZFULL + zs));
          tc_commit(bar(C::B_XEMPTY + xs));
          if (t + 1 == T) tc_commit(bar(C::B_WEMPTY + ws));
        }
        __syncwarp();
        if (++xs == NXS) { xs = 0; xph ^= 1; }
      }
    }
    // every product this warp issued has completed before the CTA tears down its TMEM
    if (elect_one()) tc_commit(bar(C::B_FIN));
    __syncwarp();
    mbar_wait_final(bar(C::B_FIN), 0, WL);
  } else {
    // ================================================================ epilogue
    // TMEM -> bf16 -> staging tile (row blocks of 128 bytes, 16-byte chunk index XORed with (row & 7): the layout
    // the tensor map's 128-byte swizzle expects, and conflict-free for these row-per-thread writes) -> one TMA
    // store per 64-label block.  Two staging buffers: the store of tile i is read out of shared memory while
    // tile i + 1 is drained into the other buffer.
    const int ep = warp - C::W_EPI;
    const int q = ep & 3, h = ep >> 2;                       // TMEM lane quarter (= warp index mod 4), column half
    const int row = q * 32 + lane;
    const bool storer = (ep == 0 && lane == 0);
    int it = 0;
    for (int gi = 0; gi < n_my_groups; ++gi) {
      const int g = blockIdx.x + gi * gridDim.x;
      const int l0 = g * G;
      for (int t = 0; t < T; ++t, ++it) {
        const int zs = it & 1;
        const bool ok = mbar_wait(bar(C::B_ZFULL + zs), (it >> 1) & 1, abort_flag, a.err, 27, WL);
        tc_fence_after();
        const uint32_t ta = tmem + (static_cast<uint32_t>(q * 32) << 16) + zs * G + h * C::EC;
        // the store that last read this staging buffer (two tiles ago) has finished reading: the storing thread
        // waited for that before it arrived here
        named_bar_sync(1, C::N_EPI * 32);
        uint8_t* crow = sm + C::OFF_C + zs * C::CSTAGE + (G == 128 ? h * C::CBLK : 0) + row * 128;
        const int chunk0 = (G == 128) ? 0 : h * (C::EC / 8);
#pragma unroll 1
        for (int c16 = 0; c16 < C::EC; c16 += 16) {
          uint32_t r[16];
          __syncwarp();
          tmem_ld16(ta + c16, r);
          tmem_ld_wait();
#pragma unroll
          for (int e8 = 0; e8 < 16; e8 += 8) {
            const uint4 v = make_uint4(pack2(__uint_as_float(r[e8 + 0]), __uint_as_float(r[e8 + 1])),
                                       pack2(__uint_as_float(r[e8 + 2]), __uint_as_float(r[e8 + 3])),
                                       pack2(__uint_as_float(r[e8 + 4]), __uint_as_float(r[e8 + 5])),
                                       pack2(__uint_as_float(r[e8 + 6]), __uint_as_float(r[e8 + 7])));
            const int chunk = chunk0 + ((c16 + e8) >> 3);         // 0..7 inside the 128-byte row
            *reinterpret_cast<uint4*>(crow + ((chunk ^ (row & 7)) << 4)) = v;
          }
        }
        tc_fence_before();
        fence_proxy_async();                                  // the staging writes become visible to the TMA store
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(C::B_ZEMPTY + zs));
        named_bar_sync(2, C::N_EPI * 32);                     // the whole staging tile is written
        if (storer) {
          if (ok && !*abort_flag) {
#pragma unroll
            for (int cb = 0; cb < C::NCB; ++cb)
              tma_store_2d(&tm_z, sbase + C::OFF_C + zs * C::CSTAGE + cb * C::CBLK, l0 + cb * 64, t * BT);
          }
          bulk_commit();
          bulk_wait_read<1>();                                // the previous tile's store has left its buffer
        }
        // The tensor-map store writes whole 16-byte chunks.  When the writable width is not a multiple of 8 columns,
        // its last columns (they lie in the last group) come out of the staging tile with 2-byte stores, one batch
        // row per thread.  The buffer is not rewritten before these threads pass the next tile's first barrier.
        const int tail0 = static_cast<int>(a.zw & ~int64_t(7)), tail_n = static_cast<int>(a.zw - tail0);
        if (tail_n > 0 && h == 0 && tail0 >= l0 && tail0 < l0 + G && ok && !*abort_flag && t * BT + row < a.B) {
          const int tc = (tail0 - l0) >> 3;                   // chunk index inside the group's row
          const uint4 v = *reinterpret_cast<const uint4*>(sm + C::OFF_C + zs * C::CSTAGE + (tc >> 3) * C::CBLK + row * 128 +
                                                          (((tc & 7) ^ (row & 7)) << 4));
          const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
          uint16_t* dst = reinterpret_cast<uint16_t*>(a.z) + (static_cast<int64_t>(t) * BT + row) * a.ldz + tail0;
#pragma unroll
          for (int i = 0; i < 7; ++i)
            if (i < tail_n) dst[i] = static_cast<uint16_t>(w4[i >> 1] >> ((i & 1) * 16));
        }
      }
    }
    if (storer) bulk_wait<0>();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, C::TM_COLS);
}

template <int G_, int F_>
static int launch_shape(const int32_t* loc, const void* xt, const void* w, const void* bias, void* z, int64_t B, int64_t D, int64_t L,
                        int64_t ldz, int64_t zw, cudaStream_t st) {
  using C = Cfg<G_, F_>;
  if (int rc = report_pending_status("tcgen05 forward")) return rc;
  int* err_dev = nullptr;
  if (int rc = device_status_word(&err_dev)) return rc;
  FwdArgs a;
  a.loc = loc; a.bias = static_cast<const __nv_bfloat16*>(bias); a.z = static_cast<__nv_bfloat16*>(z); a.err = err_dev;
  a.B = B; a.L = L; a.ldz = ldz; a.zw = zw; a.D = static_cast<int>(D); a.NG = static_cast<int>((L + C::G - 1) / C::G);
  a.wait_limit = wait_limit_cycles();
  CUtensorMap tm_x, tm_w, tm_z;
  if (int rc = make_tmap_bf16_2d(&tm_x, xt, static_cast<uint64_t>(B), static_cast<uint64_t>(D), static_cast<uint64_t>(B) * 2, 64, 1)) return rc;
  if (int rc = make_tmap_bf16_2d(&tm_w, w, static_cast<uint64_t>(C::F), static_cast<uint64_t>(L), static_cast<uint64_t>(C::F) * 2, 64, C::G)) return rc;
  // the store clips at the writable width, in whole 16-byte chunks (columns L..zw-1 of the last group receive the
  // zeros its absent weight rows produce); the kernel writes the remaining zw % 8 columns itself
  if (zw < 8) return fail(HASTE_ERR_UNSUPPORTED, "tcgen05 forward: writable width below 8 columns");
  if (int rc = make_tmap_bf16_2d(&tm_z, z, static_cast<uint64_t>(zw & ~int64_t(7)), static_cast<uint64_t>(B), static_cast<uint64_t>(ldz) * 2, 64, C::BT)) return rc;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = a.NG < sms ? a.NG : sms;
  auto k = ffi_forward_sm100_kernel<G_, F_>;
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
  if (e != cudaSuccess) return fail(HASTE_ERR_LAUNCH, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  k<<<grid, C::NTHREADS, C::SMEM_BYTES, st>>>(a, tm_x, tm_w, tm_z);
  return check_launch("ffi_forward_sm100_kernel");
}

}  // namespace f100

bool forward_sm100_supported(const void* z, const void* xt, const void* w, int64_t B, int64_t F, int64_t L, int64_t G, int64_t ldz) {
  // tensor maps need 16-byte aligned bases and row strides; coordinates are 32-bit
  return ((G == 128 && F == 64) || (G == 64 && F == 128)) && (B % 8) == 0 && (ldz % 8) == 0 && aligned16(z) && aligned16(xt) &&
         aligned16(w) && L < (int64_t(1) << 31) && B < (int64_t(1) << 31);
}

int launch_forward_sm100(const int32_t* loc, const void* xt, const void* w, const void* bias, void* z, int64_t B, int64_t D, int64_t F,
                         int64_t L, int64_t G, int64_t ldz, int64_t zw, cudaStream_t st) {
  if (G == 128 && F == 64) return f100::launch_shape<128, 64>(loc, xt, w, bias, z, B, D, L, ldz, zw, st);
  if (G == 64 && F == 128) return f100::launch_shape<64, 128>(loc, xt, w, bias, z, B, D, L, ldz, zw, st);
  return fail(HASTE_ERR_UNSUPPORTED, "tcgen05 forward: no kernel for group size %lld, fan-in %lld", (long long)G, (long long)F);
}

}  // namespace haste
