// Forward gather-GEMM of the FFI layer on tcgen05 / TMEM, group size 128, fan-in 64:
//     z[b, l] = sum_k xt[loc[l/128, k], b] * w[l, k] + bias[l]        (bf16 in, fp32 accumulate, bf16 out)
// This is the unfused forward of the autograd surface: it has to write the [B, L] logits, so it is bound by
// that HBM write (2*B*L bytes), not by the tensor pipe.
//
// Persistent, one CTA per SM, groups g = blockIdx.x, += gridDim.x; per group the batch is walked in 128-row
// tiles.  Same shared-memory operand layout as the fused train step (128-byte-swizzled row blocks; X tile as
// MN-major A, W tile as K-major B).  Warp roles (384 threads): warps 0 and 2 gather X tiles (cp.async, 6-stage
// ring) and the W tile (double-buffered); warp 1 issues the MMAs; warps 4-11 drain the accumulator: TMEM ->
// + bias -> bf16 -> a swizzled staging tile in shared memory -> 16-byte stores in which every warp instruction
// covers whole 256-byte row segments of z.  All waits are bounded (see mbar_wait).
#include "common.cuh"
#include "launchers.h"
#include "runtime.h"
#include "sm100.cuh"

namespace haste {
namespace f100 {
using namespace sm100;

constexpr int G = 128, F = 64, BT = 128;
constexpr int NXS = 6;
constexpr int XBLK = F * 128;                 // one 64-batch block of an X stage (bytes)
constexpr int XSTAGE = 2 * XBLK;              // 16 KB
constexpr int WSTAGE = G * 128;               // 16 KB
constexpr int CSTAGE = BT * G * 2;            // bf16 staging tile, 32 KB
constexpr int OFF_X = 0;
constexpr int OFF_W = OFF_X + NXS * XSTAGE;
constexpr int OFF_C = OFF_W + 2 * WSTAGE;
constexpr int OFF_BIAS = OFF_C + 2 * CSTAGE;  // float [2][G]
constexpr int OFF_BAR = OFF_BIAS + 2 * G * 4;
constexpr int OFF_MISC = OFF_BAR + 32 * 8;
constexpr int SMEM_BYTES = OFF_MISC + 64 + 1024;
static_assert(SMEM_BYTES <= 232448, "shared memory budget");
constexpr int B_XFULL = 0, B_XEMPTY = NXS, B_WFULL = 2 * NXS, B_WEMPTY = B_WFULL + 2, B_ZFULL = B_WEMPTY + 2,
              B_ZEMPTY = B_ZFULL + 2, B_BEMPTY = B_ZEMPTY + 2, NBAR = B_BEMPTY + 2;
static_assert(NBAR <= 32, "barrier space");
constexpr int N_EPI = 8;                      // epilogue warps: 4 TMEM lane quarters x 2 column halves
constexpr int N_SETS = 2;                     // sets of epilogue warps; set s takes the tiles whose Z stage (and staging buffer) is s
constexpr int N_XPROD = 1;                    // producer warps beyond the three among the first four warps
constexpr int NTHREADS = (4 + N_EPI * N_SETS + N_XPROD) * 32;
constexpr uint32_t TM_COLS = 256;             // two 128-column accumulator stages
constexpr long long WAIT_LIMIT = 4000000000ll;

struct FwdArgs {
  const int32_t* loc;
  const __nv_bfloat16* xt;
  const __nv_bfloat16* w;
  const __nv_bfloat16* bias;
  __nv_bfloat16* z;
  int* err;
  int64_t B, L, ldz, zw;   // zw: writable width of a row of z (columns L..zw-1 receive zeros)
  int D, NG;
};

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__global__ void __launch_bounds__(NTHREADS, 1) ffi_forward_sm100_kernel(FwdArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const uint32_t sbase = smem_u32(sm);
  float* bias_s = reinterpret_cast<float*>(sm + OFF_BIAS);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + OFF_MISC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + OFF_MISC + 8);
  auto bar = [&](int i) { return sbase + OFF_BAR + i * 8; };
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int T = static_cast<int>((a.B + BT - 1) / BT);

  if (tid == 0) {
    for (int i = 0; i < NXS; ++i) { mbar_init(bar(B_XFULL + i), 1); mbar_init(bar(B_XEMPTY + i), 1); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(B_WFULL + i), 1);  mbar_init(bar(B_WEMPTY + i), 1);
      mbar_init(bar(B_ZFULL + i), 1);  mbar_init(bar(B_ZEMPTY + i), N_EPI);
      mbar_init(bar(B_BEMPTY + i), N_EPI * N_SETS);     // the epilogue warps are done with the group's bias row
    }
    mbar_fence_init();
    *abort_flag = 0;
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), TM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const int n_my_groups = (a.NG > static_cast<int>(blockIdx.x)) ? (a.NG - 1 - static_cast<int>(blockIdx.x)) / static_cast<int>(gridDim.x) + 1 : 0;

  if (warp == 0 || warp == 2 || warp == 3 || warp >= 4 + N_EPI * N_SETS) {
    // ================================================================ producers
    // Each producer warp has one item (a W tile or an X tile) in flight at a time and pays the full memory latency
    // for it, so the gather rate is the number of producer warps over that latency: 3 + N_XPROD warps.  X tiles
    // are dealt by tile index and the warp count divides the ring depth, so every ring stage is always filled by
    // the same warp, which therefore sees all phases of that stage's barriers in order; the last producer warp
    // loads the W tiles and nothing else.
    constexpr int N_PROD = 3 + N_XPROD - 1;           // X producers
    static_assert(N_XPROD >= 1 && NXS % N_PROD == 0, "every X stage belongs to one producer warp");
    const int p = warp == 0 ? 0 : (warp < 4 ? warp - 1 : 3 + warp - (4 + N_EPI * N_SETS));
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
      if (p == N_PROD) {
        mbar_wait(bar(B_WEMPTY + ws), ((gi >> 1) & 1) ^ 1, abort_flag, a.err, 21, WAIT_LIMIT, 100);
        mbar_wait(bar(B_BEMPTY + ws), ((gi >> 1) & 1) ^ 1, abort_flag, a.err, 21, WAIT_LIMIT, 100);
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int c = lane * 4 + i;
          bias_s[ws * G + c] = (a.bias != nullptr && c < rows_real) ? __bfloat162float(a.bias[l0 + c]) : 0.f;
        }
        const uint32_t wb = sbase + OFF_W + ws * WSTAGE;
#pragma unroll 4
        for (int i = 0; i < 32; ++i) {
          const int idx = i * 32 + lane, r = idx >> 3, c = idx & 7;
          cp_async16(wb + r * 128 + ((c ^ (r & 7)) << 4), a.w + (l0 + r) * F + c * 8, r < rows_real);
        }
        land(bar(B_WFULL + ws));
      }
      for (int t = 0; t < T; ++t, ++it) {
        if (p == N_PROD || (it % N_PROD) != p) continue;
        const int xs = it % NXS;
        mbar_wait(bar(B_XEMPTY + xs), ((it / NXS) & 1) ^ 1, abort_flag, a.err, 22, WAIT_LIMIT, 100);
        __syncwarp();
        const int64_t b0 = static_cast<int64_t>(t) * BT;
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
    }
  } else if (warp == 1) {
    // ================================================================ MMA issuer
    // The warp runs its control flow converged; one elected lane issues the products and commits (descriptors stay
    // in uniform registers this way).
    {
      constexpr uint32_t ID_FWD = make_idesc(128, G, 1, 0);
      const uint64_t D_XA = make_sdesc(sbase + OFF_X, XBLK, 1024);    // X tile as MN-major A
      const uint64_t D_WB = make_sdesc(sbase + OFF_W, 16, 1024);      // W tile as K-major B
      const uint32_t xa_lo = static_cast<uint32_t>(D_XA), xa_hi = static_cast<uint32_t>(D_XA >> 32);
      const uint32_t wb_lo = static_cast<uint32_t>(D_WB), wb_hi = static_cast<uint32_t>(D_WB >> 32);
      const uint32_t id_fwd = ID_FWD;
      int it = 0, xs = 0, xph = 0;
      for (int gi = 0; gi < n_my_groups; ++gi) {
        const int ws = gi & 1;
        mbar_wait(bar(B_WFULL + ws), (gi >> 1) & 1, abort_flag, a.err, 23, WAIT_LIMIT);
        for (int t = 0; t < T; ++t, ++it) {
          const int zs = it & 1;
          mbar_wait(bar(B_XFULL + xs), xph, abort_flag, a.err, 24, WAIT_LIMIT);
          mbar_wait(bar(B_ZEMPTY + zs), ((it >> 1) & 1) ^ 1, abort_flag, a.err, 25, WAIT_LIMIT);
          tc_fence_after();
          const uint32_t xa = xa_lo + static_cast<uint32_t>(xs) * (XSTAGE >> 4), wb = wb_lo + (ws ? (WSTAGE >> 4) : 0u);
          const uint32_t tz = tmem + (zs ? G : 0);
          if (elect_one()) {
            umma_bf16_lohi<false>(tz, xa, xa_hi, wb, wb_hi, id_fwd);
#pragma unroll
            for (int ks = 1; ks < F / 16; ++ks)
              umma_bf16_lohi<true>(tz, xa + ((ks * 2048) >> 4), xa_hi, wb + ((ks * 32) >> 4), wb_hi, id_fwd);
            tc_commit(bar(B_ZFULL + zs));
            tc_commit(bar(B_XEMPTY + xs));
            if (t + 1 == T) tc_commit(bar(B_WEMPTY + ws));
          }
          __syncwarp();
          if (++xs == NXS) { xs = 0; xph ^= 1; }
        }
      }
    }
  } else if (warp >= 4 && warp < 4 + N_EPI * N_SETS) {
    // ================================================================ epilogue
    // Two sets of eight warps take alternate tiles: while one set drains its staging tile to global memory, the
    // other reads the next accumulator stage, so neither the TMEM reads nor the stores wait for each other.
    const int ep = warp - 4, set = ep / N_EPI, es = ep % N_EPI;
    const int q = es & 3, h = es >> 2;                       // TMEM lane quarter, column half (64 labels)
    const int row = q * 32 + lane;
    const int et = tid - 128 - set * N_EPI * 32;             // 0..255 inside the set
    int it = 0;
    for (int gi = 0; gi < n_my_groups; ++gi) {
      const int g = blockIdx.x + gi * gridDim.x;
      const int ws = gi & 1;
      const int64_t l0 = static_cast<int64_t>(g) * G;
      const int cvalid = static_cast<int>(imin64(G, a.zw - l0));      // columns of this group that exist in z (zeros past L)
      mbar_wait(bar(B_WFULL + ws), (gi >> 1) & 1, abort_flag, a.err, 26, WAIT_LIMIT);    // bias row in place
      const float4* bs4 = reinterpret_cast<const float4*>(bias_s + ws * G + h * 64);
      for (int t = 0; t < T; ++t, ++it) {
        if (N_SETS > 1 && (it & 1) != set) continue;         // the other set's tile
        const int zs = it & 1;
        const int64_t b0 = static_cast<int64_t>(t) * BT;
        mbar_wait(bar(B_ZFULL + zs), (it >> 1) & 1, abort_flag, a.err, 27, WAIT_LIMIT);
        tc_fence_after();
        const uint32_t ta = tmem + (static_cast<uint32_t>(q * 32) << 16) + (zs ? G : 0) + h * 64;
        // staging tile [128 rows][256 B], 16-byte chunk index XORed with (row & 7): conflict-free both for the
        // row-per-thread writes here and for the row-segment reads of the store loop
        uint8_t* crow = sm + OFF_C + zs * CSTAGE + row * 256;
#pragma unroll 1
        for (int c16 = 0; c16 < 64; c16 += 16) {
          uint32_t r[16];
          __syncwarp();
          tmem_ld16(ta + c16, r);
          tmem_ld_wait();
#pragma unroll
          for (int e8 = 0; e8 < 16; e8 += 8) {
            const float4 ba = bs4[(c16 + e8) >> 2], bb = bs4[((c16 + e8) >> 2) + 1];
            const uint4 v = make_uint4(pack2(__uint_as_float(r[e8 + 0]) + ba.x, __uint_as_float(r[e8 + 1]) + ba.y),
                                       pack2(__uint_as_float(r[e8 + 2]) + ba.z, __uint_as_float(r[e8 + 3]) + ba.w),
                                       pack2(__uint_as_float(r[e8 + 4]) + bb.x, __uint_as_float(r[e8 + 5]) + bb.y),
                                       pack2(__uint_as_float(r[e8 + 6]) + bb.z, __uint_as_float(r[e8 + 7]) + bb.w));
            const int chunk = (h * 64 + c16 + e8) >> 3;           // 0..15
            *reinterpret_cast<uint4*>(crow + ((chunk ^ (row & 7)) << 4)) = v;
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(B_ZEMPTY + zs));
        named_bar_sync(1 + set, N_EPI * 32);         // the set's whole staging tile is written
        // coalesced store: 16 lanes cover one 256-byte row segment; 8 KB per pass of the 256 threads
        const uint8_t* cbase = sm + OFF_C + zs * CSTAGE;
        if (!*abort_flag) {
#pragma unroll 4
          for (int pass = 0; pass < 8; ++pass) {
            const int r = pass * 16 + (et >> 4), chunk = et & 15;
            if (b0 + r < a.B && chunk * 8 < cvalid) {
              const uint4 v = *reinterpret_cast<const uint4*>(cbase + r * 256 + ((chunk ^ (r & 7)) << 4));
              __nv_bfloat16* dst = a.z + (b0 + r) * a.ldz + l0 + chunk * 8;
              if (chunk * 8 + 8 <= cvalid) {
                *reinterpret_cast<uint4*>(dst) = v;
              } else {
                const uint16_t* e = reinterpret_cast<const uint16_t*>(&v);
                for (int i = 0; chunk * 8 + i < cvalid; ++i) reinterpret_cast<uint16_t*>(dst)[i] = e[i];
              }
            }
          }
        }
        // the set's next tile reuses this staging buffer: nobody may write it before everybody has read it
        named_bar_sync(1 + set, N_EPI * 32);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(B_BEMPTY + ws));
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, TM_COLS);
}

}  // namespace f100

bool forward_sm100_supported(const void* z, int64_t B, int64_t F, int64_t G, int64_t ldz) {
  return G == f100::G && F == f100::F && (B % 8) == 0 && (ldz % 8) == 0 && aligned16(z);
}

int launch_forward_sm100(const int32_t* loc, const void* xt, const void* w, const void* bias, void* z, int64_t B, int64_t D, int64_t F,
                         int64_t L, int64_t G, int64_t ldz, int64_t zw, cudaStream_t st) {
  using namespace f100;
  if (int rc = report_pending_status("tcgen05 forward")) return rc;
  int* err_dev = nullptr;
  if (int rc = device_status_word(&err_dev)) return rc;
  FwdArgs a;
  a.loc = loc; a.xt = static_cast<const __nv_bfloat16*>(xt); a.w = static_cast<const __nv_bfloat16*>(w);
  a.bias = static_cast<const __nv_bfloat16*>(bias); a.z = static_cast<__nv_bfloat16*>(z); a.err = err_dev;
  a.B = B; a.L = L; a.ldz = ldz; a.zw = zw; a.D = static_cast<int>(D); a.NG = static_cast<int>((L + G - 1) / G);
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = a.NG < sms ? a.NG : sms;
  cudaError_t e = cudaFuncSetAttribute(ffi_forward_sm100_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  if (e != cudaSuccess) return fail(HASTE_ERR_LAUNCH, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  ffi_forward_sm100_kernel<<<grid, NTHREADS, SMEM_BYTES, st>>>(a);
  return check_launch("ffi_forward_sm100_kernel");
}

}  // namespace haste
