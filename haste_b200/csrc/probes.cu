// Stand-alone rate probes for the three resources the fused train step leans on.  They are measurement entry points
// (timed by `bench.py --aux`), not part of the training path: each isolates one access pattern of the fused kernel at
// the kernel's own sizes, so that the design choices it records can be re-measured on any box.
//   haste_probe_red_rate     fp32 reduce-add into a small [D,B] array (the dX scatter): scalar coalesced red, red.v4
//                            along one row, red.v4 across 32 rows (what a transposed accumulator would issue)
//   haste_probe_gather_rate  gathering 64 rows x 256 B of xt per tile into swizzled shared memory: TMA tile::gather4
//                            issued by 1, 2 or 4 warps against cp.async from 1, 2 or 4 warps with asynchronous barrier arrival
//   haste_probe_umma_rate    back-to-back tcgen05.mma (M = 128, K = 16) at the step's N and operand majors
#include "common.cuh"
#include "runtime.h"
#include "sm100.cuh"

namespace haste {
namespace probe {
using namespace sm100;

__device__ __forceinline__ uint32_t lcg(uint32_t& s) { s = s * 1664525u + 1013904223u; return s >> 8; }

// ---------------------------------------------------------------- reduce-add rate
// One "tile" = 64 rows x 128 floats (32 KB of adds), as one batch tile of the fused step scatters.
//   mode 0: 4 warps; warp w adds floats [32w, 32w+32) of each row: one 128-byte transaction per warp instruction
//   mode 1: red.v4, a warp covers 512 contiguous bytes of one row
//   mode 2: red.v4, lane l adds 16 bytes of row (l) — 32 rows per warp instruction
__global__ void __launch_bounds__(128) red_kernel(float* dxt, int D, int B, int tiles, int mode) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  uint32_t s = blockIdx.x * 7919u + 17u;   // same sequence for all threads of the CTA
  const int nbt = B / 128;
  for (int it = 0; it < tiles; ++it) {
    const int b0 = static_cast<int>(lcg(s) % static_cast<uint32_t>(nbt)) * 128;
    if (mode == 0) {
      for (int k = 0; k < 64; ++k) {
        const int row = static_cast<int>(lcg(s) % static_cast<uint32_t>(D));
        atomicAdd(dxt + static_cast<size_t>(row) * B + b0 + warp * 32 + lane, 1.0f);
      }
    } else if (mode == 1) {
      for (int k4 = 0; k4 < 16; ++k4) {   // warp w handles row k4*4 + w, lane l its floats [4l, 4l+4)
        int row = 0;
        for (int j = 0; j < 4; ++j) { const int r = static_cast<int>(lcg(s) % static_cast<uint32_t>(D)); if (j == warp) row = r; }
        float* p = dxt + static_cast<size_t>(row) * B + b0 + lane * 4;
        asm volatile("red.global.add.v4.f32 [%0], {%1,%1,%1,%1};" ::"l"(p), "f"(1.0f) : "memory");
      }
    } else {
      // 64 rows, one per lane of warps 0 and 1 (warps 2, 3 idle, as with an M = 64 accumulator); 32 instructions of
      // 16 bytes cover the row's 128 floats
      int row = 0;
      for (int k = 0; k < 64; ++k) { const int r = static_cast<int>(lcg(s) % static_cast<uint32_t>(D)); if (k == tid) row = r; }
      if (tid < 64) {
        float* p = dxt + static_cast<size_t>(row) * B + b0;
        for (int c = 0; c < 32; ++c) asm volatile("red.global.add.v4.f32 [%0], {%1,%1,%1,%1};" ::"l"(p + c * 4), "f"(1.0f) : "memory");
      }
    }
  }
}

// ---------------------------------------------------------------- gather rate
// Each CTA fills a 4-stage ring of 16 KB tiles (64 rows x 2 blocks x 128 B, 128-byte swizzle) `tiles` times with
// pseudo-random rows of xt [D,B]; a consumer warp waits for each stage and hands it back at once.
constexpr int G_ROWS = 64, G_STAGES = 4, G_BLK = G_ROWS * 128, G_STAGE = 2 * G_BLK;
constexpr long long G_WAIT = 2000000000ll;

__global__ void __launch_bounds__(192) gather_kernel(const __nv_bfloat16* xt, const __grid_constant__ CUtensorMap tm_x, int D, int B, int tiles,
                                                     int mode, int* err) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const uint32_t sbase = smem_u32(sm);
  __shared__ __align__(8) uint64_t bars[2 * G_STAGES];
  __shared__ int abort_word;
  __shared__ int rows_s[G_STAGES][G_ROWS];
  volatile int* abort_flag = &abort_word;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool tma = mode == 0 || mode >= 10;           // mode 0 / 12 / 14: TMA gather4 issued by 1 / 2 / 4 warps; mode 1 / 2 / 4: cp.async from that many warps
  const int n_prod = mode == 0 ? 1 : (mode >= 10 ? mode - 10 : mode);
  auto full = [&](int s) { return smem_u32(&bars[s]); };
  auto empty = [&](int s) { return smem_u32(&bars[G_STAGES + s]); };
  if (tid == 0) {
    for (int s = 0; s < G_STAGES; ++s) { mbar_init(full(s), tma ? 1 : 32); mbar_init(empty(s), 1); }
    mbar_fence_init();
    abort_word = 0;
  }
  __syncthreads();
  const int nbt = B / 128;
  if (warp >= 1 && warp <= n_prod) {
    const int p = warp - 1;
    uint32_t s = blockIdx.x * 7919u + 17u;
    for (int it = 0; it < tiles; ++it) {
      // every producer advances the same sequence; producer (it % n_prod) loads the tile
      const int b0 = static_cast<int>(lcg(s) % static_cast<uint32_t>(nbt)) * 128;
      const int r_lo = static_cast<int>(lcg(s) % static_cast<uint32_t>(D - 64));
      if (it % n_prod != p) continue;
      const int st = it % G_STAGES;
      if (!mbar_wait(empty(st), ((it / G_STAGES) & 1) ^ 1, abort_flag, err, 90, G_WAIT, 100)) break;
      __syncwarp();
      const uint32_t xb = sbase + st * G_STAGE;
      // 64 distinct rows: r_lo + a permutation step, so that neighbouring slots are not neighbouring rows
      const int my_row0 = r_lo + ((lane * 37) & 63), my_row1 = r_lo + (((lane + 32) * 37) & 63);
      if (tma) {
        rows_s[st][lane] = my_row0; rows_s[st][lane + 32] = my_row1;
        __syncwarp();
        if (lane == 0) mbar_arrive_expect_tx(full(st), G_ROWS * 256);
        __syncwarp();
        const int blk = lane >> 4, r4 = lane & 15;
        const int4 lr = reinterpret_cast<const int4*>(rows_s[st])[r4];
        asm volatile(
            "cp.async.bulk.tensor.2d.shared::cta.global.tile::gather4.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];" ::"r"(
                xb + blk * G_BLK + r4 * 512),
            "l"(&tm_x), "r"(b0 + blk * 64), "r"(lr.x), "r"(lr.y), "r"(lr.z), "r"(lr.w), "r"(full(st))
            : "memory");
      } else {
        const int j = lane & 15;
        const uint32_t dcol = (j >> 3) * G_BLK + ((j & 7) << 4);
#pragma unroll 4
        for (int i = 0; i < 32; ++i) {
          const int k = i * 2 + (lane >> 4);
          const int lk = __shfl_sync(0xffffffffu, i < 16 ? my_row0 : my_row1, k & 31);
          cp_async16(xb + ((dcol + k * 128) ^ ((k & 7) << 4)), xt + static_cast<int64_t>(lk) * B + b0 + j * 8, true);
        }
        cp_async_mbar_arrive_noinc(full(st));
      }
    }
    // copies in flight land before the CTA exits
    for (int it = max(0, tiles - G_STAGES); it < tiles; ++it)
      if (it % n_prod == p) mbar_wait_final(full(it % G_STAGES), (it / G_STAGES) & 1, G_WAIT);
  } else if (warp == 0) {
    for (int it = 0; it < tiles; ++it) {
      const int st = it % G_STAGES;
      if (!mbar_wait(full(st), (it / G_STAGES) & 1, abort_flag, err, 91, G_WAIT)) break;
      __syncwarp();
      if (lane == 0) mbar_arrive(empty(st));
    }
  }
}

// ---------------------------------------------------------------- tcgen05.mma rate
__global__ void __launch_bounds__(128) umma_kernel(uint32_t idesc, uint32_t a_lbo, uint32_t b_lbo, uint32_t a_adv, uint32_t b_adv, int iters,
                                                   long long* out) {
  extern __shared__ uint8_t raw[];
  __shared__ __align__(8) uint64_t mbar;
  __shared__ uint32_t tslot;
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~static_cast<uintptr_t>(1023));
  for (int i = threadIdx.x; i < 65536 / 4; i += 128) reinterpret_cast<uint32_t*>(base)[i] = 0x3c003c00u;
  if (threadIdx.x == 0) { mbar_init(smem_u32(&mbar), 1); mbar_fence_init(); }
  fence_proxy_async();
  __syncthreads();
  if (threadIdx.x < 32) { tmem_alloc(smem_u32(&tslot), 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tslot;
  if (threadIdx.x == 0) {
    const uint64_t da = make_sdesc(smem_u32(base), a_lbo, 1024), db = make_sdesc(smem_u32(base) + 32768, b_lbo, 1024);
    const long long t0 = clock64();
    for (int it = 0; it < iters; ++it) {
#pragma unroll
      for (int u = 0; u < 8; ++u) umma_bf16(tmem, da + static_cast<uint64_t>((u * a_adv) >> 4), db + static_cast<uint64_t>((u * b_adv) >> 4), idesc, 1u);
    }
    tc_commit(smem_u32(&mbar));
    const long long t1 = clock64();
    mbar_wait_final(smem_u32(&mbar), 0, 2000000000ll);
    const long long t2 = clock64();
    out[0] = t1 - t0;     // cycles to issue
    out[1] = t2 - t0;     // cycles until the last product has completed
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) tmem_dealloc(tmem, 512);
}

}  // namespace probe
}  // namespace haste

using namespace haste;

extern "C" {

int haste_probe_red_rate(float* dxt, int64_t D, int64_t B, int32_t mode, int32_t tiles_per_cta, haste_stream_t stream) {
  if (dxt == nullptr || D < 1 || B < 128 || (B % 128) != 0 || mode < 0 || mode > 2 || tiles_per_cta < 1)
    return fail(HASTE_ERR_BAD_ARG, "haste_probe_red_rate: bad arguments (B must be a multiple of 128, mode in 0..2)");
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  probe::red_kernel<<<sms, 128, 0, static_cast<cudaStream_t>(stream)>>>(dxt, static_cast<int>(D), static_cast<int>(B), tiles_per_cta, mode);
  return check_launch("probe red_kernel");
}

int haste_probe_gather_rate(const void* xt, int64_t D, int64_t B, int32_t mode, int32_t tiles_per_cta, haste_stream_t stream) {
  if (xt == nullptr || D < 128 || B < 128 || (B % 128) != 0 || !(mode == 0 || mode == 1 || mode == 2 || mode == 4 || mode == 12 || mode == 14) ||
      tiles_per_cta < 1)
    return fail(HASTE_ERR_BAD_ARG, "haste_probe_gather_rate: bad arguments (D >= 128, B a multiple of 128, mode 0/12/14 = TMA gather4 from 1/2/4 warps, "
                "1/2/4 = cp.async warps)");
  if (int rc = report_pending_status("haste_probe_gather_rate")) return rc;
  int* err = nullptr;
  if (int rc = device_status_word(&err)) return rc;
  CUtensorMap tm;
  if (int rc = make_tmap_bf16_2d(&tm, xt, static_cast<uint64_t>(B), static_cast<uint64_t>(D), static_cast<uint64_t>(B) * 2, 64, 1)) return rc;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int smem = probe::G_STAGES * probe::G_STAGE + 1024;
  cudaError_t e = cudaFuncSetAttribute(probe::gather_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return fail(HASTE_ERR_LAUNCH, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  probe::gather_kernel<<<sms, 192, smem, static_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16*>(xt), tm, static_cast<int>(D),
                                                                            static_cast<int>(B), tiles_per_cta, mode, err);
  return check_launch("probe gather_kernel");
}

int haste_probe_umma_rate(int32_t N, int32_t a_mn_major, int32_t b_mn_major, int32_t iters, long long* cycles_out, haste_stream_t stream) {
  if (cycles_out == nullptr || N < 16 || N > 256 || (N % 16) != 0 || iters < 1)
    return fail(HASTE_ERR_BAD_ARG, "haste_probe_umma_rate: bad arguments (N a multiple of 16 in [16,256])");
  const uint32_t idesc = sm100::make_idesc(128, N, a_mn_major ? 1 : 0, b_mn_major ? 1 : 0);
  // operand strides as the fused step uses them: an MN-major operand advances 2048 B per K step, a K-major one 32 B
  const uint32_t a_lbo = a_mn_major ? 10240u : 16u, b_lbo = b_mn_major ? 16384u : 16u;
  const uint32_t a_adv = a_mn_major ? 2048u : 32u, b_adv = b_mn_major ? 2048u : 32u;
  cudaError_t e = cudaFuncSetAttribute(probe::umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
  if (e != cudaSuccess) return fail(HASTE_ERR_LAUNCH, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  probe::umma_kernel<<<1, 128, 100 * 1024, static_cast<cudaStream_t>(stream)>>>(idesc, a_lbo, b_lbo, a_adv, b_adv, iters, cycles_out);
  return check_launch("probe umma_kernel");
}

}  // extern "C"
