// Streaming kernels of the FFI path: stochastic rounding, the SGD(+wd)(+momentum)+SR update on a
// stand-alone gradient tensor, the dX transpose+round tail, the bf16 transpose of the features and the
// COO target bucketing.  All are HBM-bound: 16-byte accesses, grid sized to a multiple of the SM count.
#include "common.cuh"

#include <mutex>
#include "launchers.h"

namespace haste {

static int grid_for(int64_t work_items, int threads) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t blocks = (work_items + threads - 1) / threads;
  const int64_t cap = static_cast<int64_t>(sms) * 16;
  return static_cast<int>(blocks < 1 ? 1 : (blocks < cap ? blocks : cap));
}

// ---------------------------------------------------------------- fp32 -> bf16 stochastic rounding
__global__ void __launch_bounds__(256) sr_round_kernel(const float* __restrict__ x, uint16_t* __restrict__ out, int64_t n, uint64_t seed) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    out[i] = sr_bf16_bits(x[i], rand16_reference(seed, i));
}

// ---------------------------------------------------------------- SGD + SR on [rows, cols]
// One thread owns 8 consecutive columns of one row when cols % 8 == 0 (one Philox call in the packed
// stream, one 16-byte weight access), else one element.
__global__ void __launch_bounds__(256) sgd_sr_vec8_kernel(uint16_t* __restrict__ w, const uint16_t* __restrict__ g, float* __restrict__ m,
                                                          int64_t rows, int cols, int64_t row0, float lr, float wd, float mu,
                                                          uint64_t seed, uint32_t step, uint32_t flags) {
  const int c8n = cols >> 3;
  const int64_t n8 = rows * c8n;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8; i += stride) {
    const int64_t r = i / c8n;
    const int c8 = static_cast<int>(i - r * c8n);
    const int64_t off = r * cols + c8 * 8;
    uint4 wv = *reinterpret_cast<const uint4*>(w + off);
    const uint4 gv = __ldg(reinterpret_cast<const uint4*>(g + off));
    uint32_t* wp = reinterpret_cast<uint32_t*>(&wv);
    const uint32_t* gp = reinterpret_cast<const uint32_t*>(&gv);
    float mv[8];
    if (m) {
      const float4 a = *reinterpret_cast<const float4*>(m + off), b = *reinterpret_cast<const float4*>(m + off + 4);
      mv[0] = a.x; mv[1] = a.y; mv[2] = a.z; mv[3] = a.w; mv[4] = b.x; mv[5] = b.y; mv[6] = b.z; mv[7] = b.w;
    }
    uint4 rp = make_uint4(0, 0, 0, 0);
    const bool sr = flags & HASTE_F_SR, packed = flags & HASTE_F_RNG_PACKED;
    if (sr && packed) rp = rand_packed8(seed, step, row0 + r, c8);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      uint32_t r16 = 0;
      if (sr) r16 = packed ? unpack16(rp, j) : rand16_reference(seed, (row0 + r) * cols + c8 * 8 + j);
      const uint16_t wb = (wp[j >> 1] >> (16 * (j & 1))) & 0xFFFFu;
      const uint16_t gb = (gp[j >> 1] >> (16 * (j & 1))) & 0xFFFFu;
      const uint16_t nb = sgd_update_bits(wb, bf16_bits_to_float(gb), m ? &mv[j] : nullptr, lr, wd, mu, flags, r16);
      wp[j >> 1] = (j & 1) ? ((wp[j >> 1] & 0xFFFFu) | (uint32_t(nb) << 16)) : ((wp[j >> 1] & 0xFFFF0000u) | nb);
    }
    *reinterpret_cast<uint4*>(w + off) = wv;
    if (m) {
      *reinterpret_cast<float4*>(m + off) = make_float4(mv[0], mv[1], mv[2], mv[3]);
      *reinterpret_cast<float4*>(m + off + 4) = make_float4(mv[4], mv[5], mv[6], mv[7]);
    }
  }
}

__global__ void __launch_bounds__(256) sgd_sr_scalar_kernel(uint16_t* __restrict__ w, const uint16_t* __restrict__ g, float* __restrict__ m,
                                                            int64_t rows, int cols, int64_t row0, float lr, float wd, float mu,
                                                            uint64_t seed, uint32_t step, uint32_t flags) {
  const int64_t n = rows * cols;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    const int64_t r = i / cols;
    const int c = static_cast<int>(i - r * cols);
    uint32_t r16 = 0;
    if (flags & HASTE_F_SR) r16 = rand16(flags, seed, step, row0 + r, c, cols);
    float mv = m ? m[i] : 0.f;
    w[i] = sgd_update_bits(w[i], bf16_bits_to_float(g[i]), m ? &mv : nullptr, lr, wd, mu, flags, r16);
    if (m) m[i] = mv;
  }
}

// ---------------------------------------------------------------- dxt [D,B] fp32 -> dx [B,D] bf16 (SR)
__global__ void __launch_bounds__(256) dxt_to_dx_sr_kernel(const float* __restrict__ dxt, uint16_t* __restrict__ dx, int64_t B, int64_t D,
                                                           uint64_t seed) {
  __shared__ float tile[32][33];
  const int64_t d0 = static_cast<int64_t>(blockIdx.x) * 32, b0 = static_cast<int64_t>(blockIdx.y) * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  for (int j = ty; j < 32; j += 8) {
    const int64_t d = d0 + j, b = b0 + tx;
    tile[j][tx] = (d < D && b < B) ? dxt[d * B + b] : 0.f;
  }
  __syncthreads();
  for (int j = ty; j < 32; j += 8) {
    const int64_t b = b0 + j, d = d0 + tx;
    if (b < B && d < D) {
      const int64_t flat = b * D + d;
      dx[flat] = sr_bf16_bits(tile[tx][j], rand16_reference(seed, flat));
    }
  }
}

__global__ void __launch_bounds__(256) transpose_bf16_kernel(const uint16_t* __restrict__ x, uint16_t* __restrict__ xt, int64_t B, int64_t D) {
  __shared__ uint16_t tile[32][34];
  const int64_t d0 = static_cast<int64_t>(blockIdx.x) * 32, b0 = static_cast<int64_t>(blockIdx.y) * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int j = ty; j < 32; j += 8) {
    const int64_t b = b0 + j, d = d0 + tx;
    tile[j][tx] = (b < B && d < D) ? x[b * D + d] : uint16_t(0);
  }
  __syncthreads();
  for (int j = ty; j < 32; j += 8) {
    const int64_t d = d0 + j, b = b0 + tx;
    if (d < D && b < B) xt[d * B + b] = tile[tx][j];
  }
}

// ---------------------------------------------------------------- target bucketing (COO -> per-group CSR)
// Pass 1 counts entries per group, pass 2 turns counts into offsets (single CTA scan) and resets the
// counters to serve as fill cursors, pass 3 scatters.  Entry order inside a group is not defined
// (the consumers only set bits).
__global__ void tgt_count_kernel(const int32_t* __restrict__ coo, int64_t nnz, int64_t label0, int64_t L, int G, int32_t* __restrict__ cnt) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nnz; i += stride) {
    const int64_t c = static_cast<int64_t>(coo[2 * i + 1]) - label0;
    if (c >= 0 && c < L) atomicAdd(&cnt[c / G], 1);
  }
}
__global__ void __launch_bounds__(1024) tgt_scan_kernel(int32_t* __restrict__ cnt, int32_t* __restrict__ ptr, int64_t NG) {
  __shared__ int warp_sums[32];
  __shared__ int carry;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  for (int64_t base = 0; base < NG; base += 1024) {
    const int64_t i = base + threadIdx.x;
    const int v = i < NG ? cnt[i] : 0;
    int s = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, s, o);
      if (lane >= o) s += t;
    }
    if (lane == 31) warp_sums[wid] = s;
    __syncthreads();
    if (wid == 0) {
      int ws = warp_sums[lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, ws, o);
        if (lane >= o) ws += t;
      }
      warp_sums[lane] = ws;
    }
    __syncthreads();
    const int excl = carry + (wid ? warp_sums[wid - 1] : 0) + s - v;
    if (i < NG) { ptr[i] = excl; cnt[i] = 0; }
    __syncthreads();
    if (threadIdx.x == 1023) carry = excl + v;
    __syncthreads();
  }
  if (threadIdx.x == 0) ptr[NG] = carry;
}
__global__ void tgt_fill_kernel(const int32_t* __restrict__ coo, int64_t nnz, int64_t label0, int64_t L, int G,
                                const int32_t* __restrict__ ptr, int32_t* __restrict__ cur, uint32_t* __restrict__ ent) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nnz; i += stride) {
    const int64_t c = static_cast<int64_t>(coo[2 * i + 1]) - label0;
    if (c >= 0 && c < L) {
      const int64_t g = c / G;
      const int pos = ptr[g] + atomicAdd(&cur[g], 1);
      ent[pos] = (static_cast<uint32_t>(coo[2 * i]) << 8) | static_cast<uint32_t>(c - g * G);
    }
  }
}

// ---------------------------------------------------------------- per-step preparation in one launch
// Block 0 buckets the COO targets entirely in shared memory (count, scan, fill: no global scratch) and clears
// the loss scalar; every other block transposes one 32x32 tile of x [B,D] -> xt [D,B] and clears the same tile
// of dxt [D,B].  Replaces one memset, the three bucketing kernels, the transpose and two fills.
constexpr int PREP_THREADS = 1024;
// VEC: B and D are multiples of 8 and the three arrays are 16-byte aligned; a block then moves a 64 (batch) x 128
// (feature) tile with 16-byte accesses on both sides, so that the whole preparation is a few dozen blocks and still
// finishes in microseconds when most SMs are held by a persistent kernel of another stream.
template <bool VEC>
__global__ void __launch_bounds__(PREP_THREADS) step_prepare_kernel(const uint16_t* __restrict__ x, uint16_t* __restrict__ xt, float* __restrict__ dxt,
                                                                    float* __restrict__ loss, const int32_t* __restrict__ coo, int64_t nnz,
                                                                    int64_t label0, int64_t L, int G, int NG, int32_t* __restrict__ ptr,
                                                                    uint32_t* __restrict__ ent, int64_t B, int64_t D, int tiles_d) {
  extern __shared__ int32_t cnt[];          // NG counters, then reused as fill cursors
  __shared__ int part[PREP_THREADS];
  const int tid = threadIdx.x;
  // the fused step that follows in the stream may place its CTAs and set up its shared memory and TMEM already (it
  // waits for this grid to complete before it reads anything this kernel writes)
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (blockIdx.x == 0) {
    // One block does the whole bucketing, so its two passes over the entries keep four independent 8-byte loads
    // in flight per thread (a batch of C5 has ~37 K entries; one load at a time costs one L2 latency per entry).
    const int2* coo2 = reinterpret_cast<const int2*>(coo);
    if (tid == 0 && loss != nullptr) *loss = 0.f;
    for (int i = tid; i < NG; i += PREP_THREADS) cnt[i] = 0;
    __syncthreads();
    for (int64_t i0 = tid; i0 < nnz; i0 += 4 * PREP_THREADS) {
      int2 e[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) { const int64_t i = i0 + k * PREP_THREADS; e[k] = i < nnz ? __ldg(coo2 + i) : make_int2(0, -1); }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int64_t c = static_cast<int64_t>(e[k].y) - label0;
        if (e[k].y >= 0 && c >= 0 && c < L) atomicAdd(&cnt[c / G], 1);
      }
    }
    __syncthreads();
    // exclusive scan of cnt[0..NG): each thread owns a contiguous chunk
    const int chunk = (NG + PREP_THREADS - 1) / PREP_THREADS, lo = min(NG, tid * chunk), hi = min(NG, lo + chunk);
    int sum = 0;
    for (int i = lo; i < hi; ++i) sum += cnt[i];
    part[tid] = sum;
    __syncthreads();
    if (tid < 32) {                        // warp 0 scans the 1024 partial sums, 32 per lane
      int loc_sum = 0;
      for (int i = 0; i < PREP_THREADS / 32; ++i) loc_sum += part[tid * (PREP_THREADS / 32) + i];
      int incl = loc_sum;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) { const int v = __shfl_up_sync(0xffffffffu, incl, o); if (tid >= o) incl += v; }
      int run = incl - loc_sum;
      for (int i = 0; i < PREP_THREADS / 32; ++i) { const int idx = tid * (PREP_THREADS / 32) + i; const int v = part[idx]; part[idx] = run; run += v; }
      if (tid == 31) ptr[NG] = run;
    }
    __syncthreads();
    int run = part[tid];
    for (int i = lo; i < hi; ++i) { const int v = cnt[i]; ptr[i] = run; cnt[i] = run; run += v; }   // cnt becomes the write cursor
    __syncthreads();
    for (int64_t i0 = tid; i0 < nnz; i0 += 4 * PREP_THREADS) {
      int2 e[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) { const int64_t i = i0 + k * PREP_THREADS; e[k] = i < nnz ? __ldg(coo2 + i) : make_int2(0, -1); }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int64_t c = static_cast<int64_t>(e[k].y) - label0;
        if (e[k].y >= 0 && c >= 0 && c < L) {
          const int64_t g = c / G;
          const int pos = atomicAdd(&cnt[g], 1);
          ent[pos] = (static_cast<uint32_t>(e[k].x) << 8) | static_cast<uint32_t>(c - g * G);
        }
      }
    }
    return;
  }
  const int blk = blockIdx.x - 1;
  if (VEC) {
    // tile [64 batch rows][128 features] in shared memory, 16-byte chunks; the chunk index is XORed with the row's
    // 8-row group so that the column reads of the transposed write-out spread over the banks
    __shared__ __align__(16) uint16_t tile[64][128];
    const int64_t d0 = static_cast<int64_t>(blk % tiles_d) * 128, b0 = static_cast<int64_t>(blk / tiles_d) * 64;
    {
      const int row = tid >> 4, ch = tid & 15;
      const int64_t b = b0 + row, d = d0 + ch * 8;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (b < B && d < D) v = *reinterpret_cast<const uint4*>(x + b * D + d);
      *reinterpret_cast<uint4*>(&tile[row][(ch ^ ((row >> 3) & 7)) * 8]) = v;
    }
    __syncthreads();
    {
      const int dl = tid >> 3, b8 = tid & 7;                 // 8 lanes write one 128-byte run of a row of xt
      const int64_t d = d0 + dl, b = b0 + b8 * 8;
      if (d < D && b < B) {
        const int col = (((dl >> 3) ^ b8) << 3) | (dl & 7);  // rows b8*8 .. b8*8+7 all lie in 8-row group b8
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) w[i] = static_cast<uint32_t>(tile[b8 * 8 + 2 * i][col]) | (static_cast<uint32_t>(tile[b8 * 8 + 2 * i + 1][col]) << 16);
        *reinterpret_cast<uint4*>(xt + d * B + b) = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int idx = tid + k * PREP_THREADS, dl = idx >> 4, c = idx & 15;
      const int64_t d = d0 + dl, b = b0 + c * 4;
      if (d < D && b < B) *reinterpret_cast<float4*>(dxt + d * B + b) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    return;
  }
  __shared__ uint16_t tile[32][34];
  const int64_t d0 = static_cast<int64_t>(blk % tiles_d) * 32, b0 = static_cast<int64_t>(blk / tiles_d) * 32;
  const int tx = tid & 31, ty = tid >> 5;            // 32 x 32 threads: one element each
  {
    const int64_t b = b0 + ty, d = d0 + tx;
    tile[ty][tx] = (b < B && d < D) ? x[b * D + d] : uint16_t(0);
  }
  __syncthreads();
  {
    const int64_t d = d0 + ty, b = b0 + tx;
    if (d < D && b < B) { xt[d * B + b] = tile[tx][ty]; dxt[d * B + b] = 0.f; }
  }
}

int launch_step_prepare(const void* x, void* xt, float* dxt, float* loss, const int32_t* coo, int64_t nnz, int64_t label0, int64_t L,
                        int64_t G, int32_t* ptr, uint32_t* ent, int64_t B, int64_t D, cudaStream_t st) {
  const int64_t NG = (L + G - 1) / G;
  if (reinterpret_cast<uintptr_t>(coo) & 7) return fail(HASTE_ERR_BAD_ARG, "haste_ffi_step_prepare: the COO target pairs must start on an 8-byte boundary");
  const size_t sm = sizeof(int32_t) * static_cast<size_t>(NG);
  if (sm > 200 * 1024) return fail(HASTE_ERR_TOO_LARGE, "haste_ffi_step_prepare: %lld label groups need more shared memory than one block has; "
                                   "use haste_transpose_bf16 + haste_targets_bucket", (long long)NG);
  const bool vec = (B % 8) == 0 && (D % 8) == 0 && aligned16(x) && aligned16(xt) && aligned16(dxt);
  auto k = vec ? step_prepare_kernel<true> : step_prepare_kernel<false>;
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sm));
  if (e != cudaSuccess) return fail(HASTE_ERR_LAUNCH, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  const int tiles_d = static_cast<int>(vec ? (D + 127) / 128 : (D + 31) / 32), tiles_b = static_cast<int>(vec ? (B + 63) / 64 : (B + 31) / 32);
  k<<<1 + tiles_d * tiles_b, PREP_THREADS, sm, st>>>((const uint16_t*)x, (uint16_t*)xt, dxt, loss, coo, nnz, label0, L, int(G), int(NG), ptr, ent, B, D,
                                                     tiles_d);
  return check_launch("step_prepare_kernel");
}

// ---------------------------------------------------------------- row padding: [rows, cols] (stride ld_src) -> [rows, ld_dst], zeros past cols
__global__ void __launch_bounds__(256) pad_rows_kernel(const uint16_t* __restrict__ src, int64_t ld_src, uint16_t* __restrict__ dst,
                                                       int64_t ld_dst, int64_t rows, int64_t cols) {
  const int64_t chunks = ld_dst >> 3;                      // ld_dst % 8 == 0, dst 16-byte aligned
  const int64_t n = rows * chunks;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    const int64_t r = i / chunks, c = (i - r * chunks) << 3;
    const uint16_t* p = src + r * ld_src + c;
    uint16_t e[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) e[k] = (c + k < cols) ? p[k] : uint16_t(0);
    uint4 v;
    v.x = e[0] | (uint32_t(e[1]) << 16); v.y = e[2] | (uint32_t(e[3]) << 16);
    v.z = e[4] | (uint32_t(e[5]) << 16); v.w = e[6] | (uint32_t(e[7]) << 16);
    *reinterpret_cast<uint4*>(dst + r * ld_dst + c) = v;
  }
}

int launch_pad_rows(const void* src, int64_t ld_src, void* dst, int64_t ld_dst, int64_t rows, int64_t cols, cudaStream_t st) {
  pad_rows_kernel<<<grid_for(rows * (ld_dst >> 3), 256), 256, 0, st>>>((const uint16_t*)src, ld_src, (uint16_t*)dst, ld_dst, rows, cols);
  return check_launch("pad_rows_kernel");
}

__global__ void check_loc_kernel(const int32_t* __restrict__ loc, int64_t n, int D, int* __restrict__ bad) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    if (loc[i] < 0 || loc[i] >= D) atomicAdd(bad, 1);
}

// ================================================================ launchers
int launch_sr_round(const float* x, void* out, int64_t n, uint64_t seed, cudaStream_t st) {
  if (n == 0) return HASTE_OK;
  sr_round_kernel<<<grid_for(n, 256), 256, 0, st>>>(x, (uint16_t*)out, n, seed);
  return check_launch("sr_round_kernel");
}

int launch_sgd_sr(void* w, const void* g, float* m, int64_t rows, int64_t cols, int64_t row0, float lr, float wd, float mu,
                  uint64_t seed, uint32_t step, uint32_t flags, cudaStream_t st) {
  if (rows * cols == 0) return HASTE_OK;
  const bool vec = (cols % 8 == 0) && aligned16(w) && aligned16(g) && (m == nullptr || aligned16(m));
  if (vec)
    sgd_sr_vec8_kernel<<<grid_for(rows * cols / 8, 256), 256, 0, st>>>((uint16_t*)w, (const uint16_t*)g, m, rows, int(cols), row0, lr, wd,
                                                                       mu, seed, step, flags);
  else
    sgd_sr_scalar_kernel<<<grid_for(rows * cols, 256), 256, 0, st>>>((uint16_t*)w, (const uint16_t*)g, m, rows, int(cols), row0, lr, wd,
                                                                     mu, seed, step, flags);
  return check_launch("sgd_sr_kernel");
}

int launch_dxt_to_dx(const float* dxt, void* dx, int64_t B, int64_t D, uint64_t seed, cudaStream_t st) {
  dim3 grid(static_cast<unsigned>((D + 31) / 32), static_cast<unsigned>((B + 31) / 32));
  dxt_to_dx_sr_kernel<<<grid, 256, 0, st>>>(dxt, (uint16_t*)dx, B, D, seed);
  return check_launch("dxt_to_dx_sr_kernel");
}

int launch_transpose(const void* x, void* xt, int64_t B, int64_t D, cudaStream_t st) {
  dim3 grid(static_cast<unsigned>((D + 31) / 32), static_cast<unsigned>((B + 31) / 32));
  transpose_bf16_kernel<<<grid, 256, 0, st>>>((const uint16_t*)x, (uint16_t*)xt, B, D);
  return check_launch("transpose_bf16_kernel");
}

int launch_targets_bucket(const int32_t* coo, int64_t nnz, int64_t label0, int64_t L, int64_t G, int32_t* ptr, uint32_t* ent,
                          int32_t* scratch, cudaStream_t st) {
  const int64_t NG = (L + G - 1) / G;
  cudaError_t e = cudaMemsetAsync(scratch, 0, sizeof(int32_t) * NG, st);
  if (e != cudaSuccess) return fail(HASTE_ERR_LAUNCH, "cudaMemsetAsync: %s", cudaGetErrorString(e));
  if (nnz > 0) tgt_count_kernel<<<grid_for(nnz, 256), 256, 0, st>>>(coo, nnz, label0, L, int(G), scratch);
  tgt_scan_kernel<<<1, 1024, 0, st>>>(scratch, ptr, NG);
  if (nnz > 0) tgt_fill_kernel<<<grid_for(nnz, 256), 256, 0, st>>>(coo, nnz, label0, L, int(G), ptr, scratch, ent);
  return check_launch("targets_bucket");
}

// ---------------------------------------------------------------- target bucketing without any allocation
// Scratch for haste_targets_bucket_noalloc: one int32 counter per label group, resident in every GPU that loads
// this library (256 KiB) until the process exits.
constexpr int64_t NOALLOC_MAX_GROUPS = 65536;
static __device__ __align__(256) int32_t g_bucket_scratch[NOALLOC_MAX_GROUPS];

// In host code `g_bucket_scratch` is only a handle for the device symbol, not a device address, so the address
// is looked up once per device (with that device current) and cached.  The cache is guarded by a mutex: host
// threads may make their first call on a device at the same time.
static int32_t* noalloc_scratch_ptr(int* rc) {
  constexpr int MAX_DEV = 64;
  static int32_t* cache[MAX_DEV] = {nullptr};
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= MAX_DEV) {
    *rc = fail(HASTE_ERR_LAUNCH, "haste_targets_bucket_noalloc: cudaGetDevice: %s (device %d)", cudaGetErrorString(e), dev);
    return nullptr;
  }
  if (cache[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_bucket_scratch);
    if (e != cudaSuccess || p == nullptr) {
      *rc = fail(HASTE_ERR_LAUNCH, "haste_targets_bucket_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
      return nullptr;
    }
    cache[dev] = static_cast<int32_t*>(p);
  }
  *rc = HASTE_OK;
  return cache[dev];
}

int launch_targets_bucket_noalloc(const int32_t* coo, int64_t nnz, int64_t label0, int64_t L, int64_t G, int32_t* ptr, uint32_t* ent,
                                  cudaStream_t st) {
  const int64_t NG = (L + G - 1) / G;
  if (NG > NOALLOC_MAX_GROUPS)
    return fail(HASTE_ERR_TOO_LARGE, "haste_targets_bucket_noalloc: %lld label groups exceed the built-in scratch of %lld groups; "
                "use haste_targets_bucket with caller-provided scratch", (long long)NG, (long long)NOALLOC_MAX_GROUPS);
  int rc = HASTE_OK;
  int32_t* scratch = noalloc_scratch_ptr(&rc);
  if (scratch == nullptr) return rc;
  // the counters keep the previous call's values: launch_targets_bucket clears the NG it uses before counting
  return launch_targets_bucket(coo, nnz, label0, L, G, ptr, ent, scratch, st);
}

int launch_check_loc(const int32_t* loc, int64_t n, int64_t D, cudaStream_t st) {
  int* bad = nullptr;
  cudaError_t e = cudaMallocAsync(reinterpret_cast<void**>(&bad), sizeof(int), st);
  if (e != cudaSuccess) return fail(HASTE_ERR_LAUNCH, "cudaMallocAsync: %s", cudaGetErrorString(e));
  cudaMemsetAsync(bad, 0, sizeof(int), st);
  check_loc_kernel<<<grid_for(n, 256), 256, 0, st>>>(loc, n, int(D), bad);
  int h = 0;
  cudaMemcpyAsync(&h, bad, sizeof(int), cudaMemcpyDeviceToHost, st);
  cudaFreeAsync(bad, st);
  e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return fail(HASTE_ERR_LAUNCH, "check_locations: %s", cudaGetErrorString(e));
  if (h != 0) return fail(HASTE_ERR_INDEX_RANGE, "%d index values outside [0,%lld)", h, (long long)D);
  return HASTE_OK;
}

}  // namespace haste
