// Rewire: prune the weakest fan-in slots of every label group, draw new input indices, re-initialise
// the affected weight columns and canonicalise (sort) the index row — one CTA per group, one pass
// over the weights (read once, written once): an HBM-bound kernel.
//
// Semantics follow GroupFixedFanIn.rewire (shared_ffi/rewire.py:143-239): the score of slot k of
// group g is the mean |w| over the group's real rows (fp32, rows added in order so the result is
// reproducible bit for bit), 'threshold' prunes score < threshold, 'fraction' prunes the n_prune
// lowest scores.  Where the reference leaves behaviour to torch (tie order of topk, the randint
// stream) this kernel defines it: ties go to the lowest slot, indices come from Philox4x32-10 with
// key (seed, step) and counter (global group, slot, attempt, 0x5245).
//
// The layer variant the reference's model instantiates (GroupFixedFanInReal.rewire,
// src/group_fanin_real.py:149-286) scores a slot by the mean or the maximum of |w| and prunes the
// globally lowest int(NG*F*fraction) slots of the whole layer.  That takes two small kernels ahead of
// the per-group one: all scores to a scratch array, then one block that finds the k-th smallest score
// by a radix select on the fp32 bit patterns (scores are >= 0, so the patterns order like the values)
// and counts, per group, the slots whose score equals it.  Ties at the k-th score go to the lowest
// flat (group, slot) index.
#include "common.cuh"
#include "launchers.h"

namespace haste {

constexpr int RW_THREADS = 128;

// blocks for a grid-stride kernel over work_items: enough to fill the GPU, no more
static int grid_for(int64_t work_items, int threads) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t blocks = (work_items + threads - 1) / threads;
  const int64_t cap = static_cast<int64_t>(sms) * 16;
  return static_cast<int>(blocks < 1 ? 1 : (blocks < cap ? blocks : cap));
}

__device__ __forceinline__ int regrow_index(uint64_t seed, uint32_t step, int64_t g, int slot, int attempt, int D) {
  const uint4 r = philox4x32_10(static_cast<uint32_t>(g), static_cast<uint32_t>(slot), static_cast<uint32_t>(attempt), 0x5245u,
                                static_cast<uint32_t>(seed), step);
  return static_cast<int>(__umulhi(r.x, static_cast<uint32_t>(D)));
}
__device__ __forceinline__ float regrow_value(uint64_t seed, uint32_t step, int64_t l, int k, float bound) {
  const uint4 r = philox4x32_10(static_cast<uint32_t>(l), static_cast<uint32_t>(k), 0u, 0x494Eu, static_cast<uint32_t>(seed), step);
  const float u = __fmul_rn(static_cast<float>(r.x >> 8), 1.0f / 16777216.0f);
  return __fmul_rn(__fsub_rn(__fmul_rn(2.0f, u), 1.0f), bound);
}

// Score of slot k from the group's weight tile in shared memory: mean (rows added in order, then one
// division) or maximum of |w| over the group's real rows.
__device__ __forceinline__ float slot_score(const uint16_t* tile, int rows, int F, int k, int score_mode) {
  float acc = 0.f;
  if (score_mode == 0) {
    for (int r = 0; r < rows; ++r) acc = __fadd_rn(acc, fabsf(bf16_bits_to_float(tile[r * F + k])));
    return __fdiv_rn(acc, static_cast<float>(rows));
  }
  for (int r = 0; r < rows; ++r) acc = fmaxf(acc, fabsf(bf16_bits_to_float(tile[r * F + k])));
  return acc;
}

// Histogram increment, aggregated over the warp: scores cluster in few bins (a max of bf16 magnitudes is a bf16
// value, so its lower 16 bits are zero and its upper 16 take a handful of values), and one atomic per lane would
// serialise on those addresses.  Called by all 32 lanes; lanes with nothing to add pass active = false.
__device__ __forceinline__ void hist_add_warp(uint32_t* hist, uint32_t bin, bool active) {
  const unsigned peers = __match_any_sync(0xffffffffu, active ? bin : 0xFFFFFFFFu);
  if (active && (threadIdx.x & 31) == __ffs(peers) - 1) atomicAdd(&hist[bin], static_cast<uint32_t>(__popc(peers)));
}

// All scores of the layer: scores[g*F + k]; also the histogram of their upper 16 bits (first pass of the select).
__global__ void __launch_bounds__(RW_THREADS) ffi_scores_kernel(const uint16_t* __restrict__ w, int F, int64_t L, int G, int score_mode,
                                                                float* __restrict__ scores, uint32_t* __restrict__ hist_hi) {
  extern __shared__ __align__(16) unsigned char smem[];
  uint16_t* tile = reinterpret_cast<uint16_t*>(smem);
  const int tid = threadIdx.x;
  const int64_t g = blockIdx.x, l0 = g * G;
  const int rows = static_cast<int>(imin64(G, L - l0));
  const uint16_t* wg = w + l0 * F;
  for (int i = tid; i < rows * F / 8; i += RW_THREADS) reinterpret_cast<uint4*>(tile)[i] = reinterpret_cast<const uint4*>(wg)[i];
  __syncthreads();
  float sc = 0.f;
  if (tid < F) {
    sc = slot_score(tile, rows, F, tid, score_mode);
    scores[g * F + tid] = sc;
  }
  hist_add_warp(hist_hi, __float_as_uint(sc) >> 16, tid < F);
}

// The k-th smallest of n non-negative floats (k >= 1) by a radix select on the bit patterns, two digits of 16
// bits.  Histograms are built by grid-wide kernels (the first inside ffi_scores_kernel); one block walks a
// histogram of 65536 bins to find the digit that holds the k-th element.
constexpr int SEL_THREADS = 1024;
// in: hist[65536], *k_in.  out: *digit, *k_out = rank of the wanted element inside that digit's bin (1-based).
__global__ void __launch_bounds__(SEL_THREADS) select_pick16_kernel(const uint32_t* __restrict__ hist, const uint32_t* __restrict__ k_in,
                                                                    uint32_t* __restrict__ digit, uint32_t* __restrict__ k_out) {
  __shared__ unsigned long long part[SEL_THREADS];
  const int tid = threadIdx.x;
  constexpr int PER = 65536 / SEL_THREADS;
  unsigned long long sum = 0;
  for (int i = 0; i < PER; ++i) sum += hist[tid * PER + i];
  part[tid] = sum;
  __syncthreads();
  if (tid == 0) {
    unsigned long long run = 0;
    for (int i = 0; i < SEL_THREADS; ++i) { const unsigned long long v = part[i]; part[i] = run; run += v; }
  }
  __syncthreads();
  const unsigned long long k = *k_in, before = part[tid];
  if (k > before && k <= before + sum) {                      // exactly one thread: its 64 bins hold the k-th element
    unsigned long long kk = k - before;
    int d = tid * PER;
    for (; d < tid * PER + PER - 1; ++d) {
      if (kk <= hist[d]) break;
      kk -= hist[d];
    }
    *digit = static_cast<uint32_t>(d);
    *k_out = static_cast<uint32_t>(kk);
  }
}
// histogram of the lower 16 bits of the scores whose upper 16 bits equal *hi
__global__ void __launch_bounds__(256) select_hist_lo_kernel(const float* __restrict__ scores, int64_t n, const uint32_t* __restrict__ hi,
                                                             uint32_t* __restrict__ hist_lo) {
  const uint32_t* bits = reinterpret_cast<const uint32_t*>(scores);
  const uint32_t want = *hi;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i0 = static_cast<int64_t>(blockIdx.x) * blockDim.x; i0 < n; i0 += stride) {      // whole warps stay in the loop together
    const int64_t i = i0 + threadIdx.x;
    const uint32_t b = i < n ? bits[i] : 0u;
    hist_add_warp(hist_lo, b & 0xFFFFu, i < n && (b >> 16) == want);
  }
}
// sel[0] = T = (hi << 16) | lo, sel[1] stays the number of scores equal to T that are to be pruned;
// eq[g] += 1 for every score of group g that equals T (eq zeroed beforehand)
__global__ void __launch_bounds__(256) select_equal_count_kernel(const float* __restrict__ scores, int64_t n, int F, const uint32_t* __restrict__ hi,
                                                                 const uint32_t* __restrict__ lo, uint32_t* __restrict__ sel) {
  const uint32_t* bits = reinterpret_cast<const uint32_t*>(scores);
  const uint32_t T = (*hi << 16) | *lo;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  if (blockIdx.x == 0 && threadIdx.x == 0) sel[0] = T;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    if (bits[i] == T) atomicAdd(&sel[2 + i / F], 1u);
}
// exclusive prefix over the groups of the per-group equal counts, in place
// *total receives the number of scores equal to T in this shard
__global__ void __launch_bounds__(SEL_THREADS) select_scan_kernel(uint32_t* __restrict__ eq, int NG, uint32_t* __restrict__ total) {
  __shared__ int part[SEL_THREADS];
  const int tid = threadIdx.x;
  const int chunk = (NG + SEL_THREADS - 1) / SEL_THREADS, lo = min(NG, tid * chunk), hi = min(NG, lo + chunk);
  int sum = 0;
  for (int g = lo; g < hi; ++g) sum += static_cast<int>(eq[g]);
  part[tid] = sum;
  __syncthreads();
  if (tid == 0) {
    int run = 0;
    for (int i = 0; i < SEL_THREADS; ++i) { const int v = part[i]; part[i] = run; run += v; }
    *total = static_cast<uint32_t>(run);
  }
  __syncthreads();
  int run = part[tid];
  for (int g = lo; g < hi; ++g) { const int c = static_cast<int>(eq[g]); eq[g] = static_cast<uint32_t>(run); run += c; }
}

__global__ void __launch_bounds__(RW_THREADS) ffi_rewire_kernel(uint16_t* __restrict__ w, int32_t* __restrict__ loc, float* __restrict__ mom,
                                                                int D, int F, int64_t L, int G, int64_t group0, int score_mode, int prune_mode,
                                                                float threshold, int n_prune, const uint32_t* __restrict__ sel,
                                                                uint32_t tie_base, int regrow_mode, int init_mode,
                                                                int regroup, float bound, uint64_t seed, uint32_t step,
                                                                int32_t* __restrict__ changed) {
  extern __shared__ __align__(16) unsigned char smem[];
  uint16_t* tile = reinterpret_cast<uint16_t*>(smem);                 // [G][F]
  float* score = reinterpret_cast<float*>(smem + size_t(G) * F * 2);  // [F]
  int* cur = reinterpret_cast<int*>(score + F);                       // [F] index row being edited
  int* pruned = cur + F;                                              // [F]
  int* src_of = pruned + F;                                           // [F] output position -> source slot
  const int tid = threadIdx.x;
  const int64_t g = blockIdx.x;
  const int64_t l0 = g * G;
  const int rows = static_cast<int>(imin64(G, L - l0));
  uint16_t* wg = w + l0 * F;

  for (int i = tid; i < rows * F / 8; i += RW_THREADS)
    reinterpret_cast<uint4*>(tile)[i] = reinterpret_cast<const uint4*>(wg)[i];
  if (tid < F) cur[tid] = loc[g * F + tid];
  __syncthreads();

  if (tid < F) score[tid] = slot_score(tile, rows, F, tid, score_mode);
  __syncthreads();
  if (tid < F) {
    int p;
    const float s = score[tid];
    if (prune_mode == 0) {
      p = s < threshold;
    } else if (prune_mode == 2) {
      // global fraction: below the k-th smallest score of the layer, or equal to it and early enough in flat order
      const uint32_t T = sel[0], sb = __float_as_uint(s);
      if (sb != T) {
        p = sb < T;
      } else {
        // rank among the scores equal to T in flat (group, slot) order; tie_base counts those on lower-ranked shards
        int64_t rank = static_cast<int64_t>(tie_base) + sel[2 + g];
        for (int j = 0; j < tid; ++j) rank += __float_as_uint(score[j]) == T;
        p = rank < static_cast<int64_t>(sel[1]);
      }
    } else {
      int rank = 0;
      for (int j = 0; j < F; ++j) {
        const float sj = score[j];
        rank += (sj < s) || (sj == s && j < tid);
      }
      p = rank < n_prune;
    }
    pruned[tid] = p;
  }
  __syncthreads();
  int n_pruned = 0;
  for (int k = 0; k < F; ++k) n_pruned += pruned[k];
  if (n_pruned == 0 && !regroup) return;

  // ---- regrow
  if (regrow_mode == 0) {
    if (tid < F && pruned[tid]) cur[tid] = regrow_index(seed, step, group0 + g, tid, 0, D);
    __syncthreads();
  } else {
    // 'unused': slots are served in ascending order; a candidate is rejected while any live slot of
    // the row (kept, or already re-grown) holds the same index.  After 64 rejections the search walks
    // upward from the last candidate, which ends within F+1 steps because at most F indices are taken.
    int live = (tid < F) ? !pruned[tid] : 0;
    for (int k = 0; k < F; ++k) {
      if (!pruned[k]) continue;                       // uniform: read from shared memory
      int v = 0;
      bool found = false;
      for (int t = 0; t < 64 && !found; ++t) {
        v = regrow_index(seed, step, group0 + g, k, t, D);
        const int clash = __syncthreads_or(live && cur[tid < F ? tid : 0] == v);
        found = !clash;
      }
      for (int t = 0; t <= F && !found; ++t) {
        v = (v + 1) % D;
        const int clash = __syncthreads_or(live && cur[tid < F ? tid : 0] == v);
        found = !clash;
      }
      if (tid == k) { cur[k] = v; live = 1; }
      __syncthreads();
    }
  }

  // ---- re-initialise pruned columns (all real rows of the group)
  for (int i = tid; i < rows * F; i += RW_THREADS) {
    const int r = i / F, k = i - r * F;
    if (pruned[k]) {
      uint16_t v = 0;
      if (init_mode == 1) v = rn_bf16_bits(regrow_value(seed, step, group0 * G + l0 + r, k, bound));
      tile[i] = v;
    }
  }
  // ---- regroup: stable sort of the index row, columns follow
  if (tid < F) {
    int pos = tid;
    if (regroup) {
      pos = 0;
      const int64_t key = static_cast<int64_t>(cur[tid]) * 256 + tid;
      for (int j = 0; j < F; ++j) pos += (static_cast<int64_t>(cur[j]) * 256 + j) < key;
    }
    src_of[pos] = tid;
  }
  __syncthreads();
  if (tid < F) loc[g * F + tid] = cur[src_of[tid]];
  for (int i = tid; i < rows * F; i += RW_THREADS) {
    const int r = i / F, p = i - r * F;
    wg[i] = tile[r * F + src_of[p]];
  }
  if (mom != nullptr) {
    float* mg = mom + l0 * F;
    for (int r = 0; r < rows; ++r) {
      float v = 0.f;
      if (tid < F) { const int s = src_of[tid]; v = pruned[s] ? 0.f : mg[r * F + s]; }
      __syncthreads();
      if (tid < F) mg[r * F + tid] = v;
    }
  }
  if (tid == 0 && changed != nullptr && n_pruned) atomicAdd(changed, n_pruned);
}

// Scratch of the layer-wide selection (32-bit words): scores[NG*F] | sel[2 + NG] | hist_hi[65536] | hist_lo[65536] |
// tmp[8] = {k, hi digit, k inside that bin, lo digit, scores equal to T in this shard, -, -, -}
struct SelectScratch {
  float* scores;
  uint32_t *sel, *hist_hi, *hist_lo, *tmp;
  int64_t n;
};
static SelectScratch select_scratch(void* scratch, int64_t NG, int64_t F) {
  SelectScratch s;
  s.scores = static_cast<float*>(scratch);
  s.sel = reinterpret_cast<uint32_t*>(s.scores + NG * F);
  s.hist_hi = s.sel + 2 + NG;
  s.hist_lo = s.hist_hi + 65536;
  s.tmp = s.hist_lo + 65536;
  s.n = NG * F;
  return s;
}

// Phase 1: scores of this shard and the histogram of their upper 16 bits.
int launch_rewire_select_begin(const void* w, int64_t F, int64_t L, int64_t G, int score_mode, void* scratch, cudaStream_t st) {
  const int64_t NG = (L + G - 1) / G;
  SelectScratch s = select_scratch(scratch, NG, F);
  cudaError_t e = cudaMemsetAsync(s.sel, 0, sizeof(uint32_t) * static_cast<size_t>(2 + NG + 2 * 65536 + 8), st);
  if (e != cudaSuccess) return fail(HASTE_ERR_LAUNCH, "cudaMemsetAsync: %s", cudaGetErrorString(e));
  e = cudaFuncSetAttribute(ffi_scores_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(size_t(G) * F * 2));
  if (e != cudaSuccess) return fail(HASTE_ERR_LAUNCH, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  ffi_scores_kernel<<<static_cast<unsigned>(NG), RW_THREADS, size_t(G) * F * 2, st>>>((const uint16_t*)w, int(F), L, int(G), score_mode, s.scores, s.hist_hi);
  return check_launch("ffi_scores_kernel");
}
// Phase 2: hist_hi now holds the histogram of the WHOLE layer (summed over the shards by the caller, or this shard's
// when there is one); find the digit of the k-th smallest score and histogram the lower 16 bits inside it.
int launch_rewire_select_refine(int64_t F, int64_t L, int64_t G, int64_t k, void* scratch, cudaStream_t st) {
  const int64_t NG = (L + G - 1) / G;
  SelectScratch s = select_scratch(scratch, NG, F);
  const uint32_t k32 = static_cast<uint32_t>(k);
  cudaError_t e = cudaMemcpyAsync(s.tmp, &k32, sizeof(uint32_t), cudaMemcpyHostToDevice, st);     // pageable source: copied before the call returns
  if (e != cudaSuccess) return fail(HASTE_ERR_LAUNCH, "cudaMemcpyAsync: %s", cudaGetErrorString(e));
  select_pick16_kernel<<<1, SEL_THREADS, 0, st>>>(s.hist_hi, s.tmp, s.tmp + 1, s.tmp + 2);
  select_hist_lo_kernel<<<static_cast<unsigned>(grid_for(s.n, 256)), 256, 0, st>>>(s.scores, s.n, s.tmp + 1, s.hist_lo);
  return check_launch("select_hist_lo_kernel");
}
// Phase 3: hist_lo holds the whole layer's histogram inside the digit; fix the threshold T = k-th smallest score, the
// number of scores equal to T that are pruned (sel[1], layer-wide), this shard's per-group positions among the scores
// equal to T (sel[2..]) and their count (tmp[4]).
int launch_rewire_select_finish(int64_t F, int64_t L, int64_t G, void* scratch, cudaStream_t st) {
  const int64_t NG = (L + G - 1) / G;
  SelectScratch s = select_scratch(scratch, NG, F);
  select_pick16_kernel<<<1, SEL_THREADS, 0, st>>>(s.hist_lo, s.tmp + 2, s.tmp + 3, s.sel + 1);
  select_equal_count_kernel<<<static_cast<unsigned>(grid_for(s.n, 256)), 256, 0, st>>>(s.scores, s.n, int(F), s.tmp + 1, s.tmp + 3, s.sel);
  select_scan_kernel<<<1, SEL_THREADS, 0, st>>>(s.sel + 2, int(NG), s.tmp + 4);
  return check_launch("select_scan_kernel");
}

// prune_mode 2: layer-wide fraction selected inside this call (one shard = the whole layer);
// prune_mode 3: the selection was prepared in `scratch` by the three phases above (layer sharded over ranks) and
//               tie_base scores equal to the threshold belong to lower-ranked shards.
int launch_rewire(void* w, int32_t* loc, float* mom, int64_t D, int64_t F, int64_t L, int64_t G, int64_t group0, int score_mode, int prune_mode,
                  float threshold, int64_t n_prune, int regrow_mode, int init_mode, int regroup, uint64_t seed, uint32_t step,
                  void* scratch, int32_t* changed, cudaStream_t st, uint32_t tie_base) {
  const int64_t NG = (L + G - 1) / G;
  const size_t sm = size_t(G) * F * 2 + size_t(F) * 4 * 4;
  cudaError_t e = cudaFuncSetAttribute(ffi_rewire_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sm));
  if (e != cudaSuccess) return fail(HASTE_ERR_LAUNCH, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  if (changed != nullptr) cudaMemsetAsync(changed, 0, sizeof(int32_t), st);
  const uint32_t* sel = nullptr;
  if (prune_mode == 2) {
    if (int rc = launch_rewire_select_begin(w, F, L, G, score_mode, scratch, st)) return rc;
    if (int rc = launch_rewire_select_refine(F, L, G, n_prune, scratch, st)) return rc;
    if (int rc = launch_rewire_select_finish(F, L, G, scratch, st)) return rc;
    tie_base = 0;
  }
  if (prune_mode == 2 || prune_mode == 3) sel = select_scratch(scratch, NG, F).sel;
  const float bound = static_cast<float>(1.0 / sqrt(static_cast<double>(F)));
  ffi_rewire_kernel<<<static_cast<unsigned>(NG), RW_THREADS, sm, st>>>((uint16_t*)w, loc, mom, int(D), int(F), L, int(G), group0, score_mode,
                                                                        prune_mode == 3 ? 2 : prune_mode, threshold, static_cast<int>(n_prune), sel,
                                                                        tie_base, regrow_mode, init_mode, regroup, bound, seed, step, changed);
  return check_launch("ffi_rewire_kernel");
}

}  // namespace haste
