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
#include "common.cuh"
#include "launchers.h"

namespace haste {

constexpr int RW_THREADS = 128;

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

__global__ void __launch_bounds__(RW_THREADS) ffi_rewire_kernel(uint16_t* __restrict__ w, int32_t* __restrict__ loc, float* __restrict__ mom,
                                                                int D, int F, int64_t L, int G, int64_t group0, int prune_mode,
                                                                float threshold, int n_prune, int regrow_mode, int init_mode,
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

  if (tid < F) {
    float acc = 0.f;
    for (int r = 0; r < rows; ++r) acc = __fadd_rn(acc, fabsf(bf16_bits_to_float(tile[r * F + tid])));
    score[tid] = __fdiv_rn(acc, static_cast<float>(rows));
  }
  __syncthreads();
  if (tid < F) {
    int p;
    const float s = score[tid];
    if (prune_mode == 0) {
      p = s < threshold;
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

int launch_rewire(void* w, int32_t* loc, float* mom, int64_t D, int64_t F, int64_t L, int64_t G, int64_t group0, int prune_mode,
                  float threshold, int n_prune, int regrow_mode, int init_mode, int regroup, uint64_t seed, uint32_t step,
                  int32_t* changed, cudaStream_t st) {
  const int64_t NG = (L + G - 1) / G;
  const size_t sm = size_t(G) * F * 2 + size_t(F) * 4 * 4;
  cudaError_t e = cudaFuncSetAttribute(ffi_rewire_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sm));
  if (e != cudaSuccess) return fail(HASTE_ERR_LAUNCH, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  if (changed != nullptr) cudaMemsetAsync(changed, 0, sizeof(int32_t), st);
  const float bound = static_cast<float>(1.0 / sqrt(static_cast<double>(F)));
  ffi_rewire_kernel<<<static_cast<unsigned>(NG), RW_THREADS, sm, st>>>((uint16_t*)w, loc, mom, int(D), int(F), L, int(G), group0,
                                                                        prune_mode, threshold, n_prune, regrow_mode, init_mode, regroup,
                                                                        bound, seed, step, changed);
  return check_launch("ffi_rewire_kernel");
}

}  // namespace haste
