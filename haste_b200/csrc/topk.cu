// Running per-row top-k over logits that arrive in label chunks (inference: the reference takes
// torch.topk(logits, 100) / topk(5) over the full [B,L] logits, src/evaluate.py:151-156, 219).
//
// The forward kernels produce a chunk of logits z[b, 0..C) for labels col0 .. col0+C-1 (a chunk is sized to stay
// in L2); this kernel folds it into the running top-k of every row, so the [B,L] matrix never exists.  One CTA per
// row keeps the row's current best k values (sorted, descending) and their label ids in shared memory.  A logit
// is a candidate only if it beats the current k-th value; after the first few hundred labels candidates are rare
// (about k ln(L/k) per row over the whole label set), so they are inserted one at a time by the whole CTA: count
// the entries that stay ahead of it, shift the rest down by one, write it.  Equal values keep the order in which
// they arrived (lower label id first), which makes the result unique.
#include "common.cuh"
#include "launchers.h"

namespace haste {

constexpr int TK_THREADS = 128;
constexpr int TK_KMAX = 128;                 // k <= TK_THREADS: one thread per kept entry during an insertion
constexpr int TK_CAND = TK_THREADS * 8;      // candidates of one 1024-label slice

__global__ void __launch_bounds__(TK_THREADS) topk_update_kernel(const uint16_t* __restrict__ z, int64_t ldz, int64_t C, int64_t col0, int k,
                                                                 float* __restrict__ vals, int32_t* __restrict__ idx) {
  __shared__ float sv[TK_KMAX];
  __shared__ int si[TK_KMAX];
  __shared__ float cv[TK_CAND];
  __shared__ int ci[TK_CAND];
  __shared__ int ncand;
  const int tid = threadIdx.x;
  const int64_t b = blockIdx.x;
  const uint16_t* zr = z + b * ldz;
  if (tid < k) { sv[tid] = vals[b * k + tid]; si[tid] = idx[b * k + tid]; }
  if (tid == 0) ncand = 0;
  __syncthreads();
  const bool vec_ok = (reinterpret_cast<uintptr_t>(zr) & 15) == 0;
  for (int64_t c0 = 0; c0 < C; c0 += TK_CAND) {
    const float thr = sv[k - 1];
    // ---- scan one slice of 1024 labels: 8 consecutive labels per thread
    const int64_t j0 = c0 + static_cast<int64_t>(tid) * 8;
    float e[8];
    if (vec_ok && j0 + 8 <= C) {
      const uint4 v = *reinterpret_cast<const uint4*>(zr + j0);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int p = 0; p < 4; ++p) { e[2 * p] = __uint_as_float(w[p] << 16); e[2 * p + 1] = __uint_as_float(w[p] & 0xFFFF0000u); }
    } else {
#pragma unroll
      for (int p = 0; p < 8; ++p) e[p] = (j0 + p < C) ? bf16_bits_to_float(zr[j0 + p]) : -INFINITY;
    }
#pragma unroll
    for (int p = 0; p < 8; ++p) {
      if (e[p] > thr) {                                       // -inf never passes; a NaN logit is never selected
        const int slot = atomicAdd(&ncand, 1);
        cv[slot] = e[p];
        ci[slot] = static_cast<int>(col0 + j0 + p);
      }
    }
    __syncthreads();
    const int n = ncand;
    // ---- insert the candidates, lowest label id first among equal values (slots are filled in any order)
    for (int c = 0; c < n; ++c) {
      const float v = cv[c];
      const int id = ci[c];
      // entries that stay ahead of the candidate: larger value, or equal value and smaller label id
      const bool ahead = tid < k && (sv[tid] > v || (sv[tid] == v && si[tid] >= 0 && si[tid] < id));
      const int pos = __syncthreads_count(ahead);
      if (pos < k) {                                          // uniform over the CTA
        float mv = 0.f;
        int mi = 0;
        const bool moves = tid >= pos && tid < k - 1;
        if (moves) { mv = sv[tid]; mi = si[tid]; }
        __syncthreads();
        if (moves) { sv[tid + 1] = mv; si[tid + 1] = mi; }
        if (tid == 0) { sv[pos] = v; si[pos] = id; }
        __syncthreads();
      }
    }
    if (tid == 0) ncand = 0;
    __syncthreads();
  }
  if (tid < k) { vals[b * k + tid] = sv[tid]; idx[b * k + tid] = si[tid]; }
}

int launch_topk_update(const void* z, int64_t ldz, int64_t B, int64_t C, int64_t col0, int k, float* vals, int32_t* idx, cudaStream_t st) {
  if (B == 0 || C == 0) return HASTE_OK;
  topk_update_kernel<<<static_cast<unsigned>(B), TK_THREADS, 0, st>>>(static_cast<const uint16_t*>(z), ldz, C, col0, k, vals, idx);
  return check_launch("topk_update_kernel");
}

}  // namespace haste
