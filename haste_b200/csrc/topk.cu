// Running per-row top-k over logits that arrive in label chunks (inference: the reference takes
// torch.topk(logits, 100) / topk(5) over the full [B,L] logits, src/evaluate.py:151-156, 219).
//
// The forward kernels produce a chunk of logits z[b, 0..C) for labels col0 .. col0+C-1 (a chunk is sized to stay
// in L2); this kernel folds it into the running top-k of every row, so the [B,L] matrix never exists.  One CTA per
// row keeps the row's current best k values (sorted, descending) and their label ids in shared memory.  A logit
// is a candidate only if it beats the current k-th value; after the first few hundred labels candidates are rare
// (about k ln(L/k) per row over the whole label set); the candidates of a range of slices are merged into the kept
// list in one step (every element computes its new position).  Equal values keep the lower label id first, which
// makes the result unique.
#include "common.cuh"
#include "launchers.h"

namespace haste {

constexpr int TK_THREADS = 128;
constexpr int TK_KMAX = 128;                 // k <= TK_THREADS: one thread per kept entry during an insertion
constexpr int TK_CAND = TK_THREADS * 8;      // candidates of one 1024-label slice
constexpr int TK_WIDE = 16;                  // slices scanned between two synchronisations once candidates are rare
constexpr int TK_BATCH = 4;                  // slices whose loads a thread has in flight at a time

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
  // Scans labels [c0, c0 + n_sub * 1024) of the chunk against the current k-th value and inserts what passes.  Returns
  // false, with nothing inserted, when more candidates passed than the buffer holds (only while the threshold is
  // still loose: the caller then repeats the range in 1024-label slices, which always fit).
  auto scan_and_insert = [&](int64_t c0, int n_sub) -> bool {
    const float thr = sv[k - 1];
    for (int sub0 = 0; sub0 < n_sub; sub0 += TK_BATCH) {
      // 8 consecutive labels per thread and 1024-label slice; TK_BATCH slices' loads are issued before any is looked at
      // (the scan is a stream out of L2: what it needs is bytes in flight)
      uint4 v[TK_BATCH];
      int64_t j0[TK_BATCH];
#pragma unroll
      for (int u = 0; u < TK_BATCH; ++u) {
        j0[u] = c0 + static_cast<int64_t>(sub0 + u) * TK_CAND + static_cast<int64_t>(tid) * 8;
        v[u] = make_uint4(0xFF80FF80u, 0xFF80FF80u, 0xFF80FF80u, 0xFF80FF80u);     // -inf: never a candidate
        if (sub0 + u < n_sub && j0[u] < C) {
          if (vec_ok && j0[u] + 8 <= C) {
            v[u] = *reinterpret_cast<const uint4*>(zr + j0[u]);
          } else {
            uint16_t t[8];
#pragma unroll
            for (int p = 0; p < 8; ++p) t[p] = (j0[u] + p < C) ? zr[j0[u] + p] : uint16_t(0xFF80);
            v[u] = make_uint4(t[0] | (uint32_t(t[1]) << 16), t[2] | (uint32_t(t[3]) << 16), t[4] | (uint32_t(t[5]) << 16), t[6] | (uint32_t(t[7]) << 16));
          }
        }
      }
#pragma unroll
      for (int u = 0; u < TK_BATCH; ++u) {
        const uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
        for (int p = 0; p < 8; ++p) {
          const float e = (p & 1) ? __uint_as_float(w[p >> 1] & 0xFFFF0000u) : __uint_as_float(w[p >> 1] << 16);
          if (e > thr) {                                      // -inf never passes; a NaN logit is never selected
            const int slot = atomicAdd(&ncand, 1);
            if (slot < TK_CAND) { cv[slot] = e; ci[slot] = static_cast<int>(col0 + j0[u] + p); }
          }
        }
      }
    }
    __syncthreads();
    const int n = ncand;
    __syncthreads();
    if (tid == 0) ncand = 0;
    if (n > TK_CAND) { __syncthreads(); return false; }
    // ---- merge the candidates into the kept list, up to TK_THREADS at a time.  Every element's new position is the
    // number of elements ahead of it (larger value, or equal value and lower label id: a strict order, label ids are
    // distinct): a kept entry moves down by the candidates ahead of it, a candidate lands behind the kept entries
    // ahead of it (binary search in the sorted list) and the other candidates ahead of it.  Two barriers per batch,
    // however many candidates it holds.
    for (int base = 0; base < n; base += TK_THREADS) {
      const int m = min(TK_THREADS, n - base);
      float ov = 0.f, cvv = 0.f;
      int oi = 0, cid = 0, opos = k, cpos = k;
      if (tid < k) {
        ov = sv[tid]; oi = si[tid];
        int ahead = 0;
        for (int c = 0; c < m; ++c) {
          const float v = cv[base + c];
          ahead += (v > ov) || (v == ov && ci[base + c] < oi);
        }
        opos = tid + ahead;
      }
      if (tid < m) {
        cvv = cv[base + tid]; cid = ci[base + tid];
        int lo = 0, hi = k;                                   // first kept entry that is not ahead of the candidate
        while (lo < hi) {
          const int mid = (lo + hi) >> 1;
          const bool ahead = sv[mid] > cvv || (sv[mid] == cvv && si[mid] >= 0 && si[mid] < cid);
          if (ahead) lo = mid + 1; else hi = mid;
        }
        int ahead_c = 0;
        for (int c = 0; c < m; ++c) {
          const float v = cv[base + c];
          ahead_c += (v > cvv) || (v == cvv && ci[base + c] < cid);
        }
        cpos = lo + ahead_c;
      }
      __syncthreads();
      if (opos < k) { sv[opos] = ov; si[opos] = oi; }
      if (cpos < k) { sv[cpos] = cvv; si[cpos] = cid; }
      __syncthreads();
    }
    __syncthreads();
    return true;
  };
  // Once the threshold has tightened candidates are rare (about k ln(L/k) per row over the whole label set), so the
  // chunk is walked in ranges of TK_WIDE slices with one synchronisation per range instead of one per slice.
  for (int64_t c0 = 0; c0 < C; c0 += static_cast<int64_t>(TK_WIDE) * TK_CAND) {
    const bool loose = sv[k - 1] == -INFINITY;                // fewer than k labels seen so far: every label is a candidate
    if (loose || !scan_and_insert(c0, TK_WIDE)) {
      for (int sub = 0; sub < TK_WIDE && c0 + static_cast<int64_t>(sub) * TK_CAND < C; ++sub) scan_and_insert(c0 + static_cast<int64_t>(sub) * TK_CAND, 1);
    }
  }
  if (tid < k) { vals[b * k + tid] = sv[tid]; idx[b * k + tid] = si[tid]; }
}

int launch_topk_update(const void* z, int64_t ldz, int64_t B, int64_t C, int64_t col0, int k, float* vals, int32_t* idx, cudaStream_t st) {
  if (B == 0 || C == 0) return HASTE_OK;
  topk_update_kernel<<<static_cast<unsigned>(B), TK_THREADS, 0, st>>>(static_cast<const uint16_t*>(z), ldz, C, col0, k, vals, idx);
  return check_launch("topk_update_kernel");
}

}  // namespace haste
