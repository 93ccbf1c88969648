/*
 * haste_ffi.h — C ABI of the B200 (sm_100a) fixed-fan-in (FFI) output-layer kernels.
 *
 * This is the drop-in boundary for the training hot path of HASTE's grouped fixed-fan-in sparse
 * output layer.  Every entry point takes raw device pointers, 64-bit sizes, scalar
 * hyper-parameters and a CUDA stream, returns an int status (0 = ok) and never throws.
 * After a non-zero status, haste_last_error_string() describes the failure (thread-local).
 * The caller makes the target device current before calling; all work is enqueued on `stream`.
 *
 * Notation: B batch, D input features, L labels (of this shard), F fan-in, G group size,
 * NG = ceil(L/G).  bf16 tensors are passed as `const void*` / `void*` (2 bytes per element).
 *   loc   int32 [NG,F]   input-feature index table, one row per group of G consecutive labels
 *   xt    bf16  [D,B]    features TRANSPOSED (batch contiguous), as the reference's kernels take them
 *   w     bf16  [L,F]    weights
 *   bias  bf16  [L]      optional (NULL = none)
 *   z/dy  bf16  [B,ld]   logits / dLoss/dLogits, row stride `ld` elements (ld >= L)
 *   dxt   fp32  [D,B]    gradient w.r.t. xt
 *
 * Supported shapes: G in {16,32,64,128}; F a multiple of 16, 16 <= F <= 128; B >= 1; any L >= 1.
 * (The reference supports G in {16,32,64}: shared_ffi/rewire.py:120.)
 */
#ifndef HASTE_FFI_H
#define HASTE_FFI_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* haste_stream_t; /* a cudaStream_t */

enum {
  HASTE_OK = 0,
  HASTE_ERR_BAD_ARG = 1,     /* null pointer, negative size, misaligned base pointer */
  HASTE_ERR_UNSUPPORTED = 2, /* (G,F) or size outside the supported set */
  HASTE_ERR_INDEX_RANGE = 3, /* loc holds a value outside [0,D) (haste_ffi_check_locations) */
  HASTE_ERR_LAUNCH = 4,      /* CUDA reported an error at launch */
  HASTE_ERR_TIMEOUT = 5,     /* a bounded device-side wait gave up */
  HASTE_ERR_TOO_LARGE = 6    /* size beyond a documented fixed capacity */
};

/* loss_kind */
enum { HASTE_LOSS_BCE = 0, HASTE_LOSS_SQHINGE = 1 };

/* flags for the update / train-step entry points */
enum {
  HASTE_F_SR = 1u << 0,          /* stochastic rounding to bf16 (else round-to-nearest-even) */
  HASTE_F_CONTRACT = 1u << 1,    /* fp32 update uses fused multiply-add, as the reference's compiled
                                    Triton kernel does; clear = separate multiply and add */
  HASTE_F_RNG_PACKED = 1u << 2,  /* random bits: one Philox4x32-10 call per 8 slots, key (seed,step),
                                    counter (global label, slot>>3,0,0); clear = the reference stream
                                    (tl.randint: key seed, counter flat element index, word 0) */
  HASTE_F_ZERO_DXT = 1u << 3,    /* clear dxt on the stream before accumulating into it */
  HASTE_F_LOSS = 1u << 4         /* accumulate the loss value into *loss */
};

const char* haste_last_error_string(void);
int haste_version(void);

/* Forward: z[b,l] = sum_k xt[loc[l/G,k], b] * w[l,k] + bias[l], fp32 accumulate, RN to bf16.
 * Columns L..ldz-1 of z are written with zeros when ldz > L (the reference pads to a multiple of 8).
 * Replaces ffi_forward_cuda (shared_ffi/ffi_forward_kernels.cu:492-719, bound at ffi_wrapper.cpp:32-44). */
int haste_ffi_forward(const int32_t* loc, const void* xt, const void* w, const void* bias, void* z,
                      int64_t B, int64_t D, int64_t F, int64_t L, int64_t G, int64_t ldz,
                      haste_stream_t stream);

/* The same forward writing into a block of columns of a wider matrix: z points at the block's first column of
 * row 0, ldz is the wider matrix's row stride, and only columns 0..zcols-1 of each row (relative to z) are written —
 * L logits, zeros in L..zcols-1.  With it the sparse tail's logits land next to a dense head's in one [B, L_head +
 * L_tail] buffer, where the reference concatenates two tensors (src/model.py:245-248). */
int haste_ffi_forward_into(const int32_t* loc, const void* xt, const void* w, const void* bias, void* z,
                           int64_t B, int64_t D, int64_t F, int64_t L, int64_t G, int64_t ldz, int64_t zcols,
                           haste_stream_t stream);

/* Backward w.r.t. features: dxt[loc[g,k], b] += sum_{l in g} w[l,k] * dy[b,l]  (fp32 atomics).
 * flags: HASTE_F_ZERO_DXT clears dxt first (the reference allocates zeros).
 * Replaces ffi_backward_features_cuda (shared_ffi/ffi_backward_features.cu:417-633). */
int haste_ffi_backward_features(const void* w, const int32_t* loc, const void* dy, float* dxt,
                                int64_t B, int64_t D, int64_t F, int64_t L, int64_t G, int64_t ldy,
                                uint32_t flags, haste_stream_t stream);

/* Backward w.r.t. weights: dw[l,k] = sum_b dy[b,l] * xt[loc[l/G,k], b], RN to bf16;
 * dbias (optional, bf16 [L]) = column sums of dy (shared_ffi/bindings.py:39-42).
 * Replaces ffi_backward_weights_cuda (shared_ffi/ffi_backward_weights.cu:486-684). */
int haste_ffi_backward_weights(const void* xt, const int32_t* loc, const void* dy, void* dw, void* dbias,
                               int64_t B, int64_t D, int64_t F, int64_t L, int64_t G, int64_t ldy,
                               haste_stream_t stream);

/* Both gradients of the autograd backward from one pass over dy: dxt as haste_ffi_backward_features, dw / dbias
 * as haste_ffi_backward_weights (dbias may be NULL).  For (G=128, F=64) and (G=64, F=128) with B % 8 == 0 one
 * tcgen05 kernel reads dy once; its rows need no alignment beyond that of a bf16 (a contiguous [B, L] gradient
 * with odd L is read in place) and whatever lies in columns L..ldy-1 is ignored.  Otherwise the two warp-mma
 * kernels run back to back.  flags: HASTE_F_ZERO_DXT.
 * Replaces the pair of calls at shared_ffi/bindings.py:44 and :52. */
int haste_ffi_backward(const void* xt, const void* w, const int32_t* loc, const void* dy, float* dxt, void* dw, void* dbias,
                       int64_t B, int64_t D, int64_t F, int64_t L, int64_t G, int64_t ldy, uint32_t flags,
                       haste_stream_t stream);

/* Copy a bf16 [rows, cols] matrix (row stride ld_src) into [rows, ld_dst] with zeros in columns cols..ld_dst-1
 * (ld_dst % 8 == 0, dst 16-byte aligned): a utility for callers that want 16-byte aligned gradient rows (no
 * entry point of this library needs them; the reference calls grad_output.contiguous() at
 * shared_ffi/bindings.py:37). */
int haste_pad_rows_bf16(const void* src, int64_t ld_src, void* dst, int64_t ld_dst, int64_t rows, int64_t cols,
                        haste_stream_t stream);

/* Backward-weights fused with the SGD(+weight decay)(+momentum) stochastic-rounding update: the
 * gradient is rounded to bf16 exactly as haste_ffi_backward_weights would store it and consumed in
 * registers; w (and bias, momentum buffers when given) are updated in place.
 * label0 = global index of this shard's first label (random-bit counters use global indices).
 * Replaces ffi_backward_weights_cuda followed by sr_triton.sgd_update
 * (shared_ffi/sr_triton.py:172-213, called from shared_ffi/optim_sr.py:99-109). */
int haste_ffi_bww_sr_sgd(const void* xt, const int32_t* loc, const void* dy, void* w, void* bias,
                         float* mom_w, float* mom_b,
                         int64_t B, int64_t D, int64_t F, int64_t L, int64_t G, int64_t ldy, int64_t label0,
                         float lr, float wd, float mu, uint64_t seed, uint32_t step, uint32_t flags,
                         haste_stream_t stream);

/* Bucket COO targets (row, col) int32 [nnz,2] by label group for the fused step.
 * Keeps entries with label0 <= col < label0+L.  Outputs: tgt_ptr int32 [NG+1] (CSR offsets),
 * tgt_ent uint32 [nnz] = (row << 8) | (col - label0) % G.  `scratch` is NG int32 of device memory.
 * The COO layout is the reference collate's (src/data.py:26-46). */
int haste_targets_bucket(const int32_t* coo, int64_t nnz, int64_t label0, int64_t L, int64_t G,
                         int32_t* tgt_ptr, uint32_t* tgt_ent, int32_t* scratch, haste_stream_t stream);

/* Everything the fused step needs per batch, in one launch: xt = transpose(x [B,D] bf16), dxt cleared, *loss
 * cleared (loss may be NULL), and the COO targets bucketed as by haste_targets_bucket (counters live in shared
 * memory, so no scratch argument; at most ~51,000 label groups — HASTE_ERR_TOO_LARGE beyond).  `coo` must be
 * 8-byte aligned (any row of an int32 [nnz,2] tensor is).
 * Replaces the transpose of shared_ffi/bindings.py:19 and the per-step zero fills. */
int haste_ffi_step_prepare(const void* x, void* xt, float* dxt, float* loss, const int32_t* coo, int64_t nnz,
                           int64_t label0, int64_t L, int64_t G, int32_t* tgt_ptr, uint32_t* tgt_ent,
                           int64_t B, int64_t D, haste_stream_t stream);

/* haste_targets_bucket for callers that must not allocate device memory.  (No counterpart in the reference.)
 *
 * Who needs it: a host that gave all device memory to its own arena at start-up and has nothing left to hand
 * out, a step loop that cannot afford the device-wide synchronisation a cudaMalloc/cudaFree may cause, or a
 * plugin that only receives raw pointers and has no allocator of the hosting framework within reach.  Such
 * callers cannot provide the `scratch` array of haste_targets_bucket; here it lives in a fixed 256 KiB array
 * inside the library (one int32 per label group) that every GPU which loads the library holds until exit.
 *
 * Same inputs, outputs and result as haste_targets_bucket.  Limits and rules:
 *   - at most 65536 label groups (ceil(L/G)); more returns HASTE_ERR_TOO_LARGE — use haste_targets_bucket then;
 *   - the first call on each device looks up the array's device address (the device must be current, as for
 *     every call; the lookup is serialised between host threads); make that first call before starting any
 *     stream capture;
 *   - all calls on a device share the one array: two calls that may overlap on the GPU (different streams)
 *     race — order them.  The array keeps the last call's contents; each call clears the part it uses itself;
 *   - calls no cudaMalloc / cudaFree nor any allocating library routine. */
int haste_targets_bucket_noalloc(const int32_t* coo, int64_t nnz, int64_t label0, int64_t L, int64_t G,
                                 int32_t* tgt_ptr, uint32_t* tgt_ent, haste_stream_t stream);

/* Fused training step of the layer for one label shard:
 *   z = forward; dy = grad_scale * dLoss/dz (BCE-with-logits sum, or squared hinge);
 *   dxt += backward-features; w,bias <- SGD(+wd)(+momentum) + stochastic rounding of backward-weights.
 * Neither z nor dy nor dw is written to memory.  Targets come from haste_targets_bucket.
 * loss (optional fp32 device scalar) is accumulated into when HASTE_F_LOSS is set.
 * Replaces GroupFFIMulFunction.forward/backward (shared_ffi/bindings.py:12-54), the loss of
 * src/runner.py:469-494 and SRSgd.step (shared_ffi/optim_sr.py:46-114) for this layer. */
int haste_ffi_train_step(const int32_t* loc, const void* xt, void* w, void* bias,
                         float* mom_w, float* mom_b,
                         const int32_t* tgt_ptr, const uint32_t* tgt_ent,
                         float* dxt, float* loss,
                         int64_t B, int64_t D, int64_t F, int64_t L, int64_t G, int64_t label0,
                         int32_t loss_kind, float grad_scale, float lr, float wd, float mu,
                         uint64_t seed, uint32_t step, uint32_t flags, haste_stream_t stream);

/* Same step with debug outputs (tests): z_dump bf16 [B,ldz] receives the logits as the epilogue rounded them,
 * dw_dump bf16 [L,F] / dbias_dump bf16 [L] the gradients the update consumed; any of them may be NULL.
 * Only the tcgen05 kernel ((G,F) = (128,64) or (64,128), B%8==0, no momentum) implements them; other shapes return
 * HASTE_ERR_UNSUPPORTED.  No counterpart in the reference (its logits and gradients are ordinary tensors). */
int haste_ffi_train_step_dbg(const int32_t* loc, const void* xt, void* w, void* bias,
                             float* mom_w, float* mom_b,
                             const int32_t* tgt_ptr, const uint32_t* tgt_ent,
                             float* dxt, float* loss,
                             int64_t B, int64_t D, int64_t F, int64_t L, int64_t G, int64_t label0,
                             int32_t loss_kind, float grad_scale, float lr, float wd, float mu,
                             uint64_t seed, uint32_t step, uint32_t flags,
                             void* z_dump, int64_t ldz, void* dw_dump, void* dbias_dump, haste_stream_t stream);

/* Cap the grid of the persistent fused-step kernel at n CTAs (0 = one per SM, the default).  A multi-GPU caller
 * leaves a few SMs free this way, so that the collective of the previous step and the preparation of the next one,
 * enqueued on other streams, run beside the kernel instead of after it.  Process-wide; no counterpart in the
 * reference (it has neither a persistent kernel nor a collective on this path). */
int haste_ffi_set_max_ctas(int32_t n);

/* Status of the kernels with bounded device-side waits (the tcgen05 step, forward and backward).  A wait that runs
 * out makes its kernel return by itself with its outputs invalid and records the fact; this call reports and clears
 * it: HASTE_OK, or HASTE_ERR_TIMEOUT with the wait's id in the message.  Synchronise the stream first.  The next
 * launch of one of those kernels reports a pending record too.  No counterpart in the reference (its kernels
 * have no waits). */
int haste_poll_status(void);

/* Test hooks for the path above.  haste_debug_set_wait_limit: clock cycles a device-side wait may last (default
 * 4e9, about two seconds).  haste_debug_stall_next_step: the next haste_ffi_train_step_dbg call withholds one
 * barrier arrival at batch tile `tile` of every CTA, so that the waits behind it run out; nothing faults or
 * traps, the kernel drains and returns. */
int haste_debug_set_wait_limit(long long cycles);
int haste_debug_stall_next_step(int32_t tile);
/* Inside haste_ffi_step the fused step is launched so that its set-up (barriers, shared memory, TMEM) may overlap
 * the tail of the preparation kernel before it (programmatic dependent launch; it waits for that kernel before it
 * reads anything); haste_debug_set_dependent_launch(0) launches it the ordinary way (measurement of the
 * difference).  haste_ffi_train_step on its own is always launched the ordinary way. */
int haste_debug_set_dependent_launch(int32_t on);

/* Elementwise stochastic rounding fp32 -> bf16 with the reference stream over the flat index.
 * Replaces sr_triton.stochastic_rounding (shared_ffi/sr_triton.py:27-59). */
int haste_sr_round(const float* x, void* out, int64_t n, uint64_t seed, haste_stream_t stream);

/* Elementwise SGD(+wd)(+momentum) + SR/RN on a [rows,cols] bf16 parameter, in place.
 * grad is bf16 [rows,cols]; mom fp32 or NULL; row0 = global index of the first row.
 * Replaces sr_triton.sgd_update (shared_ffi/sr_triton.py:109-213). */
int haste_sgd_sr_update(void* w, const void* grad, float* mom, int64_t rows, int64_t cols, int64_t row0,
                        float lr, float wd, float mu, uint64_t seed, uint32_t step, uint32_t flags,
                        haste_stream_t stream);

/* dX tail of the autograd backward: transpose fp32 dxt [D,B] to [B,D] and stochastically round to
 * bf16, counter = flat index in [B,D] (shared_ffi/bindings.py:44-50 uses the fixed seed 123). */
int haste_dxt_to_dx_sr(const float* dxt, void* dx, int64_t B, int64_t D, uint64_t seed,
                       haste_stream_t stream);

/* Transpose bf16 x [B,D] -> xt [D,B] (shared_ffi/bindings.py:19 does this with torch). */
int haste_transpose_bf16(const void* x, void* xt, int64_t B, int64_t D, haste_stream_t stream);

/* Rewire: per-group prune of the lowest-score slots, regrow, re-initialise, regroup; in place.
 *   score[g,k] = mean over the group's real rows of |w[l,k]| (fp32, rows summed in order)
 *   prune_mode 0 'threshold': score < threshold; 1 'fraction': the n_prune lowest (ties: lowest slot)
 *   regrow_mode 0 'replace' (uniform with replacement, the reference's rule), 1 'unused'
 *   init_mode 0 'zero', 1 'random' U(+-1/sqrt(F));  regroup != 0 sorts each index row ascending and
 *   permutes the group's weight and momentum columns with it.
 * group0 = global index of this shard's first group (random draws use global indices).
 * changed (optional int32 device scalar) receives the number of pruned (group,slot) pairs.
 * Replaces the tensor math of GroupFixedFanIn.rewire (shared_ffi/rewire.py:143-239). */
int haste_ffi_rewire(void* w, int32_t* loc, float* mom_w,
                     int64_t D, int64_t F, int64_t L, int64_t G, int64_t group0,
                     int32_t prune_mode, float threshold, int32_t n_prune,
                     int32_t regrow_mode, int32_t init_mode, int32_t regroup,
                     uint64_t seed, uint32_t step, int32_t* changed, haste_stream_t stream);

/* Rewire with the scoring and pruning rules of the layer class the reference's model instantiates
 * (GroupFixedFanInReal.rewire, src/group_fanin_real.py:149-286):
 *   score_mode 0 'mean' (as above), 1 'max': score[g,k] = max over the group's real rows of |w[l,k]|
 *   prune_mode 0 'threshold', 1 'fraction' per group (n_prune slots of every group, as haste_ffi_rewire),
 *              2 'fraction' over the whole layer: the n_prune = int(NG*F*fraction) lowest scores of all
 *                (group, slot) pairs (src/group_fanin_real.py:232-250); ties at the n_prune-th score go to the
 *                lowest flat (group, slot) index (the reference leaves them to torch.topk).
 * scratch (prune_mode 2 only, 16-byte aligned device memory): HASTE_REWIRE_SCRATCH_WORDS(NG, F) * 4 bytes.
 * Everything else as haste_ffi_rewire.  With a sharded layer "the whole layer" is this shard. */
#define HASTE_REWIRE_SCRATCH_WORDS(NG, F) ((int64_t)(NG) * (F) + (NG) + 2 + 2 * 65536 + 8)
int haste_ffi_rewire_ex(void* w, int32_t* loc, float* mom_w,
                        int64_t D, int64_t F, int64_t L, int64_t G, int64_t group0,
                        int32_t score_mode, int32_t prune_mode, float threshold, int64_t n_prune,
                        int32_t regrow_mode, int32_t init_mode, int32_t regroup,
                        uint64_t seed, uint32_t step, void* scratch, int32_t* changed, haste_stream_t stream);

/* The layer-wide fraction rule for a layer that is sharded over ranks (each rank holds a contiguous label range): the
 * k = int(NG_layer * F * fraction) lowest scores of ALL shards are pruned, as src/group_fanin_real.py:232-250 does on
 * one device.  Every rank makes the same four calls on its shard, with two sums and one gather in between:
 *   haste_ffi_rewire_select_begin   scores of the shard; histogram of their upper 16 bits at word
 *                                   HASTE_REWIRE_HIST_HI_WORD(NG,F) of scratch (65536 uint32)  -> sum it over the ranks
 *   haste_ffi_rewire_select_refine  k_layer = the layer-wide count; histogram of the lower 16 bits inside the k-th
 *                                   score's bin at HASTE_REWIRE_HIST_LO_WORD(NG,F)             -> sum it over the ranks
 *   haste_ffi_rewire_select_finish  threshold and tie bookkeeping; the number of this shard's scores equal to the
 *                                   threshold at HASTE_REWIRE_TIES_WORD(NG,F)                  -> gather over the ranks
 *   haste_ffi_rewire_prepared       prune / regrow / re-initialise / regroup as haste_ffi_rewire_ex does, with
 *                                   tie_base = the sum of that count over the lower-ranked shards (ties at the
 *                                   threshold go to the lowest flat (group, slot) index of the whole layer)
 * NG, L, group0 describe the shard; scratch as for haste_ffi_rewire_ex. */
#define HASTE_REWIRE_HIST_HI_WORD(NG, F) ((int64_t)(NG) * (F) + 2 + (NG))
#define HASTE_REWIRE_HIST_LO_WORD(NG, F) (HASTE_REWIRE_HIST_HI_WORD(NG, F) + 65536)
#define HASTE_REWIRE_TIES_WORD(NG, F) (HASTE_REWIRE_HIST_LO_WORD(NG, F) + 65536 + 4)
int haste_ffi_rewire_select_begin(const void* w, int64_t F, int64_t L, int64_t G, int32_t score_mode, void* scratch,
                                  haste_stream_t stream);
int haste_ffi_rewire_select_refine(int64_t F, int64_t L, int64_t G, int64_t k_layer, void* scratch, haste_stream_t stream);
int haste_ffi_rewire_select_finish(int64_t F, int64_t L, int64_t G, void* scratch, haste_stream_t stream);
int haste_ffi_rewire_prepared(void* w, int32_t* loc, float* mom_w, int64_t D, int64_t F, int64_t L, int64_t G, int64_t group0,
                              int32_t score_mode, uint32_t tie_base, int32_t regrow_mode, int32_t init_mode, int32_t regroup,
                              uint64_t seed, uint32_t step, void* scratch, int32_t* changed, haste_stream_t stream);

/* One training step from the batch as the data loader delivers it: haste_ffi_step_prepare followed by
 * haste_ffi_train_step in one call (two launches, one crossing of the language boundary).  x bf16 [B,D]; coo int32
 * [nnz,2]; xt, dxt, tgt_ptr, tgt_ent are work buffers the caller keeps between steps (sizes as in the two
 * functions); HASTE_F_ZERO_DXT is implied.  Replaces forward + loss + backward + optimizer step of
 * src/runner.py:205-230 for the FFI layer. */
int haste_ffi_step(const void* x, const int32_t* coo, int64_t nnz, const int32_t* loc, void* xt, void* w, void* bias,
                   float* mom_w, float* mom_b, int32_t* tgt_ptr, uint32_t* tgt_ent, float* dxt, float* loss,
                   int64_t B, int64_t D, int64_t F, int64_t L, int64_t G, int64_t label0, int32_t loss_kind,
                   float grad_scale, float lr, float wd, float mu, uint64_t seed, uint32_t step, uint32_t flags,
                   haste_stream_t stream);

/* Fold a chunk of logits into the running per-row top-k (inference; the reference materialises [B,L] logits and
 * calls torch.topk(logits, 100) / topk(5), src/evaluate.py:151-156, 219).  z: bf16 [B, ldz], columns 0..C-1 hold
 * the logits of labels col0 .. col0+C-1.  vals fp32 [B,k] (descending) and idx int32 [B,k] are the state: start
 * them at -inf / -1 and feed the chunks in increasing label order; equal values keep the lower label id first.
 * 1 <= k <= 128. */
int haste_topk_update(const void* z, int64_t ldz, int64_t B, int64_t C, int64_t col0, int32_t k,
                      float* vals, int32_t* idx, haste_stream_t stream);

/* The whole inference top-k in one call: the layer's labels are walked in chunks of `groups_per_chunk` label groups;
 * each chunk's logits go to zbuf (bf16 [B, ldz], ldz >= groups_per_chunk * G, ldz % 8 == 0, 16-byte aligned; sized to
 * stay in L2) through haste_ffi_forward's kernels and are folded into vals / idx by haste_topk_update's kernel, all on
 * `stream` without returning to the host in between.  vals / idx as for haste_topk_update (start at -inf / -1);
 * `label0` is added to the label ids (a shard of a larger layer).  Replaces forward + torch.topk over the full
 * [B,L] logits (src/evaluate.py:151-156, 219). */
int haste_ffi_topk(const int32_t* loc, const void* xt, const void* w, const void* bias, void* zbuf, int64_t ldz, int64_t B,
                   int64_t D, int64_t F, int64_t L, int64_t G, int64_t groups_per_chunk, int32_t k, int64_t label0,
                   float* vals, int32_t* idx, haste_stream_t stream);

/* Rate probes (measurement only; timed by the benchmark's auxiliary mode; no counterpart in the reference).  Each
 * isolates one access pattern of the fused train step at the step's own sizes:
 *   haste_probe_red_rate     fp32 reduce-add of `tiles_per_cta` tiles of 64 rows x 128 floats per SM into dxt [D,B]
 *                            (B % 128 == 0): mode 0 scalar red, one 128-byte transaction per warp instruction (what the
 *                            step issues); 1 red.v4 along one row; 2 red.v4 across 32 rows per warp instruction
 *   haste_probe_gather_rate  gathering `tiles_per_cta` tiles of 64 rows x 256 B of xt [D,B] (bf16) per SM into
 *                            swizzled shared memory: mode 0 / 12 / 14 TMA tile::gather4 issued by 1 / 2 / 4 warps; 1, 2, 4 = cp.async from that many warps
 *   haste_probe_umma_rate    8 * iters back-to-back tcgen05.mma (M=128, K=16, given N and operand majors) on one SM;
 *                            cycles_out (device, 2 x int64) receives the cycles to issue them and to complete them */
int haste_probe_red_rate(float* dxt, int64_t D, int64_t B, int32_t mode, int32_t tiles_per_cta, haste_stream_t stream);
int haste_probe_gather_rate(const void* xt, int64_t D, int64_t B, int32_t mode, int32_t tiles_per_cta, haste_stream_t stream);
int haste_probe_umma_rate(int32_t N, int32_t a_mn_major, int32_t b_mn_major, int32_t iters, long long* cycles_out,
                          haste_stream_t stream);

/* Debug check: every loc value in [0,D).  Synchronises the stream. */
int haste_ffi_check_locations(const int32_t* loc, int64_t n, int64_t D, haste_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* HASTE_FFI_H */
