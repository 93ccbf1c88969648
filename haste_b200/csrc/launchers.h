// Host-side launcher declarations shared between the kernel translation units and api.cu.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace haste {

// Everything the fused weight/bias update needs.  mom_* are NULL when momentum is off.
struct UpdateArgs {
  __nv_bfloat16* w;
  __nv_bfloat16* bias;
  float* mom_w;
  float* mom_b;
  float lr, wd, mu;
  uint64_t seed;
  uint32_t step, flags;
  int64_t label0;   // global index of the shard's first label (random-bit counters are global)
};

// zw: writable width of a row of z, L <= zw <= ldz (columns L..zw-1 receive zeros)
int launch_forward(const int32_t* loc, const void* xt, const void* w, const void* bias, void* z, int64_t B, int64_t D, int64_t F,
                   int64_t L, int64_t G, int64_t ldz, int64_t zw, cudaStream_t st);
bool forward_sm100_supported(const void* z, const void* xt, const void* w, int64_t B, int64_t F, int64_t L, int64_t G, int64_t ldz);
int launch_forward_sm100(const int32_t* loc, const void* xt, const void* w, const void* bias, void* z, int64_t B, int64_t D, int64_t F,
                         int64_t L, int64_t G, int64_t ldz, int64_t zw, cudaStream_t st);
int launch_bwd_features(const void* w, const int32_t* loc, const void* dy, float* dxt, int64_t B, int64_t D, int64_t F, int64_t L,
                        int64_t G, int64_t ldy, cudaStream_t st);
int launch_bwd_weights(const void* xt, const int32_t* loc, const void* dy, void* dw, void* dbias, const UpdateArgs* upd, int64_t B,
                       int64_t D, int64_t F, int64_t L, int64_t G, int64_t ldy, cudaStream_t st);
int launch_train_step_mma(const int32_t* loc, const void* xt, const int32_t* tgt_ptr, const uint32_t* tgt_ent, float* dxt, float* loss,
                          const UpdateArgs& u, int64_t B, int64_t D, int64_t F, int64_t L, int64_t G, int loss_kind, float grad_scale,
                          cudaStream_t st);
// Optional debug outputs of the tcgen05 fused step (tests only).
struct StepDump {
  void* z;       // bf16 [B, ldz] logits as rounded by the epilogue
  int64_t ldz;
  void* dw;      // bf16 [L,F] weight gradient consumed by the update
  void* dbias;   // bf16 [L]
};

// tcgen05 fused step: one translation unit per layer shape.  max_ctas > 0 caps the persistent grid (SMs left free for
// kernels of other streams).
int launch_train_step_sm100_g128f64(const int32_t* loc, const void* xt, const int32_t* tgt_ptr, const uint32_t* tgt_ent, float* dxt,
                                    float* loss, const UpdateArgs& u, int64_t B, int64_t D, int64_t L, int loss_kind, float grad_scale,
                                    int max_ctas, cudaStream_t st, const StepDump* dump);
int launch_train_step_sm100_g64f128(const int32_t* loc, const void* xt, const int32_t* tgt_ptr, const uint32_t* tgt_ent, float* dxt,
                                    float* loss, const UpdateArgs& u, int64_t B, int64_t D, int64_t L, int loss_kind, float grad_scale,
                                    int max_ctas, cudaStream_t st, const StepDump* dump);
int launch_train_step(const int32_t* loc, const void* xt, const int32_t* tgt_ptr, const uint32_t* tgt_ent, float* dxt, float* loss,
                      const UpdateArgs& u, int64_t B, int64_t D, int64_t F, int64_t L, int64_t G, int loss_kind, float grad_scale,
                      cudaStream_t st, const StepDump* dump = nullptr);
int launch_sr_round(const float* x, void* out, int64_t n, uint64_t seed, cudaStream_t st);
int launch_sgd_sr(void* w, const void* g, float* m, int64_t rows, int64_t cols, int64_t row0, float lr, float wd, float mu, uint64_t seed,
                  uint32_t step, uint32_t flags, cudaStream_t st);
int launch_dxt_to_dx(const float* dxt, void* dx, int64_t B, int64_t D, uint64_t seed, cudaStream_t st);
int launch_transpose(const void* x, void* xt, int64_t B, int64_t D, cudaStream_t st);
int launch_targets_bucket(const int32_t* coo, int64_t nnz, int64_t label0, int64_t L, int64_t G, int32_t* ptr, uint32_t* ent,
                          int32_t* scratch, cudaStream_t st);
int launch_targets_bucket_noalloc(const int32_t* coo, int64_t nnz, int64_t label0, int64_t L, int64_t G, int32_t* ptr, uint32_t* ent,
                                  cudaStream_t st);
int launch_step_prepare(const void* x, void* xt, float* dxt, float* loss, const int32_t* coo, int64_t nnz, int64_t label0, int64_t L,
                        int64_t G, int32_t* ptr, uint32_t* ent, int64_t B, int64_t D, cudaStream_t st);
bool backward_sm100_supported(const void* xt, const void* w, const void* dy, const void* dw, int64_t B, int64_t D, int64_t F, int64_t L,
                              int64_t G);
int launch_backward_sm100(const void* xt, const void* w, const int32_t* loc, const void* dy, float* dxt, void* dw, void* dbias,
                          const UpdateArgs* upd, int64_t B, int64_t D, int64_t F, int64_t L, int64_t G, int64_t ldy, cudaStream_t st);
int launch_pad_rows(const void* src, int64_t ld_src, void* dst, int64_t ld_dst, int64_t rows, int64_t cols, cudaStream_t st);
int launch_topk_update(const void* z, int64_t ldz, int64_t B, int64_t C, int64_t col0, int k, float* vals, int32_t* idx, cudaStream_t st);
int launch_check_loc(const int32_t* loc, int64_t n, int64_t D, cudaStream_t st);
// score_mode 0 mean / 1 max; prune_mode 0 threshold / 1 per-group fraction / 2 global fraction (n_prune is then the
// layer-wide count and scratch holds HASTE_REWIRE_SCRATCH_WORDS(NG, F) words)
int launch_rewire(void* w, int32_t* loc, float* mom, int64_t D, int64_t F, int64_t L, int64_t G, int64_t group0, int score_mode, int prune_mode,
                  float threshold, int64_t n_prune, int regrow_mode, int init_mode, int regroup, uint64_t seed, uint32_t step,
                  void* scratch, int32_t* changed, cudaStream_t st, uint32_t tie_base = 0);
// layer-wide selection in phases, for a layer sharded over ranks (the caller sums the histograms between the phases)
int launch_rewire_select_begin(const void* w, int64_t F, int64_t L, int64_t G, int score_mode, void* scratch, cudaStream_t st);
int launch_rewire_select_refine(int64_t F, int64_t L, int64_t G, int64_t k, void* scratch, cudaStream_t st);
int launch_rewire_select_finish(int64_t F, int64_t L, int64_t G, void* scratch, cudaStream_t st);

}  // namespace haste
