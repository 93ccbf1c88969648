// Fused tcgen05 train step, instantiated for group size 128, fan-in 64 (the 670K- and 2.8M-label configurations).
#include "ffi_step_sm100.cuh"

namespace haste {
int launch_train_step_sm100_g128f64(const int32_t* loc, const void* xt, const int32_t* tgt_ptr, const uint32_t* tgt_ent, float* dxt,
                                    float* loss, const UpdateArgs& u, int64_t B, int64_t D, int64_t L, int loss_kind, float grad_scale,
                                    int max_ctas, cudaStream_t st, const StepDump* dump) {
  return s100::launch_step_shape<128, 64>(loc, xt, tgt_ptr, tgt_ent, dxt, loss, u, B, D, L, loss_kind, grad_scale, max_ctas, st, dump);
}
}  // namespace haste
