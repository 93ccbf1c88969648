// Host-side plumbing shared by the tcgen05 kernels (implemented in runtime.cu).
#pragma once
#include <cuda.h>
#include <stdint.h>

namespace haste {

// Device address of the process-wide status word (allocated on first use; thread-safe).  Returns a status code.
int device_status_word(int** dev_ptr);
// Reads and clears the status word; 0 = no kernel reported anything.
int take_device_status();
// HASTE_OK, or HASTE_ERR_TIMEOUT (with message) when a kernel that finished earlier had given up on a wait.
int report_pending_status(const char* who);
// Clock cycles a device-side wait may last before it gives up.
long long wait_limit_cycles();
// 1: the fused step about to be launched by this thread may start its set-up while the preceding kernel of the
// stream finishes (only inside dependent_launch_scope(1), and unless switched off for measurement).
int dependent_launch_enabled();
void dependent_launch_scope(int on);
// Test hook: tile index at which the next debug step withholds one barrier arrival (-1 = none); reading clears it.
int take_stall_tile();

// 2-D bf16 tensor map [outer][inner] with the 128-byte swizzle, zero fill outside the tensor.
int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes, uint32_t box_inner,
                      uint32_t box_outer);

}  // namespace haste
