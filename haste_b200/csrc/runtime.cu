// Host-side plumbing shared by the tcgen05 kernels: the status word their bounded waits report through, the wait
// limit, and tensor-map construction for the TMA producers.
#include "common.cuh"
#include "runtime.h"

#include <mutex>

namespace haste {

// ---------------------------------------------------------------- device status word
// One pinned, device-mapped int per process.  A kernel whose bounded wait gives up writes the id of that wait into
// it with a plain store and returns normally; the host reads it after synchronising (haste_poll_status) or at the
// next launch of a kernel that uses it.
static std::mutex g_mu;
static int* g_status_host = nullptr;
static long long g_wait_limit = 4000000000ll;   // clock cycles (~2 s)
static int g_stall_tile = -1;                   // test hook: consumed by the next debug step
static int g_dependent_launch = 1;              // the fused step is launched with programmatic stream serialization

int device_status_word(int** dev_ptr) {
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_status_host == nullptr) {
    int* h = nullptr;
    cudaError_t e = cudaHostAlloc(reinterpret_cast<void**>(&h), sizeof(int), cudaHostAllocMapped | cudaHostAllocPortable);
    if (e != cudaSuccess) return fail(HASTE_ERR_LAUNCH, "cudaHostAlloc(status word): %s", cudaGetErrorString(e));
    *h = 0;
    g_status_host = h;
  }
  cudaError_t e = cudaHostGetDevicePointer(reinterpret_cast<void**>(dev_ptr), g_status_host, 0);
  if (e != cudaSuccess) return fail(HASTE_ERR_LAUNCH, "cudaHostGetDevicePointer(status word): %s", cudaGetErrorString(e));
  return HASTE_OK;
}

int take_device_status() {
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_status_host == nullptr) return 0;
  const int code = *reinterpret_cast<volatile int*>(g_status_host);
  *reinterpret_cast<volatile int*>(g_status_host) = 0;
  return code;
}

int report_pending_status(const char* who) {
  const int code = take_device_status();
  if (code == 0) return HASTE_OK;
  return fail(HASTE_ERR_TIMEOUT, "%s: an earlier kernel gave up waiting on an on-chip barrier (wait id %d); its outputs are invalid", who, code);
}

long long wait_limit_cycles() { return g_wait_limit; }
// The relaxed launch is only used where this library knows what precedes the step in the stream: inside haste_ffi_step,
// right behind its own preparation kernel.  (Behind an event wait on another stream — the pipelined multi-GPU step
// waits for a preparation kernel of a side stream — the relaxed edge would only cover the previous kernel of the
// same stream, and the step could read the batch before it is prepared.)
static thread_local int t_dependent_scope = 0;
void dependent_launch_scope(int on) { t_dependent_scope = on; }
int dependent_launch_enabled() { return g_dependent_launch && t_dependent_scope; }
int take_stall_tile() {
  std::lock_guard<std::mutex> lock(g_mu);
  const int t = g_stall_tile;
  g_stall_tile = -1;
  return t;
}

// ---------------------------------------------------------------- tensor maps
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess || qres != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes, uint32_t box_inner,
                      uint32_t box_outer) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return fail(HASTE_ERR_LAUNCH, "cuTensorMapEncodeTiled is not available from this driver");
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || (row_stride_bytes & 15u) != 0)
    return fail(HASTE_ERR_BAD_ARG, "tensor map: base and row stride must be multiples of 16 bytes");
  const cuuint64_t dims[2] = {inner, outer};
  const cuuint64_t strides[1] = {row_stride_bytes};
  const cuuint32_t box[2] = {box_inner, box_outer};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(HASTE_ERR_LAUNCH, "cuTensorMapEncodeTiled failed (CUresult %d)", static_cast<int>(r));
  return HASTE_OK;
}

}  // namespace haste

extern "C" {

int haste_poll_status(void) { return haste::report_pending_status("haste_poll_status"); }

int haste_debug_set_wait_limit(long long cycles) {
  if (cycles < 1000) return haste::fail(HASTE_ERR_BAD_ARG, "haste_debug_set_wait_limit: %lld cycles is too short", cycles);
  std::lock_guard<std::mutex> lock(haste::g_mu);
  haste::g_wait_limit = cycles;
  return HASTE_OK;
}

int haste_debug_set_dependent_launch(int on) {
  std::lock_guard<std::mutex> lock(haste::g_mu);
  haste::g_dependent_launch = on ? 1 : 0;
  return HASTE_OK;
}

int haste_debug_stall_next_step(int tile) {
  std::lock_guard<std::mutex> lock(haste::g_mu);
  haste::g_stall_tile = tile;
  return HASTE_OK;
}

}  // extern "C"
