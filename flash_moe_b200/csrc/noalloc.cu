// fmoe_expert_forward_static: the fine-grained expert forward for callers that cannot hand the
// library any scratch memory.
//
// Some hosts of this library have no way to allocate device memory at the point where they call
// it: code running under a framework whose allocator is off limits while a memory plan is frozen
// (an inference engine after its warm-up, a real-time loop with a fixed memory budget), or a
// binding from a language runtime that can pass the tensors it owns but has no device allocator
// of its own.  For them the scratch area of the expert forward lives inside the library image, in
// a file-scope __device__ array of kStaticScratchBytes (8 MiB) that every GPU loading the library
// carries until the process exits.
//
// Rules that follow from sharing one array:
//   * shapes whose scratch need (fmoe_expert_workspace_bytes) exceeds 8 MiB are refused with
//     FMOE_ERR_WORKSPACE - use fmoe_expert_forward with your own workspace for those;
//   * the array keeps whatever the previous call left in it; the parts that must start at zero
//     (the per-expert counters of the expert-centric schedule) are cleared on the stream by every
//     call, nothing else is assumed about its contents;
//   * two calls that overlap on the GPU (different streams, no ordering between them) race on
//     the array - serialise them on one stream or with events;
//   * the first call on each device resolves the array's device address (cudaGetSymbolAddress) - with lazy module
//     loading that can be when the driver loads this library's device code, the 8 MiB included; make that first call
//     during warm-up, outside any stream capture.
#include <atomic>

#include "common.cuh"

namespace fmoe {
namespace {

constexpr size_t kStaticScratchBytes = 8u << 20;
static __device__ __align__(256) unsigned char g_expert_scratch[kStaticScratchBytes];

// In host code `g_expert_scratch` is only a handle for the runtime, not an address a kernel can
// use; the device address is looked up once per device, with that device current.
// Host threads may race to fill a slot: they all look up the same address, and the slot is atomic.
int static_scratch(void** out) {
  static std::atomic<void*> cache[64];
  int dev = 0;
  FMOE_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return FMOE_ERR_UNSUPPORTED;
  void* p = cache[dev].load(std::memory_order_acquire);
  if (p == nullptr) {
    FMOE_CUDA_TRY(cudaGetSymbolAddress(&p, g_expert_scratch));
    if (p == nullptr) return -static_cast<int>(cudaErrorInvalidSymbol);
    cache[dev].store(p, std::memory_order_release);
  }
  *out = p;
  return FMOE_OK;
}

}  // namespace
}  // namespace fmoe

extern "C" {

size_t fmoe_expert_static_scratch_bytes(void) { return fmoe::kStaticScratchBytes; }

int fmoe_expert_forward_static(const void* x, const void* down, const void* up, const int64_t* indices,
                               const void* gates, void* out, int dtype, int out_dtype, int64_t num_tokens, int hidden,
                               int64_t num_experts, int top_k, int32_t* status, fmoe_stream_t stream) {
  if (dtype != FMOE_DTYPE_F32 && dtype != FMOE_DTYPE_BF16 && dtype != FMOE_DTYPE_F16) return FMOE_ERR_BAD_ARG;
  if (num_tokens < 0 || hidden <= 0 || num_experts <= 0 || top_k < 0) return FMOE_ERR_BAD_ARG;
  const size_t need = fmoe::expert_workspace_bytes(num_tokens, hidden, num_experts, top_k);
  if (need > fmoe::kStaticScratchBytes) return FMOE_ERR_WORKSPACE;  // beyond the built-in 8 MiB
  void* scratch = nullptr;
  const int rc = fmoe::static_scratch(&scratch);
  if (rc != FMOE_OK) return rc;
  return fmoe::launch_expert_forward(x, down, up, indices, gates, out, dtype, out_dtype, num_tokens, hidden,
                                     num_experts, top_k, scratch, fmoe::kStaticScratchBytes, status,
                                     static_cast<cudaStream_t>(stream));
}

}  // extern "C"
