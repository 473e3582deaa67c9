// dk_sample_depthwise_backward_filter_noalloc: the bank gradient of the local deformable kernel
// for callers that cannot hand the library a workspace.
//
// Who needs this: code that runs where device memory must not be requested at call time -- a
// plugin called from inside somebody else's memory-planned runtime, a real-time or safety loop
// whose memory is fixed at start-up, a host program written in a language whose FFI owns no CUDA
// allocator.  Such callers can pass their own input and output tensors but have nowhere to get
// the partial-sum buffer that dk_sample_depthwise_backward_filter asks for.  Here that buffer is
// a fixed array that lives inside the library image itself, so the call path contains no
// cudaMalloc / cudaFree and no allocating library routine.
//
// Costs and rules, all consequences of the buffer being one static array:
//   * every GPU that loads the library carries kScratchBytes of it until the process exits;
//   * shapes whose partial sums need more than kScratchBytes are refused (DK_ERR_WORKSPACE);
//   * all calls on a device share the array: two calls that overlap on the GPU (different
//     streams, different host threads) race on it -- serialise them;
//   * the kernels overwrite every partial they later read, so nothing needs clearing between calls
//     although the array keeps the previous call's contents;
//   * the first call on each device looks up the array's device address (no allocation, but a
//     runtime query), so make that first call before starting any stream capture.
#include <mutex>

#include "dk_common.cuh"

namespace dk {
namespace {

constexpr size_t kScratchBytes = 8u << 20;  // 8 MiB: covers every layer of the MobileNetV2 sweep at batch 128
static __device__ __align__(256) unsigned char g_filter_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_mutex;
void* g_scratch_ptr[kMaxDevices];  // device address of g_filter_scratch, per device; null = not looked up yet

// In host code `g_filter_scratch` is only a handle for the runtime, not an address a kernel can
// use; the address valid on the CURRENT device comes from cudaGetSymbolAddress.
int scratch_for_current_device(void** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    set_last_cuda_error(e);
    return DK_ERR_CUDA;
  }
  if (dev < 0 || dev >= kMaxDevices) return DK_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_filter_scratch);
    if (e != cudaSuccess || p == nullptr) {
      set_last_cuda_error(e);
      return DK_ERR_CUDA;
    }
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return DK_OK;
}

}  // namespace
}  // namespace dk

using namespace dk;

extern "C" {

size_t dk_sample_depthwise_backward_filter_noalloc_max_bytes(void) { return kScratchBytes; }

int dk_sample_depthwise_backward_filter_noalloc(const void* grad_output, const void* input, const void* rotation,
                                                void* grad_filter, const dk_geom* g, int dtype, void* stream) {
  Geom gg;
  if (!grad_output || !input || !rotation || !grad_filter || !make_geom(g, &gg)) return DK_ERR_BAD_ARGUMENT;
  if (dtype != DK_F32 && dtype != DK_F16 && dtype != DK_F64) return DK_ERR_BAD_ARGUMENT;
  const size_t need = dk_sample_depthwise_backward_filter_workspace_bytes(g, dtype);
  if (need > kScratchBytes) return DK_ERR_WORKSPACE;  // shape too large for the built-in scratch
  void* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case DK_F32:
      return local_backward_filter<float>((const float*)grad_output, (const float*)input, (const float*)rotation,
                                          (float*)grad_filter, gg, scratch, kScratchBytes, s);
    case DK_F16:
      return local_backward_filter<__half>((const __half*)grad_output, (const __half*)input, (const __half*)rotation,
                                           (__half*)grad_filter, gg, scratch, kScratchBytes, s);
    default:
      return local_backward_filter<double>((const double*)grad_output, (const double*)input, (const double*)rotation,
                                           (double*)grad_filter, gg, scratch, kScratchBytes, s);
  }
}

}  // extern "C"
