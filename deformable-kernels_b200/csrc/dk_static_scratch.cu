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
//   * the kernels' partial sums must fit into kScratchBytes.  The call sizes itself for the kernel
//     it will launch: the fp16 tensor-core kernel when that kernel's own partial sums fit, else the
//     general kernel with as many pixel blocks as fit (fewer, larger blocks: slower, same result up
//     to summation order).  A shape is refused (DK_ERR_WORKSPACE) only when a single block's
//     partial sums, channels x bank cells x 4 or 8 bytes, exceed the array: more than 2 Mi (fp16,
//     fp32) or 1 Mi (fp64) bank values.  dk_sample_depthwise_backward_filter_noalloc_bytes tells,
//     without touching a GPU, how much of the array a call would use (0 = refused);
//   * all calls on a device share the array: two calls that overlap on the GPU (different
//     streams, different host threads) race on it -- serialise them;
//   * the kernels overwrite every partial they later read, so nothing needs clearing between calls
//     although the array keeps the previous call's contents;
//   * the first call on each device looks up the array's device address (no allocation, but a
//     runtime query), so make that first call before starting any stream capture;
//   * the tensors must live on the current device: the array is looked up for cudaGetDevice().
#include <mutex>

#include "dk_common.cuh"

namespace dk {
namespace {

constexpr size_t kScratchBytes = 8u << 20;  // 8 MiB
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

// launch = false only sizes the call (need_out), touching no GPU
int run(const void* dy, const void* x, const void* rot, void* dw, const Geom& gg, int dtype, void* scratch, cudaStream_t s,
        bool launch, size_t* need_out) {
  switch (dtype) {
    case DK_F32:
      return local_backward_filter_fit<float>((const float*)dy, (const float*)x, (const float*)rot, (float*)dw, gg, scratch,
                                              kScratchBytes, s, launch, need_out);
    case DK_F16:
      return local_backward_filter_fit<__half>((const __half*)dy, (const __half*)x, (const __half*)rot, (__half*)dw, gg, scratch,
                                               kScratchBytes, s, launch, need_out);
    case DK_F64:
      return local_backward_filter_fit<double>((const double*)dy, (const double*)x, (const double*)rot, (double*)dw, gg, scratch,
                                               kScratchBytes, s, launch, need_out);
    default:
      return DK_ERR_BAD_ARGUMENT;
  }
}

}  // namespace
}  // namespace dk

using namespace dk;

extern "C" {

size_t dk_sample_depthwise_backward_filter_noalloc_max_bytes(void) { return kScratchBytes; }

size_t dk_sample_depthwise_backward_filter_noalloc_bytes(const dk_geom* g, int dtype) {
  Geom gg;
  if (!make_geom(g, &gg)) return 0;
  size_t need = 0;
  if (run(nullptr, nullptr, nullptr, nullptr, gg, dtype, nullptr, nullptr, false, &need) != DK_OK) return 0;
  return need;
}

int dk_sample_depthwise_backward_filter_noalloc(const void* grad_output, const void* input, const void* rotation,
                                                void* grad_filter, const dk_geom* g, int dtype, void* stream) {
  Geom gg;
  if (!grad_output || !input || !rotation || !grad_filter || !make_geom(g, &gg)) return DK_ERR_BAD_ARGUMENT;
  if (dtype != DK_F32 && dtype != DK_F16 && dtype != DK_F64) return DK_ERR_BAD_ARGUMENT;
  size_t need = 0;
  int rc = run(nullptr, nullptr, nullptr, nullptr, gg, dtype, nullptr, nullptr, false, &need);
  if (rc) return rc;  // not even one block's partial sums fit into the built-in scratch
  void* scratch = nullptr;
  rc = scratch_for_current_device(&scratch);
  if (rc) return rc;
  return run(grad_output, input, rotation, grad_filter, gg, dtype, scratch, (cudaStream_t)stream, true, nullptr);
}

}  // extern "C"
