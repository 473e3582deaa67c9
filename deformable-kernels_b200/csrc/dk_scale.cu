// Per-(sample, channel) scaling of feature planes: the global deformable kernel with a 1x1
// depthwise kernel.  There the reference runs F.conv2d(x.view(1, N*C, H, W), weight[N*C,1,1,1],
// groups=N*C) (modules/deform_kernel.py:105-118), i.e. y[n,c,:,:] = x[n,c,:,:] * k[n,c] through a
// grouped convolution with N*C groups.  Here it is one streaming pass, and the backward pass
// produces grad-input and the per-plane reduction grad-k[n,c] = sum(dy * x) together.
#include "dk_common.cuh"

namespace dk {

template <typename T>
__global__ void scale_fwd_kernel(const T* __restrict__ x, const T* __restrict__ k, T* __restrict__ y, long long planes,
                                 int hw) {
  using A = typename Compute<T>::type;
  const int lane = threadIdx.x & 31;
  const long long plane = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (plane >= planes) return;
  const A kv = ld<A>(k + plane);
  const T* xp = x + plane * hw;
  T* yp = y + plane * hw;
  for (int i = lane; i < hw; i += 32) st<T, A>(yp + i, ld<A>(xp + i) * kv);
}

// one warp per plane: dx = dy * k and dk = sum(dy * x) in the same pass
template <typename T>
__global__ void scale_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ k,
                                 T* __restrict__ dx, T* __restrict__ dk, long long planes, int hw) {
  using A = typename Compute<T>::type;
  const int lane = threadIdx.x & 31;
  const long long plane = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (plane >= planes) return;
  const A kv = ld<A>(k + plane);
  const T* gp = dy + plane * hw;
  const T* xp = x + plane * hw;
  A acc = (A)0;
  for (int i = lane; i < hw; i += 32) {
    const A g = ld<A>(gp + i);
    if (dx) st<T, A>(dx + plane * hw + i, g * kv);
    acc += g * ld<A>(xp + i);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0 && dk) st<T, A>(dk + plane, acc);
}

template <typename T>
int scale_forward(const T* x, const T* k, T* y, long long planes, int hw, cudaStream_t s) {
  const long long blocks = (planes + 7) / 8;
  if (blocks > 0x7fffffffLL) return DK_ERR_UNSUPPORTED;
  scale_fwd_kernel<T><<<(unsigned)blocks, 256, 0, s>>>(x, k, y, planes, hw);
  return check_launch();
}
template <typename T>
int scale_backward(const T* dy, const T* x, const T* k, T* dx, T* dk, long long planes, int hw, cudaStream_t s) {
  const long long blocks = (planes + 7) / 8;
  if (blocks > 0x7fffffffLL) return DK_ERR_UNSUPPORTED;
  scale_bwd_kernel<T><<<(unsigned)blocks, 256, 0, s>>>(dy, x, k, dx, dk, planes, hw);
  return check_launch();
}

// Offset clipping of the layers that produce the offsets (reference modules/deform_kernel.py:185-218, 273-276), one
// pass instead of five elementwise ones:  v = r * dilate + bias[channel];  y = (clamp(v, lo, hi) - bias) / dilate * post.
// The backward passes the gradient where lo <= v <= hi (both ends included, as torch.clamp does).  The four scalars come as
// doubles and are narrowed to the arithmetic type of the tensors in the kernel, so that fp64 tensors see fp64 bounds.
template <typename T>
__global__ void clip_fwd_kernel(const T* __restrict__ r, const float* __restrict__ bias, T* __restrict__ y, long long total,
                                int channels, int hw, double lo, double hi, double dilate, double post) {
  using A = typename Compute<T>::type;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const A b = bias ? (A)bias[(i / hw) % channels] : (A)0;
  const A v = ld<A>(r + i) * (A)dilate + b;
  const A c = v < (A)lo ? (A)lo : (v > (A)hi ? (A)hi : v);  // NaN stays NaN
  st<T, A>(y + i, (c - b) / (A)dilate * (A)post);
}
template <typename T>
__global__ void clip_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ r, const float* __restrict__ bias,
                                T* __restrict__ dr, long long total, int channels, int hw, double lo, double hi, double dilate,
                                double post) {
  using A = typename Compute<T>::type;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const A b = bias ? (A)bias[(i / hw) % channels] : (A)0;
  const A v = ld<A>(r + i) * (A)dilate + b;
  const bool pass = v >= (A)lo && v <= (A)hi;
  st<T, A>(dr + i, pass ? ld<A>(dy + i) * (A)post : (A)0);
}

template <typename T>
int clip_forward(const T* r, const float* bias, T* y, long long total, int channels, int hw, double lo, double hi, double dilate,
                 double post, cudaStream_t s) {
  const long long blocks = (total + 255) / 256;
  if (blocks > 0x7fffffffLL) return DK_ERR_UNSUPPORTED;
  clip_fwd_kernel<T><<<(unsigned)blocks, 256, 0, s>>>(r, bias, y, total, channels, hw, lo, hi, dilate, post);
  return check_launch();
}
template <typename T>
int clip_backward(const T* dy, const T* r, const float* bias, T* dr, long long total, int channels, int hw, double lo, double hi,
                  double dilate, double post, cudaStream_t s) {
  const long long blocks = (total + 255) / 256;
  if (blocks > 0x7fffffffLL) return DK_ERR_UNSUPPORTED;
  clip_bwd_kernel<T><<<(unsigned)blocks, 256, 0, s>>>(dy, r, bias, dr, total, channels, hw, lo, hi, dilate, post);
  return check_launch();
}

}  // namespace dk

using namespace dk;

extern "C" {

int dk_plane_scale_forward(const void* input, const void* scale, void* output, long long planes, int plane_size, int dtype,
                           void* stream) {
  if (!input || !scale || !output || planes <= 0 || plane_size <= 0) return DK_ERR_BAD_ARGUMENT;
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case DK_F32: return scale_forward<float>((const float*)input, (const float*)scale, (float*)output, planes, plane_size, s);
    case DK_F16: return scale_forward<__half>((const __half*)input, (const __half*)scale, (__half*)output, planes, plane_size, s);
    case DK_F64: return scale_forward<double>((const double*)input, (const double*)scale, (double*)output, planes, plane_size, s);
    default: return DK_ERR_BAD_ARGUMENT;
  }
}

int dk_plane_scale_backward(const void* grad_output, const void* input, const void* scale, void* grad_input,
                            void* grad_scale, long long planes, int plane_size, int dtype, void* stream) {
  if (!grad_output || !input || !scale || planes <= 0 || plane_size <= 0) return DK_ERR_BAD_ARGUMENT;
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case DK_F32:
      return scale_backward<float>((const float*)grad_output, (const float*)input, (const float*)scale, (float*)grad_input,
                                   (float*)grad_scale, planes, plane_size, s);
    case DK_F16:
      return scale_backward<__half>((const __half*)grad_output, (const __half*)input, (const __half*)scale,
                                    (__half*)grad_input, (__half*)grad_scale, planes, plane_size, s);
    case DK_F64:
      return scale_backward<double>((const double*)grad_output, (const double*)input, (const double*)scale,
                                    (double*)grad_input, (double*)grad_scale, planes, plane_size, s);
    default: return DK_ERR_BAD_ARGUMENT;
  }
}

int dk_offset_clip_forward(const void* offsets, const void* bias, void* output, int batch, int channels, int plane_size,
                           double lo, double hi, double dilate, double post_scale, int dtype, void* stream) {
  if (!offsets || !output || batch <= 0 || channels <= 0 || plane_size <= 0 || dilate == 0.0) return DK_ERR_BAD_ARGUMENT;
  cudaStream_t s = (cudaStream_t)stream;
  const long long total = (long long)batch * channels * plane_size;
  const float* b = (const float*)bias;
  switch (dtype) {
    case DK_F32: return clip_forward<float>((const float*)offsets, b, (float*)output, total, channels, plane_size, lo, hi, dilate, post_scale, s);
    case DK_F16: return clip_forward<__half>((const __half*)offsets, b, (__half*)output, total, channels, plane_size, lo, hi, dilate, post_scale, s);
    case DK_F64: return clip_forward<double>((const double*)offsets, b, (double*)output, total, channels, plane_size, lo, hi, dilate, post_scale, s);
    default: return DK_ERR_BAD_ARGUMENT;
  }
}

int dk_offset_clip_backward(const void* grad_output, const void* offsets, const void* bias, void* grad_offsets, int batch,
                            int channels, int plane_size, double lo, double hi, double dilate, double post_scale, int dtype,
                            void* stream) {
  if (!grad_output || !offsets || !grad_offsets || batch <= 0 || channels <= 0 || plane_size <= 0 || dilate == 0.0)
    return DK_ERR_BAD_ARGUMENT;
  cudaStream_t s = (cudaStream_t)stream;
  const long long total = (long long)batch * channels * plane_size;
  const float* b = (const float*)bias;
  switch (dtype) {
    case DK_F32: return clip_backward<float>((const float*)grad_output, (const float*)offsets, b, (float*)grad_offsets, total, channels, plane_size, lo, hi, dilate, post_scale, s);
    case DK_F16: return clip_backward<__half>((const __half*)grad_output, (const __half*)offsets, b, (__half*)grad_offsets, total, channels, plane_size, lo, hi, dilate, post_scale, s);
    case DK_F64: return clip_backward<double>((const double*)grad_output, (const double*)offsets, b, (double*)grad_offsets, total, channels, plane_size, lo, hi, dilate, post_scale, s);
    default: return DK_ERR_BAD_ARGUMENT;
  }
}

}  // extern "C"
