// Shared device/host helpers for the sm_100a deformable-kernel kernels.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdlib>

#include "dk_b200.h"

namespace dk {

// Geometry as the kernels see it (derived once on the host from dk_geom).
struct Geom {
  int N, C, H, W;
  int kH, kW, sH, sW, pH, pW, dH, dW;
  int Ho, Wo;
  int scH, scW, G;
  int taps;   // kH*kW
  int P;      // Ho*Wo
  int HW;     // H*W
  int cells;  // scH*scW
  int Cg;     // C / G channels per rotation group
};

// Storage type -> arithmetic type: fp16 and fp32 compute in fp32, fp64 in fp64.
template <typename T> struct Compute { using type = float; };
template <> struct Compute<double> { using type = double; };

template <typename A, typename T> __device__ __forceinline__ A ld(const T* p) { return static_cast<A>(__ldg(p)); }
template <> __device__ __forceinline__ float ld<float, __half>(const __half* p) { return __half2float(__ldg(p)); }

template <typename T, typename A> __device__ __forceinline__ void st(T* p, A v) { *p = static_cast<T>(v); }
template <> __device__ __forceinline__ void st<__half, float>(__half* p, float v) { *p = __float2half_rn(v); }

__device__ __forceinline__ float dk_floor(float v) { return floorf(v); }
__device__ __forceinline__ double dk_floor(double v) { return floor(v); }

// Zero-extended bilinear sampling of a rows x cols grid at (u, v): the four corner
// indices (clamped into the grid so that they are always loadable) and, per corner,
// a flag telling whether the corner lies inside the grid.  `outer` is the
// caller's validity test of the sample as a whole (-1 < u < rows, -1 < v < cols).
// Value coefficients are {hh*hw, hh*lw, lh*hw, lh*lw} * mask; the derivative wrt u is
// {-hw, -lw, +hw, +lw} * mask and wrt v {-hh, +hh, -lh, +lh} * mask: floor-based, so
// at an integer coordinate it is the right-hand derivative, and at the upper edge the
// derivative into the zero extension.
template <typename A>
struct Bilinear {
  int idx[4];
  bool m[4];
  A lh, lw, hh, hw;
};

template <typename A>
__device__ __forceinline__ void bilinear_setup(A u, A v, int rows, int cols, bool outer, Bilinear<A>& b) {
  const A fu = dk_floor(u), fv = dk_floor(v);
  // clamp before the float->int conversion so that wild offsets cannot overflow it
  const A cu = fmin(fmax(fu, (A)-2), (A)(rows + 1));
  const A cv = fmin(fmax(fv, (A)-2), (A)(cols + 1));
  const int h0 = (int)cu, w0 = (int)cv;
  const int h1 = h0 + 1, w1 = w0 + 1;
  b.lh = u - fu;
  b.lw = v - fv;
  b.hh = (A)1 - b.lh;
  b.hw = (A)1 - b.lw;
  const bool a0 = outer && h0 >= 0 && h0 <= rows - 1;
  const bool a1 = outer && h1 >= 0 && h1 <= rows - 1;
  const bool c0 = w0 >= 0 && w0 <= cols - 1;
  const bool c1 = w1 >= 0 && w1 <= cols - 1;
  b.m[0] = a0 && c0;
  b.m[1] = a0 && c1;
  b.m[2] = a1 && c0;
  b.m[3] = a1 && c1;
  const int h0c = min(max(h0, 0), rows - 1), h1c = min(max(h1, 0), rows - 1);
  const int w0c = min(max(w0, 0), cols - 1), w1c = min(max(w1, 0), cols - 1);
  b.idx[0] = h0c * cols + w0c;
  b.idx[1] = h0c * cols + w1c;
  b.idx[2] = h1c * cols + w0c;
  b.idx[3] = h1c * cols + w1c;
}

template <typename A>
__device__ __forceinline__ void bilinear_value_coefs(const Bilinear<A>& b, A (&c)[4]) {
  // selects, not products with the mask: a NaN or infinite offset must sample nothing
  c[0] = b.m[0] ? b.hh * b.hw : (A)0;
  c[1] = b.m[1] ? b.hh * b.lw : (A)0;
  c[2] = b.m[2] ? b.lh * b.hw : (A)0;
  c[3] = b.m[3] ? b.lh * b.lw : (A)0;
}
template <typename A>
__device__ __forceinline__ void bilinear_du_coefs(const Bilinear<A>& b, A (&c)[4]) {
  c[0] = b.m[0] ? -b.hw : (A)0;
  c[1] = b.m[1] ? -b.lw : (A)0;
  c[2] = b.m[2] ? b.hw : (A)0;
  c[3] = b.m[3] ? b.lw : (A)0;
}
template <typename A>
__device__ __forceinline__ void bilinear_dv_coefs(const Bilinear<A>& b, A (&c)[4]) {
  c[0] = b.m[0] ? -b.hh : (A)0;
  c[1] = b.m[1] ? b.hh : (A)0;
  c[2] = b.m[2] ? -b.lh : (A)0;
  c[3] = b.m[3] ? b.lh : (A)0;
}

// Bank coordinate of one tap: u = f + r + (scope - kernel)/2.  (The reference adds
// the last term in double and narrows, csrc/filter_sample_depthwise_cuda_kernel.cu:338-341;
// for the multiples of 0.5 that occur this equals the single correctly rounded add done here.)
template <typename A>
__device__ __forceinline__ bool bank_setup(A r_h, A r_w, int fh, int fw, const Geom& g, Bilinear<A>& b) {
  const A u = ((A)fh + r_h) + (A)(g.scH - g.kH) * (A)0.5;
  const A v = ((A)fw + r_w) + (A)(g.scW - g.kW) * (A)0.5;
  const bool valid = (u > (A)-1) && (v > (A)-1) && (u < (A)g.scH) && (v < (A)g.scW);
  bilinear_setup(u, v, g.scH, g.scW, valid, b);
  return valid;
}

// Image sample position test of DK+DCN (csrc/filter_sample_depthwise_cuda_kernel.cu:500).
template <typename A>
__device__ __forceinline__ bool image_setup(A ph, A pw, const Geom& g, Bilinear<A>& b) {
  const bool used = (ph > (A)-1) && (pw > (A)-1) && (ph < (A)g.H) && (pw < (A)g.W);
  bilinear_setup(ph, pw, g.H, g.W, used, b);
  return used;
}

template <typename A> __device__ __forceinline__ A dot4(const A (&c)[4], const A (&v)[4]) {
  return c[0] * v[0] + c[1] * v[1] + c[2] * v[2] + c[3] * v[3];
}

// ---------------------------------------------------------------- host side

// Experiment knobs read from the environment exist only in builds made with -DDK_TUNING; the product build ignores them
// (the one switch it keeps is DK_B200_DISABLE_MMA, which forces the general kernels for A/B runs).
inline const char* tuning_env(const char* name) {
#ifdef DK_TUNING
  return std::getenv(name);
#else
  (void)name;
  return nullptr;
#endif
}

struct LaunchError {
  int status;
  cudaError_t cuda;
};

bool make_geom(const dk_geom* in, Geom* out);
void set_last_cuda_error(cudaError_t e);
int check_launch();
int device_smem_optin();  // max dynamic shared memory per block (opt-in), cached per device
int device_sm_count();

template <typename K>
inline int enable_smem(K kernel, size_t bytes) {
  if (bytes > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) {
      set_last_cuda_error(e);
      return DK_ERR_CUDA;
    }
  }
  return DK_OK;
}

// typed launchers implemented in dk_local.cu / dk_deform.cu / dk_nd.cu
template <typename T> int local_forward(const T*, const T*, const T*, T*, const Geom&, cudaStream_t);
template <typename T> int local_backward_data(const T*, const T*, const T*, T*, const Geom&, cudaStream_t);
template <typename T>
int local_backward_rotation(const T*, const T*, const T*, const T*, T*, const Geom&, void* ws, size_t ws_bytes, cudaStream_t);
template <typename T>
int local_backward_filter(const T* dy, const T* x, const T* rot, T* dw, const Geom&, void* ws, size_t ws_bytes, cudaStream_t);

template <typename T>
int local_backward_filter_fit(const T* dy, const T* x, const T* rot, T* dw, const Geom&, void* ws, size_t ws_bytes, cudaStream_t,
                              bool launch, size_t* need_out);  // fixed-size workspace: the plan shrinks to fit

template <typename T> int deform_forward(const T*, const T*, const T*, const T*, T*, const Geom&, cudaStream_t);
template <typename T>
int deform_backward_data(const T* dy, const T* off, const T* rot, const T* w, T* dx, const Geom&, void* ws, size_t ws_bytes,
                         cudaStream_t);
template <typename T>
int deform_backward_coords(const T* dy, const T* x, const T* off, const T* rot, const T* w, T* doff, T* drot, const Geom&,
                           cudaStream_t);
template <typename T>
int deform_backward_filter(const T* dy, const T* x, const T* off, const T* rot, T* dw, const Geom&, void* ws,
                           size_t ws_bytes, cudaStream_t);

// fp16 tensor-core fast path (dk_local_mma.cu); DK_ERR_UNSUPPORTED = shape outside the fast path
bool mma_path_enabled();
int local_conv_mma(const __half* src, const __half* rot, const __half* w, __half* dst, const Geom& g, bool transposed,
                   cudaStream_t s);
// row-ring kernels (dk_local_ring.cu): TMA-fed producer / consumer blocks; DK_ERR_UNSUPPORTED = shape outside them
int local_conv_ring(const __half* src, const __half* rot, const __half* w, __half* dst, const Geom& g, bool transposed,
                    cudaStream_t s);
size_t local_gw_ring_workspace(const Geom& g);
int local_gw_ring(const __half* dy, const __half* x, const __half* rot, const __half* w, __half* drot, __half* dw, const Geom& g,
                  void* ws, size_t ws_bytes, cudaStream_t s);  // grad-offsets and grad-bank in one pass
// the same pass in band form for the planes the row-ring kernels do not take (dk_local_mma.cu; 4 x 4 scope)
size_t local_gw_mma_workspace(const Geom& g);
int local_gw_mma(const __half* dy, const __half* x, const __half* rot, const __half* w, __half* drot, __half* dw, const Geom& g,
                 void* ws, size_t ws_bytes, cudaStream_t s);
size_t local_bwd_ring_workspace(const Geom& g);
bool local_bwd_ring_preferred(const Geom& g);  // the one-pass backward is expected to beat grad-input + the fused offsets / bank pass
int local_bwd_ring(const __half* dy, const __half* x, const __half* rot, const __half* w, __half* dx, __half* drot, __half* dw,
                   const Geom& g, void* ws, size_t ws_bytes, cudaStream_t s);  // all three gradients in one pass
int ring_error_status();
size_t local_rot_mma_workspace(const Geom& g);
int local_rot_mma(const __half* dy, const __half* x, const __half* rot, const __half* w, __half* drot, const Geom& g,
                  void* ws, size_t ws_bytes, cudaStream_t s);
size_t local_filter_mma_workspace(const Geom& g);
int local_mma_plan_query(const Geom& g, int pass, long long out[8]);
int local_ring_plan_query(const Geom& g, int pass, long long out[8]);
int local_filter_mma(const __half* dy, const __half* x, const __half* rot, __half* dw, const Geom& g, void* ws,
                     size_t ws_bytes, cudaStream_t s);

// Plan of the two-stage bank-gradient reduction, shared by the workspace query and the launch.
struct FilterPlan {
  int warps;         // warps per block, each owning 32 channels
  int chan_blocks;   // blocks along the channels of one rotation group
  int pix_blocks;    // blocks along the flattened (n, oh, ow) axis = number of partial sums
  long long pix_per_block;
  size_t ws_bytes;   // pix_blocks * C * cells * sizeof(acc)
};
FilterPlan filter_plan(const Geom& g, size_t acc_bytes);
FilterPlan filter_plan_fit(const Geom& g, size_t acc_bytes, size_t max_bytes);
size_t deform_filter_mma_workspace(const Geom& g);
size_t deform_coords_mma_workspace(const Geom& g);
// with dw / bank_ws / bank_done the bank gradient is computed in the same pass where the plan allows (*bank_done)
size_t deform_coords_bank_workspace(const Geom& g);
int deform_coords_mma(const __half* dy, const __half* x, const __half* off, const __half* rot, const __half* w, __half* doff,
                      __half* drot, const Geom& g, void* ws, size_t ws_bytes, cudaStream_t s, __half* dw = nullptr,
                      void* bank_ws = nullptr, size_t bank_ws_bytes = 0, bool* bank_done = nullptr);
int deform_data_mma(const __half* dy, const __half* off, const __half* rot, const __half* w, __half* dx, const Geom& g,
                    void* ws, size_t ws_bytes, cudaStream_t s);
int deform_forward_mma(const __half* x, const __half* off, const __half* rot, const __half* w, __half* y, const Geom& g,
                       cudaStream_t s);  // fp16 tensor-core DK+DCN bank gradient (dk_deform_mma.cu)
int deform_filter_mma(const __half* dy, const __half* x, const __half* off, const __half* rot, __half* dw, const Geom& g,
                      void* ws, size_t ws_bytes, cudaStream_t s);
size_t deform_filter_plane_workspace(const Geom& g, int dtype);  // 0 when the shared-memory-plane variant does not apply

constexpr int kMaxNdDims = 8;
struct NdShape {
  int s[kMaxNdDims];
};
template <typename T>
int global_dk_forward(const T* x, const float* bank, const float* fc_w, const float* fc_b, const float* tap_bias, T* y,
                      float* gap, float* raw, float* coord, float* scale, int N, int C, int hw, int D, int prod,
                      const NdShape& sh, cudaStream_t s);
template <typename T>
int global_dk_backward(const T* dy, const T* x, const float* bank, const float* fc_w, const float* gap, const float* raw,
                       const float* coord, const float* scale, T* dx, float* dbank, float* dfc_w, float* dfc_b, float* ws,
                       int N, int C, int hw, int D, int prod, const NdShape& sh, cudaStream_t s);
template <typename T> int nd_forward(const T*, const T*, T*, int B, int C, int D, int prod, const NdShape&, cudaStream_t);
template <typename T> int nd_backward_data(const T*, const T*, T*, int B, int C, int D, int prod, const NdShape&, cudaStream_t);
template <typename T>
int nd_backward_coord(const T*, const T*, const T*, T*, int B, int C, int D, int prod, const NdShape&, bool sum_channels,
                      cudaStream_t);

}  // namespace dk
