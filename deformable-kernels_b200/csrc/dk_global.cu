// The global deformable kernel with a 1x1 depthwise kernel as two calls (forward, backward) instead of the ~35
// launches of its PyTorch composition (reference: modules/deform_kernel.py:76-118):
//
//   gap[n, c]   = mean over the plane of x[n, c]                                  (global average pool)
//   raw[n, d]   = fc_weight[d, :] . gap[n, :] + fc_bias[d] + tap_bias[d]           (coordinate head, D = bank dims)
//   coord[n, d] = clamp(raw[n, d], 0, shape[0] - 1)                               (the reference clamps every dim by shape[0])
//   scale[n, c] = N-d linear sample of bank[c] at coord[n]                         (dk_nd.cu semantics)
//   y[n, c]     = x[n, c] * scale[n, c]
//
// and its gradient wrt x, the bank and the head's weight and bias.  The head runs in fp32 whatever the dtype of x.
#include "dk_nd_common.cuh"

namespace dk {

namespace {

template <typename T>
__global__ void gdk_pool_kernel(const T* __restrict__ x, float* __restrict__ gap, long long planes, int hw, float inv_hw) {
  const int lane = threadIdx.x & 31;
  const long long plane = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (plane >= planes) return;
  const T* xp = x + plane * hw;
  float acc = 0.f;
  for (int i = lane; i < hw; i += 32) acc += ld<float>(xp + i);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) gap[plane] = acc * inv_hw;
}

// one block per sample: coordinates, then the sampled scale of every channel
__global__ void __launch_bounds__(256) gdk_head_fwd_kernel(const float* __restrict__ gap, const float* __restrict__ fc_w,
                                                           const float* __restrict__ fc_b, const float* __restrict__ tap_bias,
                                                           const float* __restrict__ bank, float* __restrict__ raw,
                                                           float* __restrict__ coord, float* __restrict__ scale, int C, int D,
                                                           int prod, const NdShape sh, float cmax) {
  __shared__ float red[8][kMaxNdDims];
  __shared__ float cs[kMaxNdDims];
  const int n = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float* g = gap + (size_t)n * C;
  float part[kMaxNdDims];
#pragma unroll
  for (int d = 0; d < kMaxNdDims; ++d) part[d] = 0.f;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const float gv = g[c];
#pragma unroll
    for (int d = 0; d < kMaxNdDims; ++d)
      if (d < D) part[d] += fc_w[(size_t)d * C + c] * gv;
  }
#pragma unroll
  for (int d = 0; d < kMaxNdDims; ++d) {
    if (d < D) {
      float v = part[d];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0) red[warp][d] = v;
    }
  }
  __syncthreads();
  if (threadIdx.x < D) {
    const int d = threadIdx.x;
    float v = 0.f;
    for (int k = 0; k < (int)(blockDim.x >> 5); ++k) v += red[k][d];
    v = v + fc_b[d] + tap_bias[d];
    const float cl = fminf(fmaxf(v, 0.f), cmax);
    raw[(size_t)n * D + d] = v;
    coord[(size_t)n * D + d] = cl;
    cs[d] = cl;
  }
  __syncthreads();
  NdPoint<float> pt;
  nd_point<float, float, false>(cs, D, sh, pt);
  for (int c = threadIdx.x; c < C; c += blockDim.x)
    scale[(size_t)n * C + c] = pt.valid ? nd_gather<float, float>(bank + (size_t)c * prod, D, sh, pt, -1) : 0.f;
}

template <typename T>
__global__ void gdk_apply_kernel(const T* __restrict__ x, const float* __restrict__ scale, T* __restrict__ y, long long planes,
                                 int hw) {
  const int lane = threadIdx.x & 31;
  const long long plane = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (plane >= planes) return;
  const float kv = scale[plane];
  const T* xp = x + plane * hw;
  T* yp = y + plane * hw;
  for (int i = lane; i < hw; i += 32) st<T, float>(yp + i, ld<float>(xp + i) * kv);
}

template <typename T>
__global__ void gdk_dscale_kernel(const T* __restrict__ dy, const T* __restrict__ x, float* __restrict__ dscale,
                                  long long planes, int hw) {
  const int lane = threadIdx.x & 31;
  const long long plane = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (plane >= planes) return;
  const T* gp = dy + plane * hw;
  const T* xp = x + plane * hw;
  float acc = 0.f;
  for (int i = lane; i < hw; i += 32) acc += ld<float>(gp + i) * ld<float>(xp + i);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) dscale[plane] = acc;
}

// one block per sample: gradient of the (clamped) coordinates, then of the pooled features
__global__ void __launch_bounds__(256) gdk_head_bwd_sample_kernel(const float* __restrict__ dscale, const float* __restrict__ bank,
                                                                  const float* __restrict__ raw, const float* __restrict__ coord,
                                                                  const float* __restrict__ fc_w, float* __restrict__ dcoord,
                                                                  float* __restrict__ dgap, int C, int D, int prod,
                                                                  const NdShape sh, float cmax) {
  __shared__ float red[8][kMaxNdDims];
  __shared__ float dc[kMaxNdDims];
  const int n = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  NdPoint<float> pt;
  nd_point<float, float>(coord + (size_t)n * D, D, sh, pt);
  float part[kMaxNdDims];
#pragma unroll
  for (int d = 0; d < kMaxNdDims; ++d) part[d] = 0.f;
  if (pt.valid) {
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
      const float ds = dscale[(size_t)n * C + c];
#pragma unroll
      for (int d = 0; d < kMaxNdDims; ++d)
        if (d < D) part[d] += ds * nd_gather<float, float>(bank + (size_t)c * prod, D, sh, pt, d);
    }
  }
#pragma unroll
  for (int d = 0; d < kMaxNdDims; ++d) {
    if (d < D) {
      float v = part[d];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0) red[warp][d] = v;
    }
  }
  __syncthreads();
  if (threadIdx.x < D) {
    const int d = threadIdx.x;
    float v = 0.f;
    for (int k = 0; k < (int)(blockDim.x >> 5); ++k) v += red[k][d];
    const float r = raw[(size_t)n * D + d];
    if (!(r >= 0.f && r <= cmax)) v = 0.f;  // the clamp passes the gradient inside [0, cmax] only
    dcoord[(size_t)n * D + d] = v;
    dc[d] = v;
  }
  __syncthreads();
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float v = 0.f;
#pragma unroll
    for (int d = 0; d < kMaxNdDims; ++d)
      if (d < D) v += dc[d] * fc_w[(size_t)d * C + c];
    dgap[(size_t)n * C + c] = v;
  }
}

// sums over the batch in a fixed order: bank gradient (thread = channel x cell), head weight (thread = dim x channel),
// head bias (thread = dim)
__global__ void gdk_head_bwd_param_kernel(const float* __restrict__ dscale, const float* __restrict__ coord,
                                          const float* __restrict__ dcoord, const float* __restrict__ gap,
                                          float* __restrict__ dbank, float* __restrict__ dfc_w, float* __restrict__ dfc_b, int N,
                                          int C, int D, int prod, const NdShape sh) {
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long n_bank = (long long)C * prod, n_w = (long long)D * C;
  if (tid < n_bank) {
    if (!dbank) return;
    const int cell = (int)(tid % prod), c = (int)(tid / prod);
    int pos[kMaxNdDims];
    {
      int rem = cell;
#pragma unroll
      for (int d = kMaxNdDims - 1; d >= 0; --d) {
        if (d < D) {
          pos[d] = rem % sh.s[d];
          rem /= sh.s[d];
        }
      }
    }
    float acc = 0.f;
    for (int n = 0; n < N; ++n) {
      NdPoint<float> pt;
      nd_point<float, float>(coord + (size_t)n * D, D, sh, pt);
      if (!pt.valid) continue;
      float wgt = 1.f;
#pragma unroll
      for (int d = 0; d < kMaxNdDims; ++d) {
        if (d < D) {
          const int rel = pos[d] - pt.low[d];
          wgt *= (rel == 0) ? 1.f - pt.frac[d] : (rel == 1 ? pt.frac[d] : 0.f);
        }
      }
      if (wgt != 0.f) acc += wgt * dscale[(size_t)n * C + c];
    }
    dbank[tid] = acc;
  } else if (tid < n_bank + n_w) {
    if (!dfc_w) return;
    const long long i = tid - n_bank;
    const int c = (int)(i % C), d = (int)(i / C);
    float acc = 0.f;
    for (int n = 0; n < N; ++n) acc += dcoord[(size_t)n * D + d] * gap[(size_t)n * C + c];
    dfc_w[i] = acc;
  } else if (tid < n_bank + n_w + D) {
    if (!dfc_b) return;
    const int d = (int)(tid - n_bank - n_w);
    float acc = 0.f;
    for (int n = 0; n < N; ++n) acc += dcoord[(size_t)n * D + d];
    dfc_b[d] = acc;
  }
}

template <typename T>
__global__ void gdk_dx_kernel(const T* __restrict__ dy, const float* __restrict__ scale, const float* __restrict__ dgap,
                              T* __restrict__ dx, long long planes, int hw, float inv_hw) {
  const int lane = threadIdx.x & 31;
  const long long plane = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (plane >= planes) return;
  const float kv = scale[plane], add = dgap[plane] * inv_hw;
  const T* gp = dy + plane * hw;
  T* op = dx + plane * hw;
  for (int i = lane; i < hw; i += 32) st<T, float>(op + i, ld<float>(gp + i) * kv + add);
}

}  // namespace

template <typename T>
int global_dk_forward(const T* x, const float* bank, const float* fc_w, const float* fc_b, const float* tap_bias, T* y,
                      float* gap, float* raw, float* coord, float* scale, int N, int C, int hw, int D, int prod,
                      const NdShape& sh, cudaStream_t s) {
  const long long planes = (long long)N * C;
  const long long blocks = (planes + 7) / 8;
  if (blocks > 0x7fffffffLL) return DK_ERR_UNSUPPORTED;
  gdk_pool_kernel<T><<<(unsigned)blocks, 256, 0, s>>>(x, gap, planes, hw, 1.f / (float)hw);
  gdk_head_fwd_kernel<<<N, 256, 0, s>>>(gap, fc_w, fc_b, tap_bias, bank, raw, coord, scale, C, D, prod, sh,
                                        (float)(sh.s[0] - 1));
  gdk_apply_kernel<T><<<(unsigned)blocks, 256, 0, s>>>(x, scale, y, planes, hw);
  return check_launch();
}

template <typename T>
int global_dk_backward(const T* dy, const T* x, const float* bank, const float* fc_w, const float* gap, const float* raw,
                       const float* coord, const float* scale, T* dx, float* dbank, float* dfc_w, float* dfc_b, float* ws,
                       int N, int C, int hw, int D, int prod, const NdShape& sh, cudaStream_t s) {
  const long long planes = (long long)N * C;
  const long long blocks = (planes + 7) / 8;
  if (blocks > 0x7fffffffLL) return DK_ERR_UNSUPPORTED;
  float* dscale = ws;
  float* dgap = dscale + planes;
  float* dcoord = dgap + planes;
  gdk_dscale_kernel<T><<<(unsigned)blocks, 256, 0, s>>>(dy, x, dscale, planes, hw);
  gdk_head_bwd_sample_kernel<<<N, 256, 0, s>>>(dscale, bank, raw, coord, fc_w, dcoord, dgap, C, D, prod, sh,
                                               (float)(sh.s[0] - 1));
  if (dbank || dfc_w || dfc_b) {
    const long long work = (long long)C * prod + (long long)D * C + D;
    gdk_head_bwd_param_kernel<<<(unsigned)((work + 127) / 128), 128, 0, s>>>(dscale, coord, dcoord, gap, dbank, dfc_w, dfc_b, N,
                                                                            C, D, prod, sh);
  }
  if (dx) gdk_dx_kernel<T><<<(unsigned)blocks, 256, 0, s>>>(dy, scale, dgap, dx, planes, hw, 1.f / (float)hw);
  return check_launch();
}

#define DK_INSTANTIATE_GLOBAL(T)                                                                                          \
  template int global_dk_forward<T>(const T*, const float*, const float*, const float*, const float*, T*, float*, float*,  \
                                    float*, float*, int, int, int, int, int, const NdShape&, cudaStream_t);                \
  template int global_dk_backward<T>(const T*, const T*, const float*, const float*, const float*, const float*,           \
                                     const float*, const float*, T*, float*, float*, float*, float*, int, int, int, int,  \
                                     int, const NdShape&, cudaStream_t);
DK_INSTANTIATE_GLOBAL(float)
DK_INSTANTIATE_GLOBAL(__half)
DK_INSTANTIATE_GLOBAL(double)

}  // namespace dk
