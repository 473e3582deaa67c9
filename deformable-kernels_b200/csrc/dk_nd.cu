// N-d multilinear sampling of a per-channel array at per-sample coordinates (the global
// deformable kernel's resampler): forward, gradient wrt the array (gather form, no
// atomics) and gradient wrt the coordinates (per channel, or summed over channels).
//
// Semantics (reference: csrc/nd_linear_sample_cuda_kernel.cu:45-177): a sample with any
// coordinate <= -1 or >= size is zero with zero gradients; otherwise each of the 2^D
// corners takes, per dimension, the low cell (needs floor(x) >= 0, weight 1-frac) or the
// high cell (needs floor(x)+1 <= size-1, weight frac); a corner with a missing cell is
// dropped.  The coordinate derivative replaces the factor of the differentiated
// dimension by -1 (low) or +1 (high).  Dimension 0 varies slowest.
#include "dk_nd_common.cuh"

namespace dk {

template <typename T>
__global__ void nd_fwd_kernel(const T* __restrict__ data, const T* __restrict__ coord, T* __restrict__ out, int B, int C,
                              int D, int prod, const NdShape sh) {
  using A = typename Compute<T>::type;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (tid >= (long long)B * C) return;
  const int c = (int)(tid % C), b = (int)(tid / C);
  NdPoint<A> pt;
  nd_point<T, A>(coord + (size_t)b * D, D, sh, pt);
  const A v = pt.valid ? nd_gather<T, A>(data + (size_t)c * prod, D, sh, pt, -1) : (A)0;
  st<T, A>(out + tid, v);
}

// grad wrt the array, gather form: one thread per (channel, cell) walks the batch and adds
// grad_out[b, c] * (product over dimensions of the hat weight of this cell).
template <typename T>
__global__ void nd_bwd_data_kernel(const T* __restrict__ dy, const T* __restrict__ coord, T* __restrict__ ddata, int B,
                                   int C, int D, int prod, const NdShape sh) {
  using A = typename Compute<T>::type;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (tid >= (long long)C * prod) return;
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
  A acc = (A)0;
  for (int b = 0; b < B; ++b) {
    NdPoint<A> pt;
    nd_point<T, A>(coord + (size_t)b * D, D, sh, pt);
    if (!pt.valid) continue;
    A wgt = (A)1;
#pragma unroll
    for (int d = 0; d < kMaxNdDims; ++d) {
      if (d < D) {
        const int rel = pos[d] - pt.low[d];
        wgt *= (rel == 0) ? (A)1 - pt.frac[d] : (rel == 1 ? pt.frac[d] : (A)0);
      }
    }
    if (wgt != (A)0) acc += wgt * ld<A>(dy + (size_t)b * C + c);
  }
  st<T, A>(ddata + tid, acc);
}

// per-channel coordinate gradient, layout [B, D, C] (what the reference's kernel writes)
template <typename T>
__global__ void nd_bwd_coord_kernel(const T* __restrict__ dy, const T* __restrict__ data, const T* __restrict__ coord,
                                    T* __restrict__ dcoord_c, int B, int C, int D, int prod, const NdShape sh) {
  using A = typename Compute<T>::type;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (tid >= (long long)B * D * C) return;
  const int c = (int)(tid % C);
  const int gd = (int)((tid / C) % D);
  const int b = (int)(tid / C / D);
  NdPoint<A> pt;
  nd_point<T, A>(coord + (size_t)b * D, D, sh, pt);
  A v = (A)0;
  if (pt.valid) v = ld<A>(dy + (size_t)b * C + c) * nd_gather<T, A>(data + (size_t)c * prod, D, sh, pt, gd);
  st<T, A>(dcoord_c + tid, v);
}

// coordinate gradient summed over channels inside the kernel: one block per sample
template <typename T, int BLOCK>
__global__ void __launch_bounds__(BLOCK) nd_bwd_coord_sum_kernel(const T* __restrict__ dy, const T* __restrict__ data,
                                                                 const T* __restrict__ coord, T* __restrict__ dcoord,
                                                                 int B, int C, int D, int prod, const NdShape sh) {
  using A = typename Compute<T>::type;
  __shared__ A red[BLOCK / 32][kMaxNdDims];
  const int b = blockIdx.x;
  NdPoint<A> pt;
  nd_point<T, A>(coord + (size_t)b * D, D, sh, pt);
  A g[kMaxNdDims];
#pragma unroll
  for (int d = 0; d < kMaxNdDims; ++d) g[d] = (A)0;
  if (pt.valid) {
    for (int c = threadIdx.x; c < C; c += BLOCK) {
      const A top = ld<A>(dy + (size_t)b * C + c);
#pragma unroll
      for (int d = 0; d < kMaxNdDims; ++d)
        if (d < D) g[d] += top * nd_gather<T, A>(data + (size_t)c * prod, D, sh, pt, d);
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int d = 0; d < kMaxNdDims; ++d) {
    A v = g[d];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0) red[warp][d] = v;
  }
  __syncthreads();
  if (threadIdx.x < D) {
    A s = (A)0;
    for (int q = 0; q < BLOCK / 32; ++q) s += red[q][threadIdx.x];
    st<T, A>(dcoord + (size_t)b * D + threadIdx.x, s);
  }
}

static inline bool grid_1d(long long n, int block, unsigned* out) {
  const long long b = (n + block - 1) / block;
  if (b > 0x7fffffffLL) return false;
  *out = (unsigned)(b > 0 ? b : 1);
  return true;
}

template <typename T>
int nd_forward(const T* data, const T* coord, T* out, int B, int C, int D, int prod, const NdShape& sh, cudaStream_t s) {
  unsigned grid;
  if (!grid_1d((long long)B * C, 256, &grid)) return DK_ERR_UNSUPPORTED;
  nd_fwd_kernel<T><<<grid, 256, 0, s>>>(data, coord, out, B, C, D, prod, sh);
  return check_launch();
}

template <typename T>
int nd_backward_data(const T* dy, const T* coord, T* ddata, int B, int C, int D, int prod, const NdShape& sh,
                     cudaStream_t s) {
  unsigned grid;
  if (!grid_1d((long long)C * prod, 128, &grid)) return DK_ERR_UNSUPPORTED;
  nd_bwd_data_kernel<T><<<grid, 128, 0, s>>>(dy, coord, ddata, B, C, D, prod, sh);
  return check_launch();
}

template <typename T>
int nd_backward_coord(const T* dy, const T* data, const T* coord, T* out, int B, int C, int D, int prod, const NdShape& sh,
                      bool sum_channels, cudaStream_t s) {
  if (sum_channels) {
    nd_bwd_coord_sum_kernel<T, 256><<<B, 256, 0, s>>>(dy, data, coord, out, B, C, D, prod, sh);
  } else {
    unsigned grid;
    if (!grid_1d((long long)B * D * C, 256, &grid)) return DK_ERR_UNSUPPORTED;
    nd_bwd_coord_kernel<T><<<grid, 256, 0, s>>>(dy, data, coord, out, B, C, D, prod, sh);
  }
  return check_launch();
}

#define DK_INSTANTIATE_ND(T)                                                                                     \
  template int nd_forward<T>(const T*, const T*, T*, int, int, int, int, const NdShape&, cudaStream_t);          \
  template int nd_backward_data<T>(const T*, const T*, T*, int, int, int, int, const NdShape&, cudaStream_t);    \
  template int nd_backward_coord<T>(const T*, const T*, const T*, T*, int, int, int, int, const NdShape&, bool, \
                                    cudaStream_t);
DK_INSTANTIATE_ND(float)
DK_INSTANTIATE_ND(__half)
DK_INSTANTIATE_ND(double)

}  // namespace dk
