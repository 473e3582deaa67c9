// Device helpers of the N-d multilinear sampler, shared by the operator kernels (dk_nd.cu) and the fused
// global deformable kernel (dk_global.cu).  Semantics: see dk_nd.cu.
#pragma once
#include "dk_common.cuh"

namespace dk {

template <typename A>
struct NdPoint {
  int low[kMaxNdDims];
  A frac[kMaxNdDims];
  bool valid;
};

// LDG = false reads the coordinates with plain loads (for coordinates in shared memory or written by this kernel)
template <typename T, typename A, bool LDG = true>
__device__ __forceinline__ void nd_point(const T* __restrict__ coord, int D, const NdShape& sh, NdPoint<A>& pt) {
  pt.valid = true;
#pragma unroll
  for (int d = 0; d < kMaxNdDims; ++d) {
    if (d < D) {
      const A xv = LDG ? ld<A>(coord + d) : static_cast<A>(coord[d]);
      if (xv <= (A)-1 || xv >= (A)sh.s[d]) pt.valid = false;
      if (!(xv == xv)) pt.valid = false;  // NaN samples nothing
      const A fl = dk_floor(xv);
      pt.low[d] = (int)fmin(fmax(fl, (A)-2), (A)(sh.s[d] + 1));
      pt.frac[d] = xv - fl;
    }
  }
}

// Weighted sum over the corners of one channel; GDIM >= 0 differentiates wrt that dimension.
template <typename T, typename A>
__device__ __forceinline__ A nd_gather(const T* __restrict__ data, int D, const NdShape& sh, const NdPoint<A>& pt,
                                       int gdim) {
  A val = (A)0;
  const unsigned corners = 1u << D;
  for (unsigned i = 0; i < corners; ++i) {
    int offset = 0;
    A wgt = (A)1;
    bool ok = true;
#pragma unroll
    for (int d = 0; d < kMaxNdDims; ++d) {
      if (d < D) {
        const int hi = (i >> d) & 1;
        const int pos = pt.low[d] + hi;
        ok = ok && pos >= 0 && pos <= sh.s[d] - 1;
        offset = offset * sh.s[d] + pos;
        const A f = hi ? pt.frac[d] : (A)1 - pt.frac[d];
        const A dsign = hi ? (A)1 : (A)-1;
        wgt *= (d == gdim) ? dsign : f;
      }
    }
    if (ok) val += wgt * ld<A>(data + offset);
  }
  return val;
}

}  // namespace dk
