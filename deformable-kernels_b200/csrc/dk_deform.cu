// Deformable kernel fused with deformable convolution (DK + DCN): the input is read by
// bilinear sampling at learned image-space offsets and multiplied by a kernel that is
// itself bilinear-sampled from the weight bank, all in one pass.  Forward, grad-input
// (scatter), and the two coordinate gradients (image-space offsets and kernel-space
// offsets) in one fused kernel.  The bank gradient lives in dk_local.cu (shared kernel).
#include "dk_common.cuh"

namespace dk {

// ------------------------------------------------------------------ forward
// One thread = one (n, output pixel); CC channels of one rotation group per block; taps
// outer, channels inner.  Both sampling bases (image corners, bank corners) are
// channel-independent and computed once per tap.
template <typename T, int CC, int BLOCK>
__global__ void __launch_bounds__(BLOCK) deform_fwd_kernel(const T* __restrict__ x, const T* __restrict__ off,
                                                           const T* __restrict__ rot, const T* __restrict__ w,
                                                           T* __restrict__ y, const Geom g) {
  using A = typename Compute<T>::type;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  A* bank = reinterpret_cast<A*>(smem_raw);  // [CC][cells]
  const int grp = blockIdx.z;
  const int j0 = blockIdx.y * CC;
  const int cnt = min(CC, g.Cg - j0);
  for (int i = threadIdx.x; i < CC * g.cells; i += BLOCK) {
    const int j = i / g.cells, cell = i - j * g.cells;
    bank[i] = (j < cnt) ? ld<A>(w + (size_t)(grp + g.G * (j0 + j)) * g.cells + cell) : (A)0;
  }
  __syncthreads();
  const long long total = (long long)g.N * g.P;
  const long long flat = (long long)blockIdx.x * BLOCK + threadIdx.x;
  if (flat >= total) return;
  const int n = (int)(flat / g.P);
  const int p = (int)(flat - (long long)n * g.P);
  const int oh = p / g.Wo, ow = p - oh * g.Wo;

  A acc[CC];
#pragma unroll
  for (int j = 0; j < CC; ++j) acc[j] = (A)0;
  const T* off_n = off + (size_t)n * g.taps * 2 * g.P + p;
  const T* rot_n = rot + (size_t)(n * g.G + grp) * g.taps * 2 * g.P + p;
  const T* x_n = x + ((size_t)n * g.C + grp + (size_t)g.G * j0) * g.HW;
  const size_t cstride = (size_t)g.G * g.HW;

  for (int fh = 0; fh < g.kH; ++fh) {
    const int ih = oh * g.sH - g.pH + fh * g.dH;
    for (int fw = 0; fw < g.kW; ++fw) {
      const int iw = ow * g.sW - g.pW + fw * g.dW;
      const int t = fh * g.kW + fw;
      Bilinear<A> bi;
      if (!image_setup<A>((A)ih + ld<A>(off_n + (size_t)t * 2 * g.P), (A)iw + ld<A>(off_n + (size_t)(t * 2 + 1) * g.P), g,
                          bi))
        continue;
      Bilinear<A> bb;
      if (!bank_setup<A>(ld<A>(rot_n + (size_t)t * 2 * g.P), ld<A>(rot_n + (size_t)(t * 2 + 1) * g.P), fh, fw, g, bb))
        continue;
      A ci[4], cb[4];
      bilinear_value_coefs(bi, ci);
      bilinear_value_coefs(bb, cb);
#pragma unroll
      for (int j = 0; j < CC; ++j) {
        if (j < cnt) {
          const T* xp = x_n + j * cstride;
          const A xs = ci[0] * ld<A>(xp + bi.idx[0]) + ci[1] * ld<A>(xp + bi.idx[1]) + ci[2] * ld<A>(xp + bi.idx[2]) +
                       ci[3] * ld<A>(xp + bi.idx[3]);
          const A* bk = bank + j * g.cells;
          const A k = cb[0] * bk[bb.idx[0]] + cb[1] * bk[bb.idx[1]] + cb[2] * bk[bb.idx[2]] + cb[3] * bk[bb.idx[3]];
          acc[j] += xs * k;
        }
      }
    }
  }
  T* y_n = y + ((size_t)n * g.C + grp + (size_t)g.G * j0) * g.P + p;
  const size_t ystride = (size_t)g.G * g.P;
#pragma unroll
  for (int j = 0; j < CC; ++j)
    if (j < cnt) st<T, A>(y_n + j * ystride, acc[j]);
}

template <typename T>
int deform_forward(const T* x, const T* off, const T* rot, const T* w, T* y, const Geom& g, cudaStream_t s) {
  if constexpr (std::is_same<T, __half>::value) {
    if (mma_path_enabled()) {
      const int rc = deform_forward_mma(x, off, rot, w, y, g, s);
      if (rc != DK_ERR_UNSUPPORTED) return rc;
    }
  }
  using A = typename Compute<T>::type;
  constexpr int CC = 16, BLOCK = 256;
  const long long bx = ((long long)g.N * g.P + BLOCK - 1) / BLOCK;
  const int by = (g.Cg + CC - 1) / CC;
  if (bx > 0x7fffffffLL || by > 65535 || g.G > 65535) return DK_ERR_UNSUPPORTED;
  const size_t smem = (size_t)CC * g.cells * sizeof(A);
  if (smem > (size_t)device_smem_optin()) return DK_ERR_UNSUPPORTED;
  auto kern = deform_fwd_kernel<T, CC, BLOCK>;
  int rc = enable_smem(kern, smem);
  if (rc) return rc;
  kern<<<dim3((unsigned)bx, by, g.G), BLOCK, smem, s>>>(x, off, rot, w, y, g);
  return check_launch();
}

// ------------------------------------------------------------------ grad-input (scatter)
// Same decomposition as the forward; each (pixel, tap, channel) adds dy * k * corner
// coefficient into up to four input locations with red.global.add in the compute type.
// fp16 runs accumulate in an fp32 workspace and are rounded once by a second kernel.
template <typename T, int CC, int BLOCK>
__global__ void __launch_bounds__(BLOCK) deform_data_kernel(const T* __restrict__ dy, const T* __restrict__ off,
                                                            const T* __restrict__ rot, const T* __restrict__ w,
                                                            typename Compute<T>::type* __restrict__ dx, const Geom g) {
  using A = typename Compute<T>::type;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  A* bank = reinterpret_cast<A*>(smem_raw);
  const int grp = blockIdx.z;
  const int j0 = blockIdx.y * CC;
  const int cnt = min(CC, g.Cg - j0);
  for (int i = threadIdx.x; i < CC * g.cells; i += BLOCK) {
    const int j = i / g.cells, cell = i - j * g.cells;
    bank[i] = (j < cnt) ? ld<A>(w + (size_t)(grp + g.G * (j0 + j)) * g.cells + cell) : (A)0;
  }
  __syncthreads();
  const long long total = (long long)g.N * g.P;
  const long long flat = (long long)blockIdx.x * BLOCK + threadIdx.x;
  if (flat >= total) return;
  const int n = (int)(flat / g.P);
  const int p = (int)(flat - (long long)n * g.P);
  const int oh = p / g.Wo, ow = p - oh * g.Wo;

  A dyv[CC];
  const T* dy_n = dy + ((size_t)n * g.C + grp + (size_t)g.G * j0) * g.P + p;
#pragma unroll
  for (int j = 0; j < CC; ++j) dyv[j] = (j < cnt) ? ld<A>(dy_n + (size_t)j * g.G * g.P) : (A)0;

  const T* off_n = off + (size_t)n * g.taps * 2 * g.P + p;
  const T* rot_n = rot + (size_t)(n * g.G + grp) * g.taps * 2 * g.P + p;
  A* dx_n = dx + ((size_t)n * g.C + grp + (size_t)g.G * j0) * g.HW;
  const size_t cstride = (size_t)g.G * g.HW;

  for (int fh = 0; fh < g.kH; ++fh) {
    const int ih = oh * g.sH - g.pH + fh * g.dH;
    for (int fw = 0; fw < g.kW; ++fw) {
      const int iw = ow * g.sW - g.pW + fw * g.dW;
      const int t = fh * g.kW + fw;
      Bilinear<A> bi;
      if (!image_setup<A>((A)ih + ld<A>(off_n + (size_t)t * 2 * g.P), (A)iw + ld<A>(off_n + (size_t)(t * 2 + 1) * g.P), g,
                          bi))
        continue;
      Bilinear<A> bb;
      if (!bank_setup<A>(ld<A>(rot_n + (size_t)t * 2 * g.P), ld<A>(rot_n + (size_t)(t * 2 + 1) * g.P), fh, fw, g, bb))
        continue;
      A ci[4], cb[4];
      bilinear_value_coefs(bi, ci);
      bilinear_value_coefs(bb, cb);
#pragma unroll
      for (int j = 0; j < CC; ++j) {
        if (j < cnt) {
          const A* bk = bank + j * g.cells;
          const A k = cb[0] * bk[bb.idx[0]] + cb[1] * bk[bb.idx[1]] + cb[2] * bk[bb.idx[2]] + cb[3] * bk[bb.idx[3]];
          const A v = k * dyv[j];
          A* dp = dx_n + j * cstride;
#pragma unroll
          for (int q = 0; q < 4; ++q)
            if (bi.m[q]) atomicAdd(dp + bi.idx[q], ci[q] * v);
        }
      }
    }
  }
}

// Variant for planes that fit in shared memory: a block owns sample n and CP channels, keeps their
// grad-input planes on chip in the compute type, scatters into them with shared-memory atomics and
// writes each plane out once, coalesced and already rounded -- no global atomics, no zero-fill
// pass, no fp32 scratch tensor, no conversion pass.
template <typename T, int CP, int BLOCK>
__global__ void __launch_bounds__(BLOCK) deform_data_plane_kernel(const T* __restrict__ dy, const T* __restrict__ off,
                                                                  const T* __restrict__ rot, const T* __restrict__ w,
                                                                  T* __restrict__ dx, const Geom g) {
  using A = typename Compute<T>::type;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  A* bank = reinterpret_cast<A*>(smem_raw);  // [CP][cells]
  A* planes = bank + CP * g.cells;           // [CP][HW]
  const int grp = blockIdx.z;
  const int j0 = blockIdx.y * CP;
  const int cnt = min(CP, g.Cg - j0);
  const int n = blockIdx.x;
  for (int i = threadIdx.x; i < CP * g.cells; i += BLOCK) {
    const int j = i / g.cells, cell = i - j * g.cells;
    bank[i] = (j < cnt) ? ld<A>(w + (size_t)(grp + g.G * (j0 + j)) * g.cells + cell) : (A)0;
  }
  for (int i = threadIdx.x; i < CP * g.HW; i += BLOCK) planes[i] = (A)0;
  __syncthreads();

  const T* dy_n = dy + ((size_t)n * g.C + grp + (size_t)g.G * j0) * g.P;
  const T* off_n = off + (size_t)n * g.taps * 2 * g.P;
  const T* rot_n = rot + (size_t)(n * g.G + grp) * g.taps * 2 * g.P;
  for (int p = threadIdx.x; p < g.P; p += BLOCK) {
    const int oh = p / g.Wo, ow = p - oh * g.Wo;
    A dyv[CP];
#pragma unroll
    for (int j = 0; j < CP; ++j) dyv[j] = (j < cnt) ? ld<A>(dy_n + (size_t)j * g.G * g.P + p) : (A)0;
    for (int fh = 0; fh < g.kH; ++fh) {
      const int ih = oh * g.sH - g.pH + fh * g.dH;
      for (int fw = 0; fw < g.kW; ++fw) {
        const int iw = ow * g.sW - g.pW + fw * g.dW;
        const int t = fh * g.kW + fw;
        Bilinear<A> bi;
        if (!image_setup<A>((A)ih + ld<A>(off_n + (size_t)t * 2 * g.P + p), (A)iw + ld<A>(off_n + (size_t)(t * 2 + 1) * g.P + p),
                            g, bi))
          continue;
        Bilinear<A> bb;
        if (!bank_setup<A>(ld<A>(rot_n + (size_t)t * 2 * g.P + p), ld<A>(rot_n + (size_t)(t * 2 + 1) * g.P + p), fh, fw, g, bb))
          continue;
        A ci[4], cb[4];
        bilinear_value_coefs(bi, ci);
        bilinear_value_coefs(bb, cb);
#pragma unroll
        for (int j = 0; j < CP; ++j) {
          if (j < cnt) {
            const A* bk = bank + j * g.cells;
            const A k = cb[0] * bk[bb.idx[0]] + cb[1] * bk[bb.idx[1]] + cb[2] * bk[bb.idx[2]] + cb[3] * bk[bb.idx[3]];
            const A v = k * dyv[j];
            A* dp = planes + j * g.HW;
#pragma unroll
            for (int q = 0; q < 4; ++q)
              if (bi.m[q]) atomicAdd(dp + bi.idx[q], ci[q] * v);
          }
        }
      }
    }
  }
  __syncthreads();
  for (int j = 0; j < cnt; ++j) {
    T* o = dx + ((size_t)n * g.C + grp + (size_t)g.G * (j0 + j)) * g.HW;
    const A* sp = planes + j * g.HW;
    for (int i = threadIdx.x; i < g.HW; i += BLOCK) st<T, A>(o + i, sp[i]);
  }
}

template <typename T, typename A>
__global__ void convert_kernel(const A* __restrict__ src, T* __restrict__ dst, const size_t n) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) st<T, A>(dst + i, src[i]);
}

template <typename T>
int deform_backward_data(const T* dy, const T* off, const T* rot, const T* w, T* dx, const Geom& g, void* ws,
                         size_t ws_bytes, cudaStream_t s) {
  using A = typename Compute<T>::type;
  constexpr int CC = 16, BLOCK = 256;
  if constexpr (std::is_same<T, __half>::value) {
    if (mma_path_enabled()) {
      const int rc = deform_data_mma(dy, off, rot, w, dx, g, ws, ws_bytes, s);
      if (rc != DK_ERR_UNSUPPORTED) return rc;
    }
  }
  {
    // planes of 8 channels in shared memory, when they fit
    constexpr int CP = 8;
    const size_t psmem = (size_t)CP * (g.HW + g.cells) * sizeof(A);
    const int byp = (g.Cg + CP - 1) / CP;
    if (psmem <= 110 * 1024 && psmem <= (size_t)device_smem_optin() && byp <= 65535 && g.G <= 65535 && g.P >= 64) {
      auto kern = deform_data_plane_kernel<T, CP, 512>;
      int rc = enable_smem(kern, psmem);
      if (rc) return rc;
      kern<<<dim3(g.N, byp, g.G), 512, psmem, s>>>(dy, off, rot, w, dx, g);
      return check_launch();
    }
  }
  constexpr bool direct = sizeof(T) == sizeof(A);
  const size_t count = (size_t)g.N * g.C * g.HW;
  A* accbuf;
  if (direct) {
    accbuf = reinterpret_cast<A*>(dx);
  } else {
    if (ws == nullptr || ws_bytes < count * sizeof(A)) return DK_ERR_WORKSPACE;
    accbuf = reinterpret_cast<A*>(ws);
  }
  cudaError_t e = cudaMemsetAsync(accbuf, 0, count * sizeof(A), s);
  if (e != cudaSuccess) {
    set_last_cuda_error(e);
    return DK_ERR_CUDA;
  }
  const long long bx = ((long long)g.N * g.P + BLOCK - 1) / BLOCK;
  const int by = (g.Cg + CC - 1) / CC;
  if (bx > 0x7fffffffLL || by > 65535 || g.G > 65535) return DK_ERR_UNSUPPORTED;
  const size_t smem = (size_t)CC * g.cells * sizeof(A);
  if (smem > (size_t)device_smem_optin()) return DK_ERR_UNSUPPORTED;
  auto kern = deform_data_kernel<T, CC, BLOCK>;
  int rc = enable_smem(kern, smem);
  if (rc) return rc;
  kern<<<dim3((unsigned)bx, by, g.G), BLOCK, smem, s>>>(dy, off, rot, w, accbuf, g);
  rc = check_launch();
  if (rc) return rc;
  if (!direct) {
    const size_t blocks = (count + 255) / 256;
    if (blocks > 0x7fffffffULL) return DK_ERR_UNSUPPORTED;
    convert_kernel<T, A><<<(unsigned)blocks, 256, 0, s>>>(accbuf, dx, count);
    rc = check_launch();
  }
  return rc;
}

// ------------------------------------------------------------------ coordinate gradients
// Gradient wrt the image-space offsets (sum over ALL channels) and wrt the kernel-space
// offsets (sum over the channels of each rotation group), fused: both need the same four
// image corners, the same four bank corners and the same grad-output per channel.
// Block = 32 pixels (lanes) x NW warps; warp w takes channels w, w+NW, ... ; partial sums
// meet in shared memory.  No atomics.
template <typename T, int NW, bool BANK_SMEM, bool DO_OFF, bool DO_ROT>
__global__ void __launch_bounds__(32 * NW) deform_coords_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                                                const T* __restrict__ off, const T* __restrict__ rot,
                                                                const T* __restrict__ w, T* __restrict__ doff,
                                                                T* __restrict__ drot, const Geom g) {
  using A = typename Compute<T>::type;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  A* red = reinterpret_cast<A*>(smem_raw);  // [NW][4][32]
  A* bank = red + NW * 4 * 32;              // [C][cells] if BANK_SMEM
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (BANK_SMEM) {
    for (int i = threadIdx.x; i < g.C * g.cells; i += 32 * NW) bank[i] = ld<A>(w + i);
    __syncthreads();
  }
  const long long total = (long long)g.N * g.P;
  const long long flat = (long long)blockIdx.x * 32 + lane;
  const bool active = flat < total;
  const int n = active ? (int)(flat / g.P) : 0;
  const int p = active ? (int)(flat - (long long)n * g.P) : 0;
  const int oh = p / g.Wo, ow = p - oh * g.Wo;
  const T* off_n = off + (size_t)n * g.taps * 2 * g.P + p;
  T* doff_n = doff + (size_t)n * g.taps * 2 * g.P + p;
  const T* x_n = x + (size_t)n * g.C * g.HW;
  const T* dy_n = dy + (size_t)n * g.C * g.P + p;

  for (int fh = 0; fh < g.kH; ++fh) {
    const int ih = oh * g.sH - g.pH + fh * g.dH;
    for (int fw = 0; fw < g.kW; ++fw) {
      const int iw = ow * g.sW - g.pW + fw * g.dW;
      const int t = fh * g.kW + fw;
      Bilinear<A> bi;
      bool used = false;
      A ci[4], cih[4], ciw[4];
      if (active) {
        used = image_setup<A>((A)ih + ld<A>(off_n + (size_t)t * 2 * g.P), (A)iw + ld<A>(off_n + (size_t)(t * 2 + 1) * g.P),
                              g, bi);
        bilinear_value_coefs(bi, ci);
        bilinear_du_coefs(bi, cih);
        bilinear_dv_coefs(bi, ciw);
      }
      A goh = (A)0, gow = (A)0;
      for (int grp = 0; grp < g.G; ++grp) {
        A grh = (A)0, grw = (A)0;
        if (used) {
          const T* r = rot + ((size_t)(n * g.G + grp) * g.taps + t) * 2 * g.P + p;
          Bilinear<A> bb;
          if (bank_setup<A>(ld<A>(r), ld<A>(r + g.P), fh, fw, g, bb)) {
            A cb[4], cu[4], cv[4];
            bilinear_value_coefs(bb, cb);
            bilinear_du_coefs(bb, cu);
            bilinear_dv_coefs(bb, cv);
            for (int j = warp; j < g.Cg; j += NW) {
              const size_t c = (size_t)grp + (size_t)g.G * j;
              const T* xp = x_n + c * g.HW;
              A xv[4], wv[4];
#pragma unroll
              for (int q = 0; q < 4; ++q) xv[q] = ld<A>(xp + bi.idx[q]);
              if (BANK_SMEM) {
                const A* bk = bank + c * g.cells;
#pragma unroll
                for (int q = 0; q < 4; ++q) wv[q] = bk[bb.idx[q]];
              } else {
                const T* bk = w + c * g.cells;
#pragma unroll
                for (int q = 0; q < 4; ++q) wv[q] = ld<A>(bk + bb.idx[q]);
              }
              const A dyv = ld<A>(dy_n + c * g.P);
              if (DO_OFF) {
                const A kd = dot4(cb, wv) * dyv;
                goh += dot4(cih, xv) * kd;
                gow += dot4(ciw, xv) * kd;
              }
              if (DO_ROT) {
                const A xd = dot4(ci, xv) * dyv;
                grh += xd * dot4(cu, wv);
                grw += xd * dot4(cv, wv);
              }
            }
          }
        }
        if (DO_ROT) {
          red[(warp * 4 + 0) * 32 + lane] = grh;
          red[(warp * 4 + 1) * 32 + lane] = grw;
          __syncthreads();
          if (warp < 2 && active) {
            A sum = (A)0;
#pragma unroll
            for (int q = 0; q < NW; ++q) sum += red[(q * 4 + warp) * 32 + lane];
            st<T, A>(drot + ((size_t)(n * g.G + grp) * g.taps + t) * 2 * g.P + (size_t)warp * g.P + p, sum);
          }
          __syncthreads();
        }
      }
      if (DO_OFF) {
        red[(warp * 4 + 2) * 32 + lane] = goh;
        red[(warp * 4 + 3) * 32 + lane] = gow;
        __syncthreads();
        if (warp < 2 && active) {
          A sum = (A)0;
#pragma unroll
          for (int q = 0; q < NW; ++q) sum += red[(q * 4 + 2 + warp) * 32 + lane];
          st<T, A>(doff_n + (size_t)(t * 2 + warp) * g.P, sum);
        }
        __syncthreads();
      }
    }
  }
}

template <typename T, bool DO_OFF, bool DO_ROT>
static int launch_coords(const T* dy, const T* x, const T* off, const T* rot, const T* w, T* doff, T* drot, const Geom& g,
                         cudaStream_t s) {
  using A = typename Compute<T>::type;
  constexpr int NW = 8;
  const long long bx = ((long long)g.N * g.P + 31) / 32;
  if (bx > 0x7fffffffLL) return DK_ERR_UNSUPPORTED;
  const size_t red_bytes = (size_t)NW * 4 * 32 * sizeof(A);
  const size_t bank_bytes = (size_t)g.C * g.cells * sizeof(A);
  if (red_bytes + bank_bytes <= 100 * 1024) {
    auto kern = deform_coords_kernel<T, NW, true, DO_OFF, DO_ROT>;
    int rc = enable_smem(kern, red_bytes + bank_bytes);
    if (rc) return rc;
    kern<<<(unsigned)bx, 32 * NW, red_bytes + bank_bytes, s>>>(dy, x, off, rot, w, doff, drot, g);
  } else {
    deform_coords_kernel<T, NW, false, DO_OFF, DO_ROT><<<(unsigned)bx, 32 * NW, red_bytes, s>>>(dy, x, off, rot, w, doff,
                                                                                               drot, g);
  }
  return check_launch();
}

template <typename T>
int deform_backward_coords(const T* dy, const T* x, const T* off, const T* rot, const T* w, T* doff, T* drot,
                           const Geom& g, cudaStream_t s) {
  if (doff && drot) return launch_coords<T, true, true>(dy, x, off, rot, w, doff, drot, g, s);
  if (doff) return launch_coords<T, true, false>(dy, x, off, rot, w, doff, drot, g, s);
  if (drot) return launch_coords<T, false, true>(dy, x, off, rot, w, doff, drot, g, s);
  return DK_OK;
}

#define DK_INSTANTIATE_DEFORM(T)                                                                                       \
  template int deform_forward<T>(const T*, const T*, const T*, const T*, T*, const Geom&, cudaStream_t);               \
  template int deform_backward_data<T>(const T*, const T*, const T*, const T*, T*, const Geom&, void*, size_t,         \
                                       cudaStream_t);                                                                 \
  template int deform_backward_coords<T>(const T*, const T*, const T*, const T*, const T*, T*, T*, const Geom&,        \
                                         cudaStream_t);
DK_INSTANTIATE_DEFORM(float)
DK_INSTANTIATE_DEFORM(__half)
DK_INSTANTIATE_DEFORM(double)

}  // namespace dk
