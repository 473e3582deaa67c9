// Local deformable kernel (depthwise conv whose 3x3 kernel is resampled per output
// location from a scope-sized weight bank): forward and the three gradients.
//
// Work decomposition, common to the kernels here
//   * the sampling basis of a (pixel, tap) -- four bank corner indices and their
//     coefficients -- does not depend on the channel: a thread computes it once and
//     reuses it for every channel it handles (the reference recomputes it per channel);
//   * the weight banks of the block's channels live in shared memory as fp32;
//   * all arithmetic is in the compute type (fp32 for fp16/fp32 storage).
#include <cstdlib>
#include <type_traits>

#include "dk_common.cuh"

namespace dk {

// The fp16 fast path can be switched off (DK_B200_DISABLE_MMA=1) to compare against the SIMT kernels.
bool mma_path_enabled() {
  static const bool on = [] {
    const char* v = std::getenv("DK_B200_DISABLE_MMA");
    return !(v && v[0] && v[0] != '0');
  }();
  return on;
}

// ------------------------------------------------------------------ forward / grad-input
// One thread = one (n, pixel); a block covers BLOCK consecutive pixels of the flattened
// (n, oh, ow) axis and CC channels of one rotation group; taps outer, channels inner with
// CC accumulators in registers.  TRANSPOSED = false: forward (pixel = output location,
// source = input).  TRANSPOSED = true: grad-input in gather form (pixel = input location,
// source = grad-output; a tap contributes iff (ih + pad - fh*dil) is a multiple of the
// stride and the quotient is a valid output row).
template <typename T, int CC, int BLOCK, bool TRANSPOSED>
__global__ void __launch_bounds__(BLOCK) local_conv_kernel(const T* __restrict__ src, const T* __restrict__ rot,
                                                           const T* __restrict__ w, T* __restrict__ dst, const Geom g) {
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

  const int dst_plane = TRANSPOSED ? g.HW : g.P;   // pixels per plane on the thread side
  const int dst_w = TRANSPOSED ? g.W : g.Wo;
  const int src_plane = TRANSPOSED ? g.P : g.HW;
  const long long total = (long long)g.N * dst_plane;
  const long long flat = (long long)blockIdx.x * BLOCK + threadIdx.x;
  if (flat >= total) return;
  const int n = (int)(flat / dst_plane);
  const int p = (int)(flat - (long long)n * dst_plane);
  const int ph = p / dst_w, pw = p - ph * dst_w;

  A acc[CC];
#pragma unroll
  for (int j = 0; j < CC; ++j) acc[j] = (A)0;

  const T* rot_n = rot + (size_t)(n * g.G + grp) * g.taps * 2 * g.P;
  const T* src_n = src + ((size_t)n * g.C + grp + (size_t)g.G * j0) * src_plane;
  const size_t cstride = (size_t)g.G * src_plane;

  for (int fh = 0; fh < g.kH; ++fh) {
    int sh;  // row on the source side
    bool okh;
    if (!TRANSPOSED) {
      sh = ph * g.sH - g.pH + fh * g.dH;
      okh = sh >= 0 && sh < g.H;
    } else {
      const int th = ph + g.pH - fh * g.dH;
      sh = th / g.sH;
      okh = th >= 0 && (th - sh * g.sH) == 0 && sh < g.Ho;
    }
    for (int fw = 0; fw < g.kW; ++fw) {
      int sw;
      bool okw;
      if (!TRANSPOSED) {
        sw = pw * g.sW - g.pW + fw * g.dW;
        okw = sw >= 0 && sw < g.W;
      } else {
        const int tw = pw + g.pW - fw * g.dW;
        sw = tw / g.sW;
        okw = tw >= 0 && (tw - sw * g.sW) == 0 && sw < g.Wo;
      }
      if (!(okh && okw)) continue;
      // output location whose offsets drive this tap
      const int op = TRANSPOSED ? (sh * g.Wo + sw) : p;
      const int so = TRANSPOSED ? op : (sh * g.W + sw);
      const T* r = rot_n + (size_t)((fh * g.kW + fw) * 2) * g.P + op;
      Bilinear<A> b;
      bank_setup<A>(ld<A>(r), ld<A>(r + g.P), fh, fw, g, b);
      A c[4];
      bilinear_value_coefs(b, c);
      const T* sp = src_n + so;
#pragma unroll
      for (int j = 0; j < CC; ++j) {
        if (j < cnt) {
          const A* bk = bank + j * g.cells;
          const A k = c[0] * bk[b.idx[0]] + c[1] * bk[b.idx[1]] + c[2] * bk[b.idx[2]] + c[3] * bk[b.idx[3]];
          acc[j] += ld<A>(sp + j * cstride) * k;
        }
      }
    }
  }
  T* dst_n = dst + ((size_t)n * g.C + grp + (size_t)g.G * j0) * dst_plane + p;
  const size_t dstride = (size_t)g.G * dst_plane;
#pragma unroll
  for (int j = 0; j < CC; ++j)
    if (j < cnt) st<T, A>(dst_n + j * dstride, acc[j]);
}

template <typename T, bool TRANSPOSED, int CC, int BLOCK>
static int launch_local_conv_simt(const T* src, const T* rot, const T* w, T* dst, const Geom& g, long long total, cudaStream_t s) {
  using A = typename Compute<T>::type;
  const long long bx = (total + BLOCK - 1) / BLOCK;
  const int by = (g.Cg + CC - 1) / CC;
  if (bx > 0x7fffffffLL || by > 65535 || g.G > 65535) return DK_ERR_UNSUPPORTED;
  const size_t smem = (size_t)CC * g.cells * sizeof(A);
  if (smem > (size_t)device_smem_optin()) return DK_ERR_UNSUPPORTED;
  auto kern = local_conv_kernel<T, CC, BLOCK, TRANSPOSED>;
  int rc = enable_smem(kern, smem);
  if (rc) return rc;
  kern<<<dim3((unsigned)bx, by, g.G), BLOCK, smem, s>>>(src, rot, w, dst, g);
  return check_launch();
}

template <typename T, bool TRANSPOSED>
static int launch_local_conv(const T* src, const T* rot, const T* w, T* dst, const Geom& g, cudaStream_t s) {
  using A = typename Compute<T>::type;
  if constexpr (std::is_same<T, __half>::value) {
    if (mma_path_enabled()) {
      int rc = local_conv_ring(src, rot, w, dst, g, TRANSPOSED, s);
      if (rc != DK_ERR_UNSUPPORTED) return rc;
      rc = local_conv_mma(src, rot, w, dst, g, TRANSPOSED, s);
      if (rc != DK_ERR_UNSUPPORTED) return rc;
    }
  }
  const long long total = (long long)g.N * (TRANSPOSED ? g.HW : g.P);
  // 16 channels per thread amortise the sampling basis of a (pixel, tap); a call too small to fill the GPU that way
  // (under two blocks per SM) takes 4 channels per thread and blocks of 64 instead: four times the threads, a quarter
  // of the serial work in each
  const bool tiny = ((total + 255) / 256) * ((g.Cg + 15) / 16) * g.G < 2LL * device_sm_count() && g.Cg > 4;
  return tiny ? launch_local_conv_simt<T, TRANSPOSED, 4, 64>(src, rot, w, dst, g, total, s)
              : launch_local_conv_simt<T, TRANSPOSED, 16, 256>(src, rot, w, dst, g, total, s);
}

template <typename T>
int local_forward(const T* x, const T* rot, const T* w, T* y, const Geom& g, cudaStream_t s) {
  return launch_local_conv<T, false>(x, rot, w, y, g, s);
}
template <typename T>
int local_backward_data(const T* dy, const T* rot, const T* w, T* dx, const Geom& g, cudaStream_t s) {
  return launch_local_conv<T, true>(dy, rot, w, dx, g, s);
}

// ------------------------------------------------------------------ grad-offsets (rotation)
// Block = 32 pixels (lanes) x NW warps; warp w takes channels w, w+NW, ... of the group and
// keeps the (h, w) offset gradient of the current tap in registers; the NW partial sums
// meet in shared memory.  No atomics, fixed summation order.
template <typename T, int NW, bool BANK_SMEM>
__global__ void __launch_bounds__(32 * NW) local_rot_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                                            const T* __restrict__ rot, const T* __restrict__ w,
                                                            T* __restrict__ drot, const Geom g) {
  using A = typename Compute<T>::type;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  A* red = reinterpret_cast<A*>(smem_raw);          // [NW][2][32]
  A* bank = red + NW * 2 * 32;                      // [Cg][cells] if BANK_SMEM

  const int grp = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (BANK_SMEM) {
    for (int i = threadIdx.x; i < g.Cg * g.cells; i += 32 * NW) {
      const int j = i / g.cells, cell = i - j * g.cells;
      bank[i] = ld<A>(w + (size_t)(grp + g.G * j) * g.cells + cell);
    }
    __syncthreads();
  }
  const long long total = (long long)g.N * g.P;
  const long long flat = (long long)blockIdx.x * 32 + lane;
  const bool active = flat < total;
  const int n = active ? (int)(flat / g.P) : 0;
  const int p = active ? (int)(flat - (long long)n * g.P) : 0;
  const int oh = p / g.Wo, ow = p - oh * g.Wo;
  const T* rot_n = rot + (size_t)(n * g.G + grp) * g.taps * 2 * g.P + p;
  T* drot_n = drot + (size_t)(n * g.G + grp) * g.taps * 2 * g.P + p;
  const T* x_n = x + ((size_t)n * g.C + grp) * g.HW;
  const T* dy_n = dy + ((size_t)n * g.C + grp) * g.P + p;

  for (int fh = 0; fh < g.kH; ++fh) {
    const int ih = oh * g.sH - g.pH + fh * g.dH;
    for (int fw = 0; fw < g.kW; ++fw) {
      const int iw = ow * g.sW - g.pW + fw * g.dW;
      const int t = fh * g.kW + fw;
      const bool inside = active && ih >= 0 && ih < g.H && iw >= 0 && iw < g.W;
      A gu = (A)0, gv = (A)0;
      if (inside) {
        Bilinear<A> b;
        const bool valid = bank_setup<A>(ld<A>(rot_n + (size_t)t * 2 * g.P), ld<A>(rot_n + (size_t)(t * 2 + 1) * g.P), fh,
                                         fw, g, b);
        if (valid) {
          A cu[4], cv[4];
          bilinear_du_coefs(b, cu);
          bilinear_dv_coefs(b, cv);
          const T* xp = x_n + ih * g.W + iw;
          for (int j = warp; j < g.Cg; j += NW) {
            const size_t c = (size_t)g.G * j;
            const A s = ld<A>(xp + c * g.HW) * ld<A>(dy_n + c * g.P);
            A wv[4];
            if (BANK_SMEM) {
              const A* bk = bank + j * g.cells;
#pragma unroll
              for (int q = 0; q < 4; ++q) wv[q] = bk[b.idx[q]];
            } else {
              const T* bk = w + (size_t)(grp + c) * g.cells;
#pragma unroll
              for (int q = 0; q < 4; ++q) wv[q] = ld<A>(bk + b.idx[q]);
            }
            gu += s * dot4(cu, wv);
            gv += s * dot4(cv, wv);
          }
        }
      }
      red[(warp * 2 + 0) * 32 + lane] = gu;
      red[(warp * 2 + 1) * 32 + lane] = gv;
      __syncthreads();
      if (warp < 2 && active) {
        A sum = (A)0;
#pragma unroll
        for (int q = 0; q < NW; ++q) sum += red[(q * 2 + warp) * 32 + lane];
        st<T, A>(drot_n + (size_t)(t * 2 + warp) * g.P, sum);
      }
      __syncthreads();
    }
  }
}

template <typename T>
int local_backward_rotation(const T* dy, const T* x, const T* rot, const T* w, T* drot, const Geom& g, void* ws,
                            size_t ws_bytes, cudaStream_t s) {
  using A = typename Compute<T>::type;
  if constexpr (std::is_same<T, __half>::value) {
    if (mma_path_enabled()) {
      const int rc = local_rot_mma(dy, x, rot, w, drot, g, ws, ws_bytes, s);
      if (rc != DK_ERR_UNSUPPORTED) return rc;
    }
  }
  constexpr int NW = 8;
  const long long bx = ((long long)g.N * g.P + 31) / 32;
  if (bx > 0x7fffffffLL || g.G > 65535) return DK_ERR_UNSUPPORTED;
  const size_t red_bytes = (size_t)NW * 2 * 32 * sizeof(A);
  const size_t bank_bytes = (size_t)g.Cg * g.cells * sizeof(A);
  const bool fits = red_bytes + bank_bytes <= 100 * 1024;
  if (fits) {
    auto kern = local_rot_kernel<T, NW, true>;
    int rc = enable_smem(kern, red_bytes + bank_bytes);
    if (rc) return rc;
    kern<<<dim3((unsigned)bx, g.G), 32 * NW, red_bytes + bank_bytes, s>>>(dy, x, rot, w, drot, g);
  } else {
    local_rot_kernel<T, NW, false><<<dim3((unsigned)bx, g.G), 32 * NW, red_bytes, s>>>(dy, x, rot, w, drot, g);
  }
  return check_launch();
}

// ------------------------------------------------------------------ grad-weight (bank)
// Lanes = channels.  A warp owns 32 channels of one rotation group and walks a range of
// the flattened (n, oh, ow) axis; its bank-gradient accumulators sit in shared memory as
// [cell][lane], so every read-modify-write is private to one lane and free of bank
// conflicts -- the same-address atomics of the reference
// (csrc/filter_sample_depthwise_cuda_kernel.cu:910-916) disappear.  The sampling basis of a batch of
// pixels is computed once per block into shared memory and shared by all warps.  Each
// block writes one fp32 partial bank gradient; a second kernel sums the partials in a
// fixed order.
// One table entry per (pixel of the batch, tap).  For DK+DCN (DEFORM) the input sample is
// itself bilinear: four image corners and their coefficients.
template <typename A, bool DEFORM>
struct TapEntry {
  int src[DEFORM ? 4 : 1];   // offsets of the input sample(s) inside the plane; src[0] < 0: tap unused
  A sc[DEFORM ? 4 : 1];      // image corner coefficients (DEFORM only)
  int idx[4];                // bank corner cells
  A c[4];                    // bank value coefficients
};

constexpr int kFilterPixBatch = 32;

template <typename T, bool DEFORM>
__global__ void filter_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ off,
                              const T* __restrict__ rot, typename Compute<T>::type* __restrict__ partial, const Geom g,
                              const long long pix_per_block, const int warps) {
  using A = typename Compute<T>::type;
  using Entry = TapEntry<A, DEFORM>;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  A* acc_all = reinterpret_cast<A*>(smem_raw);                                      // [warps][cells][32]
  Entry* table = reinterpret_cast<Entry*>(acc_all + (size_t)warps * g.cells * 32);  // [batch][taps]

  const int grp = blockIdx.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nthreads = warps * 32;
  const int j = (blockIdx.y * warps + warp) * 32 + lane;  // channel index inside the group
  const bool chan_ok = j < g.Cg;
  const size_t c = (size_t)grp + (size_t)g.G * (chan_ok ? j : 0);
  A* acc = acc_all + (size_t)warp * g.cells * 32;
  for (int i = lane; i < g.cells * 32; i += 32) acc[i] = (A)0;

  const long long total = (long long)g.N * g.P;
  const long long begin = (long long)blockIdx.x * pix_per_block;
  const long long end = begin + pix_per_block < total ? begin + pix_per_block : total;

  for (long long base = begin; base < end; base += kFilterPixBatch) {
    const int nb = (int)((end - base) < kFilterPixBatch ? (end - base) : kFilterPixBatch);
    __syncthreads();
    for (int i = threadIdx.x; i < nb * g.taps; i += nthreads) {
      const int pl = i / g.taps, t = i - pl * g.taps;
      const long long flat = base + pl;
      const int n = (int)(flat / g.P);
      const int p = (int)(flat - (long long)n * g.P);
      const int oh = p / g.Wo, ow = p - oh * g.Wo;
      const int fh = t / g.kW, fw = t - fh * g.kW;
      const int ih = oh * g.sH - g.pH + fh * g.dH, iw = ow * g.sW - g.pW + fw * g.dW;
      Entry e;
      e.src[0] = -1;
#pragma unroll
      for (int q = 0; q < 4; ++q) { e.idx[q] = 0; e.c[q] = (A)0; }
      bool used;
      Bilinear<A> bi;
      if (DEFORM) {
        const T* o = off + ((size_t)n * g.taps + t) * 2 * g.P + p;
        used = image_setup<A>((A)ih + ld<A>(o), (A)iw + ld<A>(o + g.P), g, bi);
      } else {
        used = ih >= 0 && ih < g.H && iw >= 0 && iw < g.W;
      }
      if (used) {
        const T* r = rot + ((size_t)(n * g.G + grp) * g.taps + t) * 2 * g.P + p;
        Bilinear<A> b;
        if (bank_setup<A>(ld<A>(r), ld<A>(r + g.P), fh, fw, g, b)) {
          bilinear_value_coefs(b, e.c);
#pragma unroll
          for (int q = 0; q < 4; ++q) e.idx[q] = b.idx[q];
          if (DEFORM) {
            A sc[4];
            bilinear_value_coefs(bi, sc);
#pragma unroll
            for (int q = 0; q < (DEFORM ? 4 : 1); ++q) { e.src[q] = bi.idx[q]; e.sc[q] = sc[q]; }
          } else {
            e.src[0] = ih * g.W + iw;
          }
        }
      }
      table[i] = e;
    }
    __syncthreads();
    if (chan_ok) {
      for (int pl = 0; pl < nb; ++pl) {
        const long long flat = base + pl;
        const int n = (int)(flat / g.P);
        const int p = (int)(flat - (long long)n * g.P);
        const A dyv = ld<A>(dy + ((size_t)n * g.C + c) * g.P + p);
        const T* xp = x + ((size_t)n * g.C + c) * g.HW;
        for (int t = 0; t < g.taps; ++t) {
          const Entry& e = table[pl * g.taps + t];
          if (e.src[0] >= 0) {
            A xv;
            if (DEFORM) {
              xv = (A)0;
#pragma unroll
              for (int q = 0; q < (DEFORM ? 4 : 1); ++q) xv += e.sc[q] * ld<A>(xp + e.src[q]);
            } else {
              xv = ld<A>(xp + e.src[0]);
            }
            const A s = xv * dyv;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              A* a = acc + e.idx[q] * 32 + lane;
              *a += e.c[q] * s;
            }
          }
        }
      }
    }
  }
  if (chan_ok) {
    A* out = partial + ((size_t)blockIdx.x * g.C + c) * g.cells;
    for (int cell = 0; cell < g.cells; ++cell) out[cell] = acc[cell * 32 + lane];
  }
}

// Variant for DK + DCN on planes that fit in shared memory: the block keeps the whole input plane of
// its 32 channels on chip ([channel][pixel], pitch chosen so that the 32 lanes of a warp -- one
// channel each -- hit 32 different banks), so the four data-dependent image samples of a tap are
// shared-memory reads instead of 32 scattered global lines per warp load.  Warps split the pixels of
// a batch; each has private accumulators; a block walks several samples and writes one partial.
template <typename T, bool DEFORM>
__global__ void filter_plane_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ off,
                                    const T* __restrict__ rot, typename Compute<T>::type* __restrict__ partial,
                                    const Geom g, const int pitch, const int batch) {
  using A = typename Compute<T>::type;
  using Entry = TapEntry<A, DEFORM>;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int warps = blockDim.x >> 5;
  A* acc_all = reinterpret_cast<A*>(smem_raw);                                      // [warps][cells][32]
  Entry* table = reinterpret_cast<Entry*>(acc_all + (size_t)warps * g.cells * 32);  // [batch][taps]
  T* planes = reinterpret_cast<T*>(table + (size_t)batch * g.taps);                 // [32][pitch]

  const int grp = blockIdx.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int j0 = blockIdx.y * 32;
  const bool chan_ok = j0 + lane < g.Cg;
  const size_t c = (size_t)grp + (size_t)g.G * (chan_ok ? j0 + lane : 0);
  A* acc = acc_all + (size_t)warp * g.cells * 32;
  for (int i = lane; i < g.cells * 32; i += 32) acc[i] = (A)0;
  const T* myplane = planes + (size_t)lane * pitch;

  for (int n = blockIdx.x; n < g.N; n += gridDim.x) {
    __syncthreads();
    for (int ch = warp; ch < 32; ch += warps) {
      if (j0 + ch < g.Cg) {
        const T* sp = x + ((size_t)n * g.C + grp + (size_t)g.G * (j0 + ch)) * g.HW;
        T* dp = planes + (size_t)ch * pitch;
        for (int i = lane; i < g.HW; i += 32) dp[i] = __ldg(sp + i);
      }
    }
    for (int base = 0; base < g.P; base += batch) {
      const int nb = min(batch, g.P - base);
      __syncthreads();
      for (int i = threadIdx.x; i < nb * g.taps; i += blockDim.x) {
        const int pl = i / g.taps, t = i - pl * g.taps;
        const int p = base + pl;
        const int oh = p / g.Wo, ow = p - oh * g.Wo;
        const int fh = t / g.kW, fw = t - fh * g.kW;
        const int ih = oh * g.sH - g.pH + fh * g.dH, iw = ow * g.sW - g.pW + fw * g.dW;
        Entry e;
        e.src[0] = -1;
#pragma unroll
        for (int q = 0; q < 4; ++q) { e.idx[q] = 0; e.c[q] = (A)0; }
        bool used;
        Bilinear<A> bi;
        if (DEFORM) {
          const T* o = off + ((size_t)n * g.taps + t) * 2 * g.P + p;
          used = image_setup<A>((A)ih + ld<A>(o), (A)iw + ld<A>(o + g.P), g, bi);
        } else {
          used = ih >= 0 && ih < g.H && iw >= 0 && iw < g.W;
        }
        if (used) {
          const T* r = rot + ((size_t)(n * g.G + grp) * g.taps + t) * 2 * g.P + p;
          Bilinear<A> b;
          if (bank_setup<A>(ld<A>(r), ld<A>(r + g.P), fh, fw, g, b)) {
            bilinear_value_coefs(b, e.c);
#pragma unroll
            for (int q = 0; q < 4; ++q) e.idx[q] = b.idx[q];
            if (DEFORM) {
              A sc[4];
              bilinear_value_coefs(bi, sc);
#pragma unroll
              for (int q = 0; q < (DEFORM ? 4 : 1); ++q) { e.src[q] = bi.idx[q]; e.sc[q] = sc[q]; }
            } else {
              e.src[0] = ih * g.W + iw;
            }
          }
        }
        table[i] = e;
      }
      __syncthreads();
      if (chan_ok) {
        for (int pl = warp; pl < nb; pl += warps) {
          const A dyv = ld<A>(dy + ((size_t)n * g.C + c) * g.P + base + pl);
          for (int t = 0; t < g.taps; ++t) {
            const Entry& e = table[pl * g.taps + t];
            if (e.src[0] >= 0) {
              A xv;
              if (DEFORM) {
                xv = (A)0;
#pragma unroll
                for (int q = 0; q < (DEFORM ? 4 : 1); ++q) xv += e.sc[q] * static_cast<A>(myplane[e.src[q]]);
              } else {
                xv = static_cast<A>(myplane[e.src[0]]);
              }
              const A sv = xv * dyv;
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                A* a = acc + e.idx[q] * 32 + lane;
                *a += e.c[q] * sv;
              }
            }
          }
        }
      }
    }
  }
  __syncthreads();
  if (chan_ok) {
    A* out = partial + ((size_t)blockIdx.x * g.C + c) * g.cells;
    for (int cell = warp; cell < g.cells; cell += warps) {
      A sum = (A)0;
      for (int wv = 0; wv < warps; ++wv) sum += acc_all[((size_t)wv * g.cells + cell) * 32 + lane];
      out[cell] = sum;
    }
  }
}

struct PlanePlan {
  bool ok;
  int warps, batch, pitch, slots, chan_blocks;
  size_t smem, ws_bytes;
};

template <typename T, bool DEFORM>
static PlanePlan plane_plan(const Geom& g) {
  using A = typename Compute<T>::type;
  PlanePlan pl;
  pl.batch = 16;
  // lanes = channels read element i of 32 planes: the plane pitch in 32-bit words must be odd
  if (sizeof(T) == 2) {
    pl.pitch = (g.HW + 3) & ~3;
    pl.pitch += 2;
  } else {
    pl.pitch = g.HW | 1;
  }
  for (pl.warps = 16; pl.warps >= 4; pl.warps >>= 1) {
    pl.smem = (size_t)pl.warps * g.cells * 32 * sizeof(A) + (size_t)pl.batch * g.taps * sizeof(TapEntry<A, DEFORM>) +
              (size_t)32 * pl.pitch * sizeof(T);
    if (pl.smem <= 226 * 1024 || pl.warps == 4) break;
  }
  pl.chan_blocks = (g.Cg + 31) / 32;
  const long long chan_ctas = (long long)pl.chan_blocks * g.G;
  long long slots = (2LL * 148 + chan_ctas - 1) / chan_ctas;
  if (slots > g.N) slots = g.N;
  if (slots < 1) slots = 1;
  pl.slots = (int)slots;
  pl.ws_bytes = (size_t)pl.slots * g.C * g.cells * sizeof(A);
  pl.ok = pl.smem <= 226 * 1024 && pl.chan_blocks <= 65535 && g.G <= 65535 && g.Cg >= 32;
  return pl;
}

size_t deform_filter_plane_workspace(const Geom& g, int dtype) {
  PlanePlan pl;
  if (dtype == DK_F16) pl = plane_plan<__half, true>(g);
  else if (dtype == DK_F64) pl = plane_plan<double, true>(g);
  else pl = plane_plan<float, true>(g);
  return pl.ok ? pl.ws_bytes : 0;
}

// out[i] = sum over partial blocks, fixed order.  A block of 256 threads takes 32 outputs: thread (x, y) sums the partials
// y, y + 8, ... of output x (coalesced over x), the eight sums of an output meet in shared memory.
template <typename T>
__global__ void reduce_partials_kernel(const typename Compute<T>::type* __restrict__ partial, T* __restrict__ out,
                                       const int n_out, const int n_part) {
  using A = typename Compute<T>::type;
  __shared__ A part[8][33];
  const int x = threadIdx.x & 31, y = threadIdx.x >> 5;
  const int i = blockIdx.x * 32 + x;
  A s = (A)0;
  if (i < n_out)
    for (int k = y; k < n_part; k += 8) s += partial[(size_t)k * n_out + i];
  part[y][x] = s;
  __syncthreads();
  if (y == 0 && i < n_out) {
    A t = part[0][x];
#pragma unroll
    for (int j = 1; j < 8; ++j) t += part[j][x];
    st<T, A>(out + i, t);
  }
}

FilterPlan filter_plan(const Geom& g, size_t acc_bytes) {
  FilterPlan pl;
  int warps = (g.Cg + 31) / 32;
  if (warps > 8) warps = 8;
  // accumulators [warps][cells][32] must fit beside the basis table
  while (warps > 1 && (size_t)warps * g.cells * 32 * acc_bytes > 96 * 1024) warps >>= 1;
  pl.warps = warps;
  pl.chan_blocks = (g.Cg + 32 * warps - 1) / (32 * warps);
  const long long total = (long long)g.N * g.P;
  const long long chan_ctas = (long long)pl.chan_blocks * g.G;
  long long want = (4LL * 148 + chan_ctas - 1) / chan_ctas;  // ~4 blocks per SM over the grid
  const long long max_by_work = (total + 3) / 4;  // at least four pixels per block, so that small problems still spread out
  if (want > max_by_work) want = max_by_work;
  if (want > 2048) want = 2048;
  if (want < 1) want = 1;
  pl.pix_per_block = (total + want - 1) / want;
  pl.pix_blocks = (int)((total + pl.pix_per_block - 1) / pl.pix_per_block);
  pl.ws_bytes = (size_t)pl.pix_blocks * g.C * g.cells * acc_bytes;
  return pl;
}

// The same plan with fewer, larger pixel blocks where its partial sums would not fit into max_bytes (pix_blocks = 0
// when not even one block's partial sums fit).
FilterPlan filter_plan_fit(const Geom& g, size_t acc_bytes, size_t max_bytes) {
  FilterPlan pl = filter_plan(g, acc_bytes);
  if (pl.ws_bytes <= max_bytes) return pl;
  const size_t per_block = (size_t)g.C * g.cells * acc_bytes;
  const long long fit = (long long)(max_bytes / per_block);
  if (fit < 1) {
    pl.pix_blocks = 0;
    pl.ws_bytes = 0;
    return pl;
  }
  const long long total = (long long)g.N * g.P;
  pl.pix_per_block = (total + fit - 1) / fit;
  pl.pix_blocks = (int)((total + pl.pix_per_block - 1) / pl.pix_per_block);
  pl.ws_bytes = (size_t)pl.pix_blocks * per_block;
  return pl;
}

template <typename T, bool DEFORM>
static int filter_backward(const T* dy, const T* x, const T* off, const T* rot, T* dw, const Geom& g, void* ws,
                           size_t ws_bytes, cudaStream_t s, bool fit = false) {
  using A = typename Compute<T>::type;
  if (DEFORM) {
    const PlanePlan pp = plane_plan<T, DEFORM>(g);
    if (pp.ok && pp.smem <= (size_t)device_smem_optin()) {
      if (ws == nullptr || ws_bytes < pp.ws_bytes) return DK_ERR_WORKSPACE;
      auto kern = filter_plane_kernel<T, DEFORM>;
      int rc = enable_smem(kern, pp.smem);
      if (rc) return rc;
      kern<<<dim3(pp.slots, pp.chan_blocks, g.G), pp.warps * 32, pp.smem, s>>>(dy, x, off, rot, reinterpret_cast<A*>(ws), g,
                                                                            pp.pitch, pp.batch);
      rc = check_launch();
      if (rc) return rc;
      const int n_out = g.C * g.cells;
      reduce_partials_kernel<T><<<(n_out + 31) / 32, 256, 0, s>>>(reinterpret_cast<const A*>(ws), dw, n_out, pp.slots);
      return check_launch();
    }
  }
  const FilterPlan pl = fit ? filter_plan_fit(g, sizeof(A), ws_bytes) : filter_plan(g, sizeof(A));
  if (ws == nullptr || ws_bytes < pl.ws_bytes || pl.pix_blocks < 1) return DK_ERR_WORKSPACE;
  if (pl.chan_blocks > 65535 || g.G > 65535) return DK_ERR_UNSUPPORTED;
  const size_t smem =
      (size_t)pl.warps * g.cells * 32 * sizeof(A) + (size_t)kFilterPixBatch * g.taps * sizeof(TapEntry<A, DEFORM>);
  if (smem > (size_t)device_smem_optin()) return DK_ERR_UNSUPPORTED;
  auto kern = filter_kernel<T, DEFORM>;
  int rc = enable_smem(kern, smem);
  if (rc) return rc;
  kern<<<dim3(pl.pix_blocks, pl.chan_blocks, g.G), pl.warps * 32, smem, s>>>(dy, x, off, rot, reinterpret_cast<A*>(ws),
                                                                            g, pl.pix_per_block, pl.warps);
  rc = check_launch();
  if (rc) return rc;
  const int n_out = g.C * g.cells;
  reduce_partials_kernel<T><<<(n_out + 31) / 32, 256, 0, s>>>(reinterpret_cast<const A*>(ws), dw, n_out, pl.pix_blocks);
  return check_launch();
}

template <typename T>
int local_backward_filter(const T* dy, const T* x, const T* rot, T* dw, const Geom& g, void* ws, size_t ws_bytes,
                          cudaStream_t s) {
  if constexpr (std::is_same<T, __half>::value) {
    if (mma_path_enabled()) {
      const int rc = local_filter_mma(dy, x, rot, dw, g, ws, ws_bytes, s);
      if (rc != DK_ERR_UNSUPPORTED) return rc;
    }
  }
  return filter_backward<T, false>(dy, x, nullptr, rot, dw, g, ws, ws_bytes, s);
}
// The same for a caller whose workspace has a fixed size: the tensor-core kernel when its own partial sums fit, else the
// general kernel with as many pixel blocks as fit.  need_out (optional) receives the bytes the call uses.
template <typename T>
int local_backward_filter_fit(const T* dy, const T* x, const T* rot, T* dw, const Geom& g, void* ws, size_t ws_bytes,
                              cudaStream_t s, bool launch, size_t* need_out) {
  if constexpr (std::is_same<T, __half>::value) {
    if (mma_path_enabled()) {
      const size_t fast = local_filter_mma_workspace(g);
      if (fast > 0 && fast <= ws_bytes) {
        if (need_out) *need_out = fast;
        if (!launch) return DK_OK;
        const int rc = local_filter_mma(dy, x, rot, dw, g, ws, ws_bytes, s);
        if (rc != DK_ERR_UNSUPPORTED) return rc;
      }
    }
  }
  using A = typename Compute<T>::type;
  const FilterPlan pl = filter_plan_fit(g, sizeof(A), ws_bytes);
  if (pl.pix_blocks < 1) return DK_ERR_WORKSPACE;
  if (need_out) *need_out = pl.ws_bytes;
  if (!launch) return DK_OK;
  return filter_backward<T, false>(dy, x, nullptr, rot, dw, g, ws, ws_bytes, s, true);
}
template <typename T>
int deform_backward_filter(const T* dy, const T* x, const T* off, const T* rot, T* dw, const Geom& g, void* ws,
                           size_t ws_bytes, cudaStream_t s) {
  if constexpr (std::is_same<T, __half>::value) {
    if (mma_path_enabled()) {
      const int rc = deform_filter_mma(dy, x, off, rot, dw, g, ws, ws_bytes, s);
      if (rc != DK_ERR_UNSUPPORTED) return rc;
    }
  }
  return filter_backward<T, true>(dy, x, off, rot, dw, g, ws, ws_bytes, s);
}

#define DK_INSTANTIATE_LOCAL(T)                                                                                  \
  template int local_forward<T>(const T*, const T*, const T*, T*, const Geom&, cudaStream_t);                     \
  template int local_backward_data<T>(const T*, const T*, const T*, T*, const Geom&, cudaStream_t);               \
  template int local_backward_rotation<T>(const T*, const T*, const T*, const T*, T*, const Geom&, void*, size_t, \
                                          cudaStream_t);                                                           \
  template int local_backward_filter<T>(const T*, const T*, const T*, T*, const Geom&, void*, size_t, cudaStream_t); \
  template int local_backward_filter_fit<T>(const T*, const T*, const T*, T*, const Geom&, void*, size_t, cudaStream_t, bool,  \
                                            size_t*);                                                                          \
  template int deform_backward_filter<T>(const T*, const T*, const T*, const T*, T*, const Geom&, void*, size_t,      \
                                         cudaStream_t);
DK_INSTANTIATE_LOCAL(float)
DK_INSTANTIATE_LOCAL(__half)
DK_INSTANTIATE_LOCAL(double)

}  // namespace dk
