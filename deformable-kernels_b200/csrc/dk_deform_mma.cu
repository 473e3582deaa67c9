// fp16 tensor-core paths of the DK + DCN operator: forward, bank gradient, gradients of both offset fields, and
// grad-input.
//
// y[c, p]      = sum over taps of K[c, p, tap] * xs[c, p, tap],          K = W * beta^T
// dW[c, cell]  = sum over (sample, pixel, tap) of dy[c, p] * xs[c, p, tap] * beta[(p, tap), cell]
// where beta are the hat products of the bank coordinate (see dk_local_mma.cu) and xs is the bilinear image
// sample at the tap's deformed position: four data-dependent reads per (pixel, tap, channel).  A block keeps the
// WHOLE input plane of its channels in shared memory, so those reads never leave the SM, and builds, three taps
// at a time, a table of (byte offset, coefficient) x 4 corners per (pixel, tap) that all its channels reuse.
// The products with beta are mma.sync.m16n8k16 as for the local operator.  The offset gradients and grad-input
// (a scatter into on-chip planes) are described at their kernels further down.
//
// Covers fp16, 3x3, pad 1, dilation 1, stride 1 or 2, one rotation group, <= 16 bank cells, C % 16 == 0 and
// planes small enough for 16 of them to fit on chip (56 x 56 and below); other shapes use the SIMT kernels.
#include <cstdlib>

#include "dk_mma_common.cuh"

namespace dk {

using namespace mma;

namespace {

constexpr size_t kOnePerSm = 226 * 1024;

// ------------------------------------------------------------------ channel-pair planes
// The kernels that sample the image keep its planes as 32-bit words (channel j | channel j + 8 << 16), eight words per pixel
// ("chunk"), so that one shared-memory read serves both channel rows of a lane's mma fragments and the eight
// lanes of a pixel read 32 contiguous bytes.  Chunks are permuted inside groups of 8 (stride 1) or 16 (stride 2)
// pixels so that the four pixel pairs of a warp, 2 (or 4) source pixels apart when the offsets are smooth, start
// in four different bank groups.
template <int S>
__device__ __forceinline__ int chunk_of(int i) {
  if (S == 1) return (i & ~7) | ((i >> 1) & 3) | ((i & 1) << 2);
  return (i & ~15) | ((i >> 2) & 3) | ((i & 3) << 2);
}

template <int S>
__device__ __forceinline__ void load_pair_planes(unsigned* __restrict__ xw, const __half* __restrict__ x, int n, int C, int c0,
                                                 int HW, bool vec) {
  const __half* s0 = x + ((size_t)n * C + c0) * HW;
  if (vec) {
    const int tasks = HW;  // (HW / 8 groups of 8 pixels) x 8 channel pairs
#pragma unroll 2
    for (int task = threadIdx.x; task < tasks; task += blockDim.x) {
      const int j = task & 7, grp = task >> 3;
      const uint4 a = __ldg(reinterpret_cast<const uint4*>(s0 + (size_t)j * HW) + grp);
      const uint4 b = __ldg(reinterpret_cast<const uint4*>(s0 + (size_t)(j + 8) * HW) + grp);
      const unsigned aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int k2 = 0; k2 < 4; ++k2) {
        const int i = grp * 8 + 2 * k2;
        xw[chunk_of<S>(i) * 8 + j] = __byte_perm(aw[k2], bw[k2], 0x5410);
        xw[chunk_of<S>(i + 1) * 8 + j] = __byte_perm(aw[k2], bw[k2], 0x7632);
      }
    }
  } else {
    const int tasks = HW * 8;
    for (int task = threadIdx.x; task < tasks; task += blockDim.x) {
      const int j = task & 7, i = task >> 3;
      const unsigned lo = __half_as_ushort(__ldg(s0 + (size_t)j * HW + i));
      const unsigned hi = __half_as_ushort(__ldg(s0 + (size_t)(j + 8) * HW + i));
      xw[chunk_of<S>(i) * 8 + j] = lo | (hi << 16);
    }
  }
}

constexpr int kPairTabWords = 3 * 80;  // per warp: 3 taps x 4 pixel pairs x (2 x 8 words + 4 of padding)

// Sampling table of the three taps of kernel row fh for the 8 pixels of an item: per (pixel, tap) the byte
// offsets of the four corner chunks and the four corner coefficients, each duplicated into both halves of a
// word.  A tap whose deformed position is outside (-1, H) x (-1, W) gets zero coefficients.  Lanes 0..23.
// With ACC_PLANE the entries address the accumulator planes of the grad-input kernel instead (the shared-memory
// address of the pixel's first group of eight channels, see acc_word) and the coefficients are fp32.
template <int S>
__device__ __forceinline__ unsigned acc_word(int i, int ch) {  // word of (pixel i, channel ch) in the fp32 planes
  const int row = i >> 1, r = (S == 1 ? row : row >> 1) & 3;
  return (unsigned)(row * 32 + (((((ch >> 3) << 1) | (i & 1)) ^ r) << 3) + (ch & 7));
}
template <int S, bool ACC_PLANE>
__device__ __forceinline__ void pair_table_entry(unsigned* __restrict__ tab, const Geom& g, int fh, int oh, int ow0, int lane,
                                                 float o_h, float o_w, unsigned acc_saddr) {
  const int px = lane & 7, fw = lane >> 3;
  const int pc = ow0 + px;
  const float ph = (float)(oh * S - 1 + fh) + o_h;
  const float pw = (float)(pc * S - 1 + fw) + o_w;
  const bool used = pc < g.Wo && ph > -1.f && pw > -1.f && ph < (float)g.H && pw < (float)g.W;
  uint4 o4 = make_uint4(0, 0, 0, 0), c4 = make_uint4(0, 0, 0, 0);
  if (ACC_PLANE) {  // an unused tap adds zeros at its undeformed position (distinct addresses per lane)
    const int hn = min(max(oh * S - 1 + fh, 0), g.H - 1), wn = min(max(pc * S - 1 + fw, 0), g.W - 1);
    const unsigned a = acc_saddr + acc_word<S>(hn * g.W + wn, 0) * 4u;
    o4 = make_uint4(a, a, a, a);
  }
  if (used) {
    const float fph = floorf(ph), fpw = floorf(pw);
    const int h0 = (int)fph, w0 = (int)fpw;
    const float lh = ph - fph, lw = pw - fpw;
    const float hh = 1.f - lh, hw = 1.f - lw;
    const bool r0 = h0 >= 0, r1 = h0 + 1 <= g.H - 1, k0 = w0 >= 0, k1 = w0 + 1 <= g.W - 1;
    const int h0c = max(h0, 0), h1c = min(h0 + 1, g.H - 1), w0c = max(w0, 0), w1c = min(w0 + 1, g.W - 1);
    auto where = [&](int hh_, int ww_) {
      const int i = hh_ * g.W + ww_;
      return ACC_PLANE ? acc_saddr + acc_word<S>(i, 0) * 4u : (unsigned)chunk_of<S>(i) * 32u;
    };
    auto coef = [&](bool ok, float v) { return !ok ? 0u : (ACC_PLANE ? __float_as_uint(v) : pack2(v, v)); };
    o4.x = where(h0c, w0c);
    o4.y = where(h0c, w1c);
    o4.z = where(h1c, w0c);
    o4.w = where(h1c, w1c);
    c4.x = coef(r0 && k0, hh * hw);
    c4.y = coef(r0 && k1, hh * lw);
    c4.z = coef(r1 && k0, lh * hw);
    c4.w = coef(r1 && k1, lh * lw);
  }
  uint4* e = reinterpret_cast<uint4*>(tab + fw * 80 + (px >> 1) * 20 + (px & 1) * 8);
  e[0] = o4;
  e[1] = c4;
}
template <int S>
__device__ __forceinline__ void build_pair_table(unsigned* __restrict__ tab, const __half* __restrict__ oband, const Band& bo,
                                                 const Geom& g, int fh, int oh, int ow0, int lane) {
  if (lane < 24) {
    const int t = fh * 3 + (lane >> 3);
    const __half* op = oband + (size_t)(2 * t) * bo.pitch_c + kSlack + oh * bo.Wp + ow0 + (lane & 7) - bo.org;
    pair_table_entry<S, false>(tab, g, fh, oh, ow0, lane, __half2float(op[0]), __half2float(op[bo.pitch_c]), 0u);
  }
}

__device__ __forceinline__ unsigned hfma2u(unsigned a, unsigned b, unsigned c) {
  const __half2 r = __hfma2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b),
                            *reinterpret_cast<const __half2*>(&c));
  return *reinterpret_cast<const unsigned*>(&r);
}
// (sample of channel j, sample of channel j + 8) of one (pixel, tap): base points at the lane's word of chunk 0
__device__ __forceinline__ unsigned sample_pair(const char* __restrict__ base, const uint4 o, const uint4 cf) {
  unsigned r = hmul2u(*reinterpret_cast<const unsigned*>(base + o.x), cf.x);
  r = hfma2u(*reinterpret_cast<const unsigned*>(base + o.y), cf.y, r);
  r = hfma2u(*reinterpret_cast<const unsigned*>(base + o.z), cf.z, r);
  r = hfma2u(*reinterpret_cast<const unsigned*>(base + o.w), cf.w, r);
  return r;
}

// hat-product fragments (as beta_direct without the image mask) from offsets held in registers; with all-zero
// offsets (rot == nullptr in the kernels below: the kernel is the same for every pixel) they are built once per warp
__device__ __forceinline__ void beta_from_regs(unsigned (&bf)[9][2], const unsigned (&rp)[9], const Geom& g, const LaneCells& lc,
                                               bool sc44, bool valid) {
  const float uh0 = (float)(g.scH - 3) * 0.5f, uw0 = (float)(g.scW - 3) * 0.5f;
#pragma unroll
  for (int fh = 0; fh < 3; ++fh) {
#pragma unroll
    for (int fw = 0; fw < 3; ++fw) {
      const int t = fh * 3 + fw;
      const float u = ((float)fh + lo2f(rp[t])) + uh0;
      const float v = valid ? ((float)fw + hi2f(rp[t])) + uw0 : 1e30f;
      if (sc44) {
        const float hh0 = hat(u - lc.ca[0]), hh1 = hat(u - lc.ca[2]);
        const float hw0 = hat(v - lc.cb[0]), hw1 = hat(v - lc.cb[1]);
        bf[t][0] = pack2(hh0 * hw0, hh0 * hw1);
        bf[t][1] = pack2(hh1 * hw0, hh1 * hw1);
      } else {
        float b4[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) b4[k] = lc.ok[k] ? hat(u - lc.ca[k]) * hat(v - lc.cb[k]) : 0.f;
        bf[t][0] = pack2(b4[0], b4[1]);
        bf[t][1] = pack2(b4[2], b4[3]);
      }
    }
  }
}

struct DcnPlan {
  int NS, BH, warps, bands, units_per_block, blocks_x;
  int mode_rot, mode_off, mode_dy;
  bool vec;
  size_t smem, ws_bytes;
};

// y[c, p] = sum over taps of K[c, p, tap] * xs[c, p, tap]:  K = W * beta^T from one mma per tap (as in the local
// forward), xs sampled from the channel-pair planes.  A block owns 16 * NS channels and walks over units
// (sample, band of output rows); the planes are reloaded only when the sample changes.
template <int S, int NS, bool ZR>
__global__ void __launch_bounds__(512, 1) mma_deform_fwd_kernel(const __half* __restrict__ x, const __half* __restrict__ off,
                                                               const __half* __restrict__ rot, const __half* __restrict__ w,
                                                               __half* __restrict__ y, const Geom g, const DcnPlan pl) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int c0 = blockIdx.y * (16 * NS);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int gq = lane >> 2, q = lane & 3;
  const int NB = (g.Wo + 7) >> 3;
  const int items = pl.BH * NB;
  const int Wpo = g.Wo + (g.Wo & 1);
  const int HW16 = (g.HW + 15) & ~15;
  const int ypitch = band_pitch(pl.BH, Wpo);

  unsigned* xw = reinterpret_cast<unsigned*>(smem_raw);                      // [NS][HW16 * 8]
  __half* rband = reinterpret_cast<__half*>(xw + (size_t)NS * HW16 * 8);     // [18][ypitch]
  __half* oband = rband + (size_t)18 * ypitch;                               // [18][ypitch]
  unsigned* tab = reinterpret_cast<unsigned*>(oband + (size_t)18 * ypitch) + warp * kPairTabWords;
  const LaneCells lc = lane_cells(g, q);
  const bool sc44 = g.scH == 4 && g.scW == 4;

  // A fragments of the bank slabs: rows = channels (gq, gq + 8), k = cells (2q, 2q+1) and (2q+8, 2q+9)
  unsigned wa[NS][4];
#pragma unroll
  for (int sidx = 0; sidx < NS; ++sidx) {
    const __half* w0 = w + (size_t)(c0 + 16 * sidx + gq) * g.cells;
    const __half* w1 = w0 + (size_t)8 * g.cells;
    auto cell2 = [&](const __half* p, int k) {
      const unsigned lo = k < g.cells ? (unsigned)__half_as_ushort(__ldg(p + k)) : 0u;
      const unsigned hi = k + 1 < g.cells ? (unsigned)__half_as_ushort(__ldg(p + k + 1)) : 0u;
      return lo | (hi << 16);
    };
    wa[sidx][0] = cell2(w0, 2 * q);
    wa[sidx][1] = cell2(w1, 2 * q);
    wa[sidx][2] = cell2(w0, 2 * q + 8);
    wa[sidx][3] = cell2(w1, 2 * q + 8);
  }

  const int total_units = g.N * pl.bands;
  const int u_begin = blockIdx.x * pl.units_per_block;
  const int u_end = min(u_begin + pl.units_per_block, total_units);
  const bool even_w = (g.Wo & 1) == 0;
  constexpr bool zero_rot = ZR;  // rot == nullptr
  unsigned bf[9][2];
  if (zero_rot) {
    const unsigned z[9] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
    beta_from_regs(bf, z, g, lc, sc44, true);
  }
  int cur_n = -1;
  for (int unit = u_begin; unit < u_end; ++unit) {
    const int n = unit / pl.bands;
    const int oh0 = (unit - n * pl.bands) * pl.BH;
    const Band br = make_band(oh0, pl.BH, g.Ho, g.Wo, pl.mode_rot);
    const Band bo = make_band(oh0, pl.BH, g.Ho, g.Wo, pl.mode_off);
    __syncthreads();  // readers of the previous unit are done
    if (!zero_rot) load_band(rband, br, rot, n, 18, 0, 18, g.Ho, g.Wo);
    load_band(oband, bo, off, n, 18, 0, 18, g.Ho, g.Wo);
    if (n != cur_n) {
#pragma unroll
      for (int sidx = 0; sidx < NS; ++sidx) load_pair_planes<S>(xw + (size_t)sidx * HW16 * 8, x, n, g.C, c0 + 16 * sidx, g.HW, pl.vec);
      cur_n = n;
    }
    cp_async_wait_all();
    __syncthreads();

    for (int item = warp; item < items; item += nwarps) {
      const int dr = item / NB;
      const int oh = oh0 + dr;
      if (oh >= g.Ho) break;
      const int ow0 = (item - dr * NB) << 3;
      if (!zero_rot) beta_direct<S, false, false>(bf, rband, br, g, lc, sc44, oh, ow0, g.H, g.W, g.Wo, gq);
      float acc[NS][4];
#pragma unroll
      for (int sidx = 0; sidx < NS; ++sidx) acc[sidx][0] = acc[sidx][1] = acc[sidx][2] = acc[sidx][3] = 0.f;
      const char* lane_base = reinterpret_cast<const char*>(xw) + gq * 4;
#pragma unroll
      for (int fh = 0; fh < 3; ++fh) {
        __syncwarp();
        build_pair_table<S>(tab, oband, bo, g, fh, oh, ow0, lane);
        __syncwarp();
#pragma unroll
        for (int fw = 0; fw < 3; ++fw) {
          const int t = fh * 3 + fw;
          const uint4* e0 = reinterpret_cast<const uint4*>(tab + fw * 80 + q * 20);
          const uint4 oA = e0[0], cA = e0[1], oB = e0[2], cB = e0[3];  // pixel 2q, pixel 2q + 1
#pragma unroll
          for (int sidx = 0; sidx < NS; ++sidx) {
            unsigned kk[2];  // K of (channel gq | gq + 8) x (pixel 2q, 2q + 1)
            mma16816_h(kk, wa[sidx], bf[t][0], bf[t][1]);
            const char* base = lane_base + (size_t)sidx * HW16 * 32;
            const unsigned r0 = sample_pair(base, oA, cA), r1 = sample_pair(base, oB, cB);
            fma_hh<0, 0>(acc[sidx][0], kk[0], r0);
            fma_hh<1, 0>(acc[sidx][1], kk[0], r1);
            fma_hh<0, 1>(acc[sidx][2], kk[1], r0);
            fma_hh<1, 1>(acc[sidx][3], kk[1], r1);
          }
        }
      }
      const int ow = ow0 + 2 * q;
      if (ow < g.Wo) {
#pragma unroll
        for (int sidx = 0; sidx < NS; ++sidx) {
          __half* y0 = y + ((size_t)n * g.C + c0 + 16 * sidx + gq) * g.P + (size_t)oh * g.Wo + ow;
          __half* y1 = y0 + (size_t)8 * g.P;
          if (even_w) {
            *reinterpret_cast<unsigned*>(y0) = pack2(acc[sidx][0], acc[sidx][1]);
            *reinterpret_cast<unsigned*>(y1) = pack2(acc[sidx][2], acc[sidx][3]);
          } else {
            y0[0] = __float2half_rn(acc[sidx][0]);
            y1[0] = __float2half_rn(acc[sidx][2]);
            if (ow + 1 < g.Wo) {
              y0[1] = __float2half_rn(acc[sidx][1]);
              y1[1] = __float2half_rn(acc[sidx][3]);
            }
          }
        }
      }
    }
  }
}

// Bank gradient.  dK = dy * xs is the A operand (rows = channels, k = 8 pixels x 2 taps), beta the B operand;
// the accumulators live in registers over all units of the block, are reduced across its warps at the end and
// written as one partial [16 * NS channels][16 cells] per block.
template <int S, int NS, bool ZR>
__global__ void __launch_bounds__(512, 1) mma_deform_filter_kernel(const __half* __restrict__ dy, const __half* __restrict__ x,
                                                                  const __half* __restrict__ off, const __half* __restrict__ rot,
                                                                  float* __restrict__ partial, const Geom g, const DcnPlan pl) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int CG = 16 * NS;
  const int c0 = blockIdx.y * CG;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int gq = lane >> 2, q = lane & 3;
  const int NB = (g.Wo + 7) >> 3;
  const int items = pl.BH * NB;
  const int Wpo = g.Wo + (g.Wo & 1);
  const int HW16 = (g.HW + 15) & ~15;
  const int ypitch = band_pitch(pl.BH, Wpo);

  unsigned* xw = reinterpret_cast<unsigned*>(smem_raw);                      // [NS][HW16 * 8]
  __half* yband = reinterpret_cast<__half*>(xw + (size_t)NS * HW16 * 8);     // [CG][ypitch]
  __half* rband = yband + (size_t)CG * ypitch;                               // [18][ypitch]
  __half* oband = rband + (size_t)18 * ypitch;                               // [18][ypitch]
  unsigned* tab = reinterpret_cast<unsigned*>(oband + (size_t)18 * ypitch) + warp * kPairTabWords;
  const LaneCells lc = lane_cells(g, q);
  const bool sc44 = g.scH == 4 && g.scW == 4;

  float acc[NS][2][4];
#pragma unroll
  for (int sidx = 0; sidx < NS; ++sidx)
#pragma unroll
    for (int k = 0; k < 4; ++k) acc[sidx][0][k] = acc[sidx][1][k] = 0.f;

  constexpr bool zero_rot = ZR;  // rot == nullptr
  unsigned bw[9][2];  // beta as B fragments: [tap][cells 0-7 | cells 8-15]
  if (zero_rot) {
    const unsigned z[9] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
    unsigned bf[9][2];
    beta_from_regs(bf, z, g, lc, sc44, true);
#pragma unroll
    for (int t = 0; t < 9; ++t) {
      bw[t][0] = movmatrix_trans(bf[t][0]);
      bw[t][1] = movmatrix_trans(bf[t][1]);
    }
  }

  const int total_units = g.N * pl.bands;
  const int u_begin = blockIdx.x * pl.units_per_block;
  const int u_end = min(u_begin + pl.units_per_block, total_units);
  int cur_n = -1;
  for (int unit = u_begin; unit < u_end; ++unit) {
    const int n = unit / pl.bands;
    const int oh0 = (unit - n * pl.bands) * pl.BH;
    const Band by = make_band(oh0, pl.BH, g.Ho, g.Wo, pl.mode_dy);
    const Band br = make_band(oh0, pl.BH, g.Ho, g.Wo, pl.mode_rot);
    const Band bo = make_band(oh0, pl.BH, g.Ho, g.Wo, pl.mode_off);
    __syncthreads();  // readers of the previous unit are done
    load_band(yband, by, dy, n, g.C, c0, CG, g.Ho, g.Wo);
    if (!zero_rot) load_band(rband, br, rot, n, 18, 0, 18, g.Ho, g.Wo);
    load_band(oband, bo, off, n, 18, 0, 18, g.Ho, g.Wo);
    if (n != cur_n) {
#pragma unroll
      for (int sidx = 0; sidx < NS; ++sidx) load_pair_planes<S>(xw + (size_t)sidx * HW16 * 8, x, n, g.C, c0 + 16 * sidx, g.HW, pl.vec);
      cur_n = n;
    }
    cp_async_wait_all();
    __syncthreads();

    for (int item = warp; item < items; item += nwarps) {
      const int dr = item / NB;
      const int oh = oh0 + dr;
      if (oh >= g.Ho) break;
      const int ow0 = (item - dr * NB) << 3;
      if (!zero_rot) {
        unsigned bf[9][2];
        beta_direct<S, false, false>(bf, rband, br, g, lc, sc44, oh, ow0, g.H, g.W, g.Wo, gq);
#pragma unroll
        for (int t = 0; t < 9; ++t) {
          bw[t][0] = movmatrix_trans(bf[t][0]);
          bw[t][1] = movmatrix_trans(bf[t][1]);
        }
      }
      const int yoff = kSlack + oh * by.Wp + ow0 + 2 * q - by.org;
      unsigned dy0[NS], dy1[NS];
#pragma unroll
      for (int sidx = 0; sidx < NS; ++sidx) {
        dy0[sidx] = *reinterpret_cast<const unsigned*>(yband + (size_t)(16 * sidx + gq) * by.pitch_c + yoff);
        dy1[sidx] = *reinterpret_cast<const unsigned*>(yband + (size_t)(16 * sidx + gq + 8) * by.pitch_c + yoff);
      }
      const char* lane_base = reinterpret_cast<const char*>(xw) + gq * 4;
      unsigned pa[NS], pb[NS];  // dK of the even tap of the current pair, kept until its odd partner is sampled
#pragma unroll
      for (int fh = 0; fh < 3; ++fh) {
        __syncwarp();
        build_pair_table<S>(tab, oband, bo, g, fh, oh, ow0, lane);
        __syncwarp();
#pragma unroll
        for (int fw = 0; fw < 3; ++fw) {
          const int t = fh * 3 + fw;
          const uint4* e0 = reinterpret_cast<const uint4*>(tab + fw * 80 + q * 20);
          const uint4 oA = e0[0], cA = e0[1], oB = e0[2], cB = e0[3];  // pixel 2q, pixel 2q + 1
#pragma unroll
          for (int sidx = 0; sidx < NS; ++sidx) {
            const char* base = lane_base + (size_t)sidx * HW16 * 32;
            const unsigned r0 = sample_pair(base, oA, cA), r1 = sample_pair(base, oB, cB);
            const unsigned ka = hmul2u(dy0[sidx], __byte_perm(r0, r1, 0x5410));  // channel gq: pixels 2q, 2q + 1
            const unsigned kb = hmul2u(dy1[sidx], __byte_perm(r0, r1, 0x7632));  // channel gq + 8
            if ((t & 1) == 0 && t < 8) {
              pa[sidx] = ka;
              pb[sidx] = kb;
            } else if (t & 1) {  // k = 16 = 8 pixels x taps (t - 1, t)
              mma16816_acc(acc[sidx][0], pa[sidx], pb[sidx], ka, kb, bw[t - 1][0], bw[t][0]);
              mma16816_acc(acc[sidx][1], pa[sidx], pb[sidx], ka, kb, bw[t - 1][1], bw[t][1]);
            } else {  // the ninth tap, paired with zeros
              mma16816_acc(acc[sidx][0], ka, kb, 0u, 0u, bw[8][0], 0u);
              mma16816_acc(acc[sidx][1], ka, kb, 0u, 0u, bw[8][1], 0u);
            }
          }
        }
      }
    }
  }
  // reduce the warps' accumulators and write this block's partial bank gradient [CG channels][16 cells]
  __syncthreads();
  float* red = reinterpret_cast<float*>(smem_raw);  // [nwarps][CG][16]
#pragma unroll
  for (int sidx = 0; sidx < NS; ++sidx) {
    float* r0 = red + ((size_t)warp * CG + 16 * sidx + gq) * 16;
    float* r1 = r0 + 8 * 16;
    r0[2 * q] = acc[sidx][0][0]; r0[2 * q + 1] = acc[sidx][0][1];
    r1[2 * q] = acc[sidx][0][2]; r1[2 * q + 1] = acc[sidx][0][3];
    r0[8 + 2 * q] = acc[sidx][1][0]; r0[8 + 2 * q + 1] = acc[sidx][1][1];
    r1[8 + 2 * q] = acc[sidx][1][2]; r1[8 + 2 * q + 1] = acc[sidx][1][3];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < CG * 16; i += blockDim.x) {
    float sum = 0.f;
    for (int wv = 0; wv < nwarps; ++wv) sum += red[(size_t)wv * CG * 16 + i];
    partial[((size_t)blockIdx.x * g.C + c0) * 16 + i] = sum;
  }
}

// ------------------------------------------------------------------ grad-input
// dx[c, corner] += coefficient * K[c, p, tap] * dy[c, p]: a data-dependent scatter.  The block keeps the gradient
// planes of its 16 channels in shared memory, processes whole samples and writes each plane once.
//
// Accumulation is in 32-bit FIXED POINT with native integer atomics: on this GPU a shared-memory float add is a
// compare-and-swap loop (measured 5-10 updates per clock per SM, and two lanes of a warp on one address make the
// loser retry), an integer add is one instruction (27 per clock per SM) and indifferent to collisions.  Per sample
// and channel the scale is the power of two that maps B = max|dy| * max|W| (no single contribution can exceed it:
// |K| <= max|W| because the hat weights are non-negative and sum to at most 1, and a tap's four corner coefficients
// sum to at most 1) to 2^(30 - ceil(log2(M))), where M is the largest number of (pixel, tap) samples that touch one
// input pixel of this sample, counted beforehand by dcn_hit_count_kernel from the offsets alone: the accumulator
// cannot overflow whatever the offsets are.  With M of a few dozen a contribution is resolved to 2^-23 B or better,
// the level of an fp32 sum of values up to B; the sum itself is exact and order-independent, so the gradient is
// bit-reproducible from run to run.
//
// Layout: a row of 32 words per pixel pair = four groups of eight channels (channel half x pixel parity), the
// group index XOR-ed with the low bits of the row (acc_word): a lane quartet's four pixels, 2 (or 4) source pixels
// apart when the offsets are smooth, then fall into four different bank groups.
// Offsets are read straight from global memory one item ahead of their use, so the warps never wait on each
// other between the zeroing and the write-out of a sample.
struct DDataPlan {
  int warps, samples_per_block, blocks_x;
  bool pair_dy;
  size_t smem;
};

// hits[n] = max over input pixels of the number of (output pixel, tap) samples of sample n with a corner on it
template <int S>
__global__ void __launch_bounds__(1024) dcn_hit_count_kernel(const __half* __restrict__ off, int* __restrict__ hits, const Geom g) {
  extern __shared__ int cnt[];
  __shared__ int wmax[32];
  const int n = blockIdx.x;
  for (int i = threadIdx.x; i < g.HW; i += blockDim.x) cnt[i] = 0;
  __syncthreads();
  const __half* off_n = off + (size_t)n * 18 * g.P;
  for (int idx = threadIdx.x; idx < 9 * g.P; idx += blockDim.x) {
    const int t = idx / g.P, p = idx - t * g.P;
    const int oh = p / g.Wo, ow = p - oh * g.Wo;
    const float ph = (float)(oh * S - 1 + t / 3) + __half2float(__ldg(off_n + (size_t)(2 * t) * g.P + p));
    const float pw = (float)(ow * S - 1 + t % 3) + __half2float(__ldg(off_n + (size_t)(2 * t + 1) * g.P + p));
    if (ph > -1.f && pw > -1.f && ph < (float)g.H && pw < (float)g.W) {
      const int h0 = (int)floorf(ph), w0 = (int)floorf(pw);
      const int h0c = max(h0, 0), h1c = min(h0 + 1, g.H - 1), w0c = max(w0, 0), w1c = min(w0 + 1, g.W - 1);
      atomicAdd(&cnt[h0c * g.W + w0c], 1);
      atomicAdd(&cnt[h0c * g.W + w1c], 1);
      atomicAdd(&cnt[h1c * g.W + w0c], 1);
      atomicAdd(&cnt[h1c * g.W + w1c], 1);
    }
  }
  __syncthreads();
  int m = 1;
  for (int i = threadIdx.x; i < g.HW; i += blockDim.x) m = max(m, cnt[i]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0) wmax[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int k = 1; k < (int)(blockDim.x >> 5); ++k) m = max(m, wmax[k]);
    hits[n] = m;
  }
}

__device__ __forceinline__ void red_shared_s32(unsigned a, int v) {
  asm volatile("red.shared.add.s32 [%0], %1;\n" ::"r"(a), "r"(v) : "memory");
}

// o: shared addresses of the four corners' first channel group; lane_off = 4 * (channel & 7);
// ga, gb: scaled K * dy of this pixel for channel rows gq and gq + 8
__device__ __forceinline__ void scatter8(const uint4 o, const uint4 cf, float ga, float gb, unsigned lane_off) {
  constexpr float kMagic = 12582912.f;  // 1.5 * 2^23: (v + kMagic) has rint(v) in its low mantissa bits for |v| < 2^22
  constexpr int kMagicBits = 0x4B400000;
  const unsigned ok[4] = {o.x, o.y, o.z, o.w};
  const unsigned ck[4] = {cf.x, cf.y, cf.z, cf.w};
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const unsigned a = ok[k] + lane_off;
    const float c = __uint_as_float(ck[k]);
    red_shared_s32(a, __float_as_int(fmaf(c, ga, kMagic)) - kMagicBits);
    red_shared_s32(a ^ 64u, __float_as_int(fmaf(c, gb, kMagic)) - kMagicBits);  // channels 8..15: group index ^ 2
  }
}

// everything an item needs from global memory: kernel-space offsets of pixel gq (9 taps, h | w << 16), image-space
// offsets of the table builder's (pixel, tap column) for the three kernel rows, dy of the lane's two pixels
struct ItemRegs {
  unsigned rp[9], op[3], dy0, dy1;
};
__device__ __forceinline__ void fetch_item(ItemRegs& r, const __half* __restrict__ dy, const __half* __restrict__ off,
                                           const __half* __restrict__ rot, const Geom& g, int n, int c0, int oh, int ow0, int lane,
                                           bool pair_dy) {
  const int gq = lane >> 2, q = lane & 3;
  const size_t row = (size_t)oh * g.Wo;
  {
    const int pc = ow0 + gq;
    const __half* rp = rot + (size_t)n * 18 * g.P + row + pc;
#pragma unroll
    for (int t = 0; t < 9; ++t) {
      r.rp[t] = 0u;
      if (rot != nullptr && pc < g.Wo)
        r.rp[t] = (unsigned)__half_as_ushort(__ldg(rp + (size_t)(2 * t) * g.P)) |
                  ((unsigned)__half_as_ushort(__ldg(rp + (size_t)(2 * t + 1) * g.P)) << 16);
    }
  }
  {
    const int pc = ow0 + (lane & 7), fw = lane >> 3;
    const __half* op = off + (size_t)n * 18 * g.P + row + pc;
#pragma unroll
    for (int fh = 0; fh < 3; ++fh) {
      r.op[fh] = 0u;
      if (lane < 24 && pc < g.Wo) {
        const int t = fh * 3 + fw;
        r.op[fh] = (unsigned)__half_as_ushort(__ldg(op + (size_t)(2 * t) * g.P)) |
                   ((unsigned)__half_as_ushort(__ldg(op + (size_t)(2 * t + 1) * g.P)) << 16);
      }
    }
  }
  r.dy0 = r.dy1 = 0u;
  const int ow = ow0 + 2 * q;
  if (ow < g.Wo) {
    const __half* p0 = dy + ((size_t)n * g.C + c0 + gq) * g.P + row + ow;
    const __half* p1 = p0 + (size_t)8 * g.P;
    if (pair_dy) {
      r.dy0 = __ldg(reinterpret_cast<const unsigned*>(p0));
      r.dy1 = __ldg(reinterpret_cast<const unsigned*>(p1));
    } else {
      r.dy0 = __half_as_ushort(__ldg(p0));
      r.dy1 = __half_as_ushort(__ldg(p1));
      if (ow + 1 < g.Wo) {
        r.dy0 |= (unsigned)__half_as_ushort(__ldg(p0 + 1)) << 16;
        r.dy1 |= (unsigned)__half_as_ushort(__ldg(p1 + 1)) << 16;
      }
    }
  }
}

template <int S, bool ZR>
__global__ void __launch_bounds__(512, 1) mma_deform_data_kernel(const __half* __restrict__ dy, const __half* __restrict__ off,
                                                                const __half* __restrict__ rot, const __half* __restrict__ w,
                                                                const int* __restrict__ hits, __half* __restrict__ dx,
                                                                const Geom g, const DDataPlan pl) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int c0 = blockIdx.y * 16;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int gq = lane >> 2, q = lane & 3;
  const int NB = (g.Wo + 7) >> 3;
  const int items = g.Ho * NB;
  const int rows = (g.HW + 1) >> 1;  // pixel pairs

  // planes on a 128-byte boundary: the channel-half select is an XOR of the address with 64
  const unsigned raw_saddr = (unsigned)__cvta_generic_to_shared(smem_raw);
  const unsigned pad = (128u - (raw_saddr & 127u)) & 127u;
  int* acc = reinterpret_cast<int*>(smem_raw + pad);  // [rows][32]
  const unsigned acc_saddr = raw_saddr + pad;
  float* scales = reinterpret_cast<float*>(acc + (size_t)rows * 32);  // [16] scale, [16] 1 / scale
  unsigned* tab = reinterpret_cast<unsigned*>(scales + 32) + warp * kPairTabWords;
  const LaneCells lc = lane_cells(g, q);
  const bool sc44 = g.scH == 4 && g.scW == 4;

  unsigned wa[4];  // A fragments of the bank slab (see the forward)
  {
    const __half* w0 = w + (size_t)(c0 + gq) * g.cells;
    const __half* w1 = w0 + (size_t)8 * g.cells;
    auto cell2 = [&](const __half* p, int k) {
      const unsigned lo = k < g.cells ? (unsigned)__half_as_ushort(__ldg(p + k)) : 0u;
      const unsigned hi = k + 1 < g.cells ? (unsigned)__half_as_ushort(__ldg(p + k + 1)) : 0u;
      return lo | (hi << 16);
    };
    wa[0] = cell2(w0, 2 * q);
    wa[1] = cell2(w1, 2 * q);
    wa[2] = cell2(w0, 2 * q + 8);
    wa[3] = cell2(w1, 2 * q + 8);
  }
  const unsigned lane_off = gq * 4;
  constexpr bool zero_rot = ZR;  // rot == nullptr
  unsigned bf[9][2];
  if (zero_rot) {
    const unsigned z[9] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
    beta_from_regs(bf, z, g, lc, sc44, true);
  }

  const int n_begin = blockIdx.x * pl.samples_per_block;
  const int n_end = min(n_begin + pl.samples_per_block, g.N);
  for (int n = n_begin; n < n_end; ++n) {
    ItemRegs cur;
    if (warp < items) fetch_item(cur, dy, off, rot, g, n, c0, warp / NB, (warp % NB) << 3, lane, pl.pair_dy);
    __syncthreads();  // the previous sample's planes have been written out
    {
      uint4* a4 = reinterpret_cast<uint4*>(acc);
      const uint4 z = make_uint4(0, 0, 0, 0);
      for (int i = threadIdx.x; i < rows * 8; i += blockDim.x) a4[i] = z;
    }
    // scale of each channel from max |dy| over its plane: warp k scans channel k
    for (int ch = warp; ch < 16; ch += nwarps) {
      const __half* p = dy + ((size_t)n * g.C + c0 + ch) * g.P;
      float m = 0.f;
      if (pl.pair_dy) {
        const unsigned* p2 = reinterpret_cast<const unsigned*>(p);
        for (int i = lane; i < (g.P >> 1); i += 32) {
          const unsigned v = __ldg(p2 + i);
          m = fmaxf(m, fmaxf(fabsf(lo2f(v)), fabsf(hi2f(v))));
        }
      } else {
        for (int i = lane; i < g.P; i += 32) m = fmaxf(m, fabsf(__half2float(__ldg(p + i))));
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
      if (lane == 0) {
        float wm = 0.f;
        for (int k = 0; k < g.cells; ++k) wm = fmaxf(wm, fabsf(__half2float(__ldg(w + (size_t)(c0 + ch) * g.cells + k))));
        const float bound = m * wm * 1.01f;
        // at most hits[n] contributions per accumulator, each at most 2^limit: no overflow of 31 bits; and each
        // below 2^22, the range of the float -> integer conversion in scatter8
        const int limit_log2 = min(21, 30 - (32 - __clz(max(__ldg(hits + n), 1) - 1)));
        int e = 0;  // scale = 2^e with bound * 2^e <= 2^limit_log2
        if (bound > 0.f && bound < 3e38f) {
          const float lim = ldexpf(1.f, limit_log2) / bound;
          e = ((__float_as_int(lim) >> 23) & 0xff) - 127;  // floor(log2(lim))
          e = max(-100, min(100, e));
        }
        scales[ch] = __int_as_float((e + 127) << 23);
        scales[16 + ch] = __int_as_float((127 - e) << 23);
      }
    }
    __syncthreads();
    const float sa = scales[gq], sb = scales[gq + 8];
    for (int item = warp; item < items; item += nwarps) {
      const int oh = item / NB;
      const int ow0 = (item - oh * NB) << 3;
      ItemRegs nxt;
      const int item2 = item + nwarps;
      if (item2 < items) {
        const int oh2 = item2 / NB;
        fetch_item(nxt, dy, off, rot, g, n, c0, oh2, (item2 - oh2 * NB) << 3, lane, pl.pair_dy);
      }
      if (!zero_rot) beta_from_regs(bf, cur.rp, g, lc, sc44, ow0 + gq < g.Wo);
#pragma unroll
      for (int fh = 0; fh < 3; ++fh) {
        __syncwarp();
        if (lane < 24) pair_table_entry<S, true>(tab, g, fh, oh, ow0, lane, lo2f(cur.op[fh]), hi2f(cur.op[fh]), acc_saddr);
        __syncwarp();
#pragma unroll
        for (int fw = 0; fw < 3; ++fw) {
          const int t = fh * 3 + fw;
          const uint4* e0 = reinterpret_cast<const uint4*>(tab + fw * 80 + q * 20);
          const uint4 oA = e0[0], cA = e0[1], oB = e0[2], cB = e0[3];  // pixel 2q, pixel 2q + 1
          unsigned kk[2];
          mma16816_h(kk, wa, bf[t][0], bf[t][1]);
          const unsigned g0 = hmul2u(kk[0], cur.dy0), g1 = hmul2u(kk[1], cur.dy1);  // K * dy of channel gq, gq + 8
          scatter8(oA, cA, lo2f(g0) * sa, lo2f(g1) * sb, lane_off);
          scatter8(oB, cB, hi2f(g0) * sa, hi2f(g1) * sb, lane_off);
        }
      }
      if (item2 < items) cur = nxt;
    }
    __syncthreads();
    // write the planes: a warp covers 8 channels x 4 pixel pairs, which sit in 32 different banks
    __half* dx_n = dx + ((size_t)n * g.C + c0) * g.HW;
    const bool pair_dx = (g.HW & 1) == 0 && pl.pair_dy;
    for (int task = threadIdx.x; task < rows * 16; task += blockDim.x) {
      const int rw = task >> 3;
      const int half = rw / rows, row = rw - half * rows;
      const int ch = half * 8 + (task & 7), i = row * 2;
      const float inv = scales[16 + ch];
      const float v0 = (float)acc[acc_word<S>(i, ch)] * inv, v1 = (float)acc[acc_word<S>(i + 1, ch)] * inv;
      __half* o = dx_n + (size_t)ch * g.HW + i;
      if (pair_dx) {
        *reinterpret_cast<unsigned*>(o) = pack2(v0, v1);
      } else {
        o[0] = __float2half_rn(v0);
        if (i + 1 < g.HW) o[1] = __float2half_rn(v1);
      }
    }
  }
}

// ------------------------------------------------------------------ gradients of the two offset fields
// d(kernel offset)[p, tap, dir] = sum_c dy * xs * dK/d(u|v)   and   d(image offset)[p, tap, dir] = sum_c dy * K * dxs/d(h|w).
// The first goes through G = W^T * (dy * xs) and the derivative hat weights exactly as in the local operator
// (dk_local_mma.cu).  For the second, K comes from one mma per tap as in the forward, dxs/dh and dxs/dw are two more
// coefficient sets over the same four image reads, and the sum over channels of E = dy * K * dxs is an mma with a
// matrix of ones: the transposed E fragments (rows = 8 pixels x 2 directions, k = 16 channels) are its A operand.
// A block owns 16 * NS channels; when that is not all of them, blocks add their partial sums into an fp32 buffer
// [sample][36 planes][pixel] (image offsets first) with red.global.add.f32 and a second kernel rounds it.
struct DCoordPlan {
  int NS, BH, warps, bands, units_per_block, blocks_x, groups;
  int mode_dy, mode_rot, mode_off;
  bool vec;
  size_t smem, ws_bytes;
};
constexpr int kCoordTabWords = 3 * 144;                   // 3 taps x 4 pixel pairs x (2 x 16 words + 4 of padding)
constexpr int kCoordWarpWords = kCoordTabWords + 2 * 72;  // + the (u, v) of the item's 72 (pixel, tap) pairs
constexpr int kBankPitch = 24;                            // halves per channel row of the bank copy (conflict-free fragments)

// Sampling table with derivatives: per (pixel, tap) four corner offsets, then three sets of four coefficients
// (value, d/dh, d/dw), each duplicated into both halves of a word.  Lanes 0..23.
template <int S>
__device__ __forceinline__ void build_coord_table(unsigned* __restrict__ tab, const __half* __restrict__ oband, const Band& bo,
                                                  const Geom& g, int fh, int oh, int ow0, int lane) {
  if (lane < 24) {
    const int px = lane & 7, fw = lane >> 3;
    const int pc = ow0 + px;
    const int t = fh * 3 + fw;
    const __half* op = oband + (size_t)(2 * t) * bo.pitch_c + kSlack + oh * bo.Wp + pc - bo.org;
    const float ph = (float)(oh * S - 1 + fh) + __half2float(op[0]);
    const float pw = (float)(pc * S - 1 + fw) + __half2float(op[bo.pitch_c]);
    const bool used = pc < g.Wo && ph > -1.f && pw > -1.f && ph < (float)g.H && pw < (float)g.W;
    uint4 o4 = make_uint4(0, 0, 0, 0), cv = o4, ch = o4, cw = o4;
    if (used) {
      const float fph = floorf(ph), fpw = floorf(pw);
      const int h0 = (int)fph, w0 = (int)fpw;
      const float lh = ph - fph, lw = pw - fpw;
      const float hh = 1.f - lh, hw = 1.f - lw;
      const bool r0 = h0 >= 0, r1 = h0 + 1 <= g.H - 1, k0 = w0 >= 0, k1 = w0 + 1 <= g.W - 1;
      const int h0c = max(h0, 0), h1c = min(h0 + 1, g.H - 1), w0c = max(w0, 0), w1c = min(w0 + 1, g.W - 1);
      o4.x = (unsigned)chunk_of<S>(h0c * g.W + w0c) * 32u;
      o4.y = (unsigned)chunk_of<S>(h0c * g.W + w1c) * 32u;
      o4.z = (unsigned)chunk_of<S>(h1c * g.W + w0c) * 32u;
      o4.w = (unsigned)chunk_of<S>(h1c * g.W + w1c) * 32u;
      auto dup = [](bool ok, float v) { return ok ? pack2(v, v) : 0u; };
      cv = make_uint4(dup(r0 && k0, hh * hw), dup(r0 && k1, hh * lw), dup(r1 && k0, lh * hw), dup(r1 && k1, lh * lw));
      ch = make_uint4(dup(r0 && k0, -hw), dup(r0 && k1, -lw), dup(r1 && k0, hw), dup(r1 && k1, lw));
      cw = make_uint4(dup(r0 && k0, -hh), dup(r0 && k1, hh), dup(r1 && k0, -lh), dup(r1 && k1, lh));
    }
    uint4* e = reinterpret_cast<uint4*>(tab + fw * 144 + (px >> 1) * 36 + (px & 1) * 16);
    e[0] = o4;
    e[1] = cv;
    e[2] = ch;
    e[3] = cw;
  }
}

// value and both derivatives of (channel j | channel j + 8) at one (pixel, tap)
__device__ __forceinline__ void sample_pair3(unsigned& v, unsigned& dh, unsigned& dw, const char* __restrict__ base,
                                             const uint4* __restrict__ e) {
  const uint4 o = e[0], cv = e[1], ch = e[2], cw = e[3];
  const unsigned x0 = *reinterpret_cast<const unsigned*>(base + o.x), x1 = *reinterpret_cast<const unsigned*>(base + o.y);
  const unsigned x2 = *reinterpret_cast<const unsigned*>(base + o.z), x3 = *reinterpret_cast<const unsigned*>(base + o.w);
  v = hfma2u(x3, cv.w, hfma2u(x2, cv.z, hfma2u(x1, cv.y, hmul2u(x0, cv.x))));
  dh = hfma2u(x3, ch.w, hfma2u(x2, ch.z, hfma2u(x1, ch.y, hmul2u(x0, ch.x))));
  dw = hfma2u(x3, cw.w, hfma2u(x2, cw.z, hfma2u(x1, cw.y, hmul2u(x0, cw.x))));
}

// DO_BANK: the bank gradient dW += (dy * xs) * beta rides along (the products dy * xs are formed here anyway for the
// kernel-offset gradient): accumulators in registers over all units of the block, one partial [CG][16] per block at the end.
template <int S, int NS, bool DO_OFF, bool DO_ROT, bool ZR, bool DO_BANK>
__global__ void __launch_bounds__(DO_BANK ? 384 : 512, 1)  // the bank accumulators need the registers of four warps
    mma_deform_coords_kernel(const __half* __restrict__ dy, const __half* __restrict__ x, const __half* __restrict__ off,
                             const __half* __restrict__ rot, const __half* __restrict__ w, __half* __restrict__ doff,
                             __half* __restrict__ drot, float* __restrict__ partial, float* __restrict__ bank_partial,
                             const Geom g, const DCoordPlan pl) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int CG = 16 * NS;
  constexpr int pitchT = CG + 8;
  const int c0 = blockIdx.y * CG;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int gq = lane >> 2, q = lane & 3;
  const int NB = (g.Wo + 7) >> 3;
  const int items = pl.BH * NB;
  const int Wpo = g.Wo + (g.Wo & 1);
  const int HW16 = (g.HW + 15) & ~15;
  const int ypitch = band_pitch(pl.BH, Wpo);

  unsigned* xw = reinterpret_cast<unsigned*>(smem_raw);                      // [NS][HW16 * 8]
  __half* yband = reinterpret_cast<__half*>(xw + (size_t)NS * HW16 * 8);     // [CG][ypitch]
  __half* rband = yband + (size_t)CG * ypitch;                               // [18][ypitch]
  __half* oband = rband + (size_t)18 * ypitch;                               // [18][ypitch]
  __half* bankT = oband + (size_t)18 * ypitch;                               // [16 cells][CG + 8]
  __half* bank = bankT + 16 * pitchT;                                        // [CG][kBankPitch]
  unsigned* tab = reinterpret_cast<unsigned*>(bank + CG * kBankPitch) + warp * kCoordWarpWords;
  float* Gs = reinterpret_cast<float*>(tab);                   // [3 taps][16 cells][8 px], aliases the table
  float2* uv = reinterpret_cast<float2*>(tab + kCoordTabWords);  // [9 taps][8 px]
  const LaneCells lc = lane_cells(g, q);
  const bool sc44 = g.scH == 4 && g.scW == 4;

  for (int i = threadIdx.x; i < 16 * CG; i += blockDim.x) {
    const int cell = i / CG, c = i - cell * CG;
    const __half v = cell < g.cells ? __ldg(w + (size_t)(c0 + c) * g.cells + cell) : __float2half(0.f);
    bankT[cell * pitchT + c] = v;
    bank[c * kBankPitch + cell] = v;
  }

  constexpr bool zero_rot = ZR;  // rot == nullptr; then DO_ROT is false: there is nothing to differentiate
  unsigned bf[9][2];
  if (zero_rot) {
    const unsigned z[9] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
    beta_from_regs(bf, z, g, lc, sc44, true);
  }

  float acc[DO_BANK ? NS : 1][2][4];  // bank gradient: slabs of 16 channels x (cells 0-7 | cells 8-15)
#pragma unroll
  for (int sidx = 0; sidx < (DO_BANK ? NS : 1); ++sidx)
#pragma unroll
    for (int k = 0; k < 4; ++k) acc[sidx][0][k] = acc[sidx][1][k] = 0.f;

  const int total_units = g.N * pl.bands;
  const int u_begin = blockIdx.x * pl.units_per_block;
  const int u_end = min(u_begin + pl.units_per_block, total_units);
  int cur_n = -1;
  for (int unit = u_begin; unit < u_end; ++unit) {
    const int n = unit / pl.bands;
    const int oh0 = (unit - n * pl.bands) * pl.BH;
    const Band by = make_band(oh0, pl.BH, g.Ho, g.Wo, pl.mode_dy);
    const Band br = make_band(oh0, pl.BH, g.Ho, g.Wo, pl.mode_rot);
    const Band bo = make_band(oh0, pl.BH, g.Ho, g.Wo, pl.mode_off);
    __syncthreads();  // readers of the previous unit are done
    load_band(yband, by, dy, n, g.C, c0, CG, g.Ho, g.Wo);
    if (!zero_rot) load_band(rband, br, rot, n, 18, 0, 18, g.Ho, g.Wo);
    load_band(oband, bo, off, n, 18, 0, 18, g.Ho, g.Wo);
    if (n != cur_n) {
#pragma unroll
      for (int sidx = 0; sidx < NS; ++sidx) load_pair_planes<S>(xw + (size_t)sidx * HW16 * 8, x, n, g.C, c0 + 16 * sidx, g.HW, pl.vec);
      cur_n = n;
    }
    cp_async_wait_all();
    __syncthreads();

    constexpr bool want_off = DO_OFF, want_rot = DO_ROT;  // a field nobody asked for is not computed
    __half* doff_n = doff ? doff + (size_t)n * 18 * g.P : nullptr;
    __half* drot_n = drot ? drot + (size_t)n * 18 * g.P : nullptr;
    float* part_n = partial + (size_t)n * 36 * g.P;
    for (int item = warp; item < items; item += nwarps) {
      const int dr = item / NB;
      const int oh = oh0 + dr;
      if (oh >= g.Ho) break;
      const int ow0 = (item - dr * NB) << 3;
      if (!zero_rot) beta_direct<S, false, false>(bf, rband, br, g, lc, sc44, oh, ow0, g.H, g.W, g.Wo, gq);
      __syncwarp();
      if (DO_ROT) item_uv<S, false>(uv, rband, br, g, oh, ow0, lane);
      const int yoff = kSlack + oh * by.Wp + ow0 + 2 * q - by.org;
      unsigned dy0[NS], dy1[NS];
#pragma unroll
      for (int sidx = 0; sidx < NS; ++sidx) {
        dy0[sidx] = *reinterpret_cast<const unsigned*>(yband + (size_t)(16 * sidx + gq) * by.pitch_c + yoff);
        dy1[sidx] = *reinterpret_cast<const unsigned*>(yband + (size_t)(16 * sidx + gq + 8) * by.pitch_c + yoff);
      }
      const char* lane_base = reinterpret_cast<const char*>(xw) + gq * 4;
      const size_t row = (size_t)oh * g.Wo + ow0;
#pragma unroll
      for (int fh = 0; fh < 3; ++fh) {
        __syncwarp();  // the previous pass has read Gs (the table's storage)
        build_coord_table<S>(tab, oband, bo, g, fh, oh, ow0, lane);
        __syncwarp();
        float G[3][4], D[3][4];
#pragma unroll
        for (int fw = 0; fw < 3; ++fw)
#pragma unroll
          for (int k = 0; k < 4; ++k) G[fw][k] = D[fw][k] = 0.f;
        unsigned bw[3][2];  // DO_BANK: the hat products of this kernel row as B fragments of dW += dK * beta
        if (DO_BANK) {
#pragma unroll
          for (int fw = 0; fw < 3; ++fw) {
            bw[fw][0] = movmatrix_trans(bf[fh * 3 + fw][0]);
            bw[fw][1] = movmatrix_trans(bf[fh * 3 + fw][1]);
          }
        }
#pragma unroll
        for (int sidx = 0; sidx < NS; ++sidx) {
          const int cb16 = 16 * sidx;
          unsigned pa = 0u, pb = 0u;  // DO_BANK: dK of tap 0, waiting for tap 1 to fill the k = 16 of one mma
          // A = W slab (rows = channels gq, gq + 8; k = cells) and A = W^T slab (rows = cells; k = channels)
          const unsigned* b0 = reinterpret_cast<const unsigned*>(bank + (cb16 + gq) * kBankPitch);
          const unsigned* b1 = reinterpret_cast<const unsigned*>(bank + (cb16 + gq + 8) * kBankPitch);
          const unsigned wa[4] = {b0[q], b1[q], b0[q + 4], b1[q + 4]};
          const unsigned* wt0 = reinterpret_cast<const unsigned*>(bankT + gq * pitchT + cb16);
          const unsigned* wt1 = reinterpret_cast<const unsigned*>(bankT + (gq + 8) * pitchT + cb16);
          const unsigned t0 = wt0[q], t1 = wt1[q], t2 = wt0[q + 4], t3 = wt1[q + 4];
          const char* base = lane_base + (size_t)sidx * HW16 * 32;
#pragma unroll
          for (int fw = 0; fw < 3; ++fw) {
            const uint4* e0 = reinterpret_cast<const uint4*>(tab + fw * 144 + q * 36);
            unsigned vA, hA, wA, vB, hB, wB;  // pixel 2q and pixel 2q + 1: (channel gq | channel gq + 8)
            sample_pair3(vA, hA, wA, base, e0);
            sample_pair3(vB, hB, wB, base, e0 + 4);
            if (want_rot || DO_BANK) {
              const unsigned ka = hmul2u(dy0[sidx], __byte_perm(vA, vB, 0x5410));  // dK of channel gq: pixels 2q, 2q + 1
              const unsigned kb = hmul2u(dy1[sidx], __byte_perm(vA, vB, 0x7632));  // channel gq + 8
              // kernel offsets: G += W^T * (dy * xs)
              if (want_rot) mma16816_acc(G[fw], t0, t1, t2, t3, movmatrix_trans(ka), movmatrix_trans(kb));
              if (DO_BANK) {
                if (fw == 0) {
                  pa = ka;
                  pb = kb;
                } else if (fw == 1) {  // k = 16 = 8 pixels x (tap 0 | tap 1)
                  mma16816_acc(acc[DO_BANK ? sidx : 0][0], pa, pb, ka, kb, bw[0][0], bw[1][0]);
                  mma16816_acc(acc[DO_BANK ? sidx : 0][1], pa, pb, ka, kb, bw[0][1], bw[1][1]);
                } else {  // the third tap, paired with zeros
                  mma16816_acc(acc[DO_BANK ? sidx : 0][0], ka, kb, 0u, 0u, bw[2][0], 0u);
                  mma16816_acc(acc[DO_BANK ? sidx : 0][1], ka, kb, 0u, 0u, bw[2][1], 0u);
                }
              }
            }
            if (want_off) {  // image offsets: D[pixel, dir] += sum over the slab's channels of dy * K * dxs
              unsigned kk[2];
              mma16816_h(kk, wa, bf[fh * 3 + fw][0], bf[fh * 3 + fw][1]);
              const unsigned ya = hmul2u(kk[0], dy0[sidx]), yb = hmul2u(kk[1], dy1[sidx]);
              const unsigned eha = hmul2u(ya, __byte_perm(hA, hB, 0x5410)), ehb = hmul2u(yb, __byte_perm(hA, hB, 0x7632));
              const unsigned ewa = hmul2u(ya, __byte_perm(wA, wB, 0x5410)), ewb = hmul2u(yb, __byte_perm(wA, wB, 0x7632));
              mma16816_acc(D[fw], movmatrix_trans(eha), movmatrix_trans(ewa), movmatrix_trans(ehb), movmatrix_trans(ewb),
                           0x3C003C00u, 0x3C003C00u);
            }
          }
        }
        // image offsets: row gq of D = pixel gq, direction h; row gq + 8 = direction w (every column holds the sum)
        if (want_off && q == 0 && ow0 + gq < g.Wo) {
#pragma unroll
          for (int fw = 0; fw < 3; ++fw) {
            const size_t o = (size_t)(2 * (fh * 3 + fw)) * g.P + row + gq;
            if (pl.groups == 1) {
              if (doff_n) {
                doff_n[o] = __float2half_rn(D[fw][0]);
                doff_n[o + g.P] = __float2half_rn(D[fw][2]);
              }
            } else {
              atomicAdd(part_n + o, D[fw][0]);
              atomicAdd(part_n + o + g.P, D[fw][2]);
            }
          }
        }
        if (!want_rot) continue;
        // kernel offsets: sum over the four corner cells of G * d(hat weight)/d(u or v)
        __syncwarp();  // the table has been read by every lane
#pragma unroll
        for (int fw = 0; fw < 3; ++fw) {
          *reinterpret_cast<float2*>(Gs + (fw * 16 + gq) * 8 + 2 * q) = make_float2(G[fw][0], G[fw][1]);
          *reinterpret_cast<float2*>(Gs + (fw * 16 + gq + 8) * 8 + 2 * q) = make_float2(G[fw][2], G[fw][3]);
        }
        __syncwarp();
        if (lane < 24) {
          const int px = lane & 7, fw = lane >> 3;
          const int t = fh * 3 + fw;
          const float2 c = uv[t * 8 + px];
          float gu = 0.f, gv = 0.f;
          if (c.x < 1e29f) {
            const float fu = floorf(c.x), fv = floorf(c.y);
            const int h0 = (int)fu, w0 = (int)fv;
            const float lh = c.x - fu, lw = c.y - fv;
            const float hh = 1.f - lh, hw = 1.f - lw;
            const float* Gp = Gs + fw * 128 + px;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const int a = h0 + (k >> 1), b = w0 + (k & 1);
              if (a >= 0 && a < g.scH && b >= 0 && b < g.scW) {
                const float gval = Gp[(a * g.scW + b) * 8];
                const float du = (k >> 1) ? ((k & 1) ? lw : hw) : ((k & 1) ? -lw : -hw);
                const float dv = (k & 1) ? ((k >> 1) ? lh : hh) : ((k >> 1) ? -lh : -hh);
                gu += du * gval;
                gv += dv * gval;
              }
            }
          }
          if (ow0 + px < g.Wo) {
            const size_t o = (size_t)(2 * t) * g.P + row + px;
            if (pl.groups == 1) {
              if (drot_n) {
                drot_n[o] = __float2half_rn(gu);
                drot_n[o + g.P] = __float2half_rn(gv);
              }
            } else {
              atomicAdd(part_n + 18 * g.P + o, gu);
              atomicAdd(part_n + 18 * g.P + o + g.P, gv);
            }
          }
        }
      }
      __syncwarp();
    }
  }
  if (DO_BANK) {  // reduce the warps' accumulators and write this block's partial bank gradient [CG channels][16 cells]
    __syncthreads();
    float* red = reinterpret_cast<float*>(smem_raw);  // [nwarps][CG][16]
#pragma unroll
    for (int sidx = 0; sidx < (DO_BANK ? NS : 1); ++sidx) {
      float* r0 = red + ((size_t)warp * CG + 16 * sidx + gq) * 16;
      float* r1 = r0 + 8 * 16;
      r0[2 * q] = acc[sidx][0][0]; r0[2 * q + 1] = acc[sidx][0][1];
      r1[2 * q] = acc[sidx][0][2]; r1[2 * q + 1] = acc[sidx][0][3];
      r0[8 + 2 * q] = acc[sidx][1][0]; r0[8 + 2 * q + 1] = acc[sidx][1][1];
      r1[8 + 2 * q] = acc[sidx][1][2]; r1[8 + 2 * q + 1] = acc[sidx][1][3];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < CG * 16; i += blockDim.x) {
      float sum = 0.f;
      for (int wv = 0; wv < nwarps; ++wv) sum += red[(size_t)wv * CG * 16 + i];
      bank_partial[((size_t)blockIdx.x * g.C + c0) * 16 + i] = sum;
    }
  }
}

// out = fp16(partial) for one of the two offset fields: partial is [N][36][P], the field's 18 planes start at `first`
__global__ void round_coord_partials_kernel(const float* __restrict__ partial, __half* __restrict__ out, int N, size_t plane18,
                                            int first) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)N * plane18) return;
  const size_t n = i / plane18, r = i - n * plane18;
  out[i] = __float2half_rn(partial[n * 2 * plane18 + (size_t)first * (plane18 / 18) + r]);
}

__global__ void reduce_dcn_bank_partials_kernel(const float* __restrict__ partial, __half* __restrict__ out, int C, int cells,
                                                int nblocks) {
  const int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (i >= C * cells) return;
  const int c = i / cells, cell = i - c * cells;
  float s = 0.f;
  for (int k = lane; k < nblocks; k += 32) s += partial[((size_t)k * C + c) * 16 + cell];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) out[i] = __float2half_rn(s);
}

bool dcn_fast_shape(const Geom& g) {
  if (g.kH != 3 || g.kW != 3 || g.dH != 1 || g.dW != 1 || g.pH != 1 || g.pW != 1) return false;
  if (g.sH != g.sW || (g.sH != 1 && g.sH != 2)) return false;
  if (g.G != 1 || g.cells > 16 || (g.C & 15)) return false;
  return true;
}

int min_items() {  // DK_B200_DCN_MIN_ITEMS: fewest items per band for which more than one slab per block is taken (tuning knob)
  const char* e = tuning_env("DK_B200_DCN_MIN_ITEMS");
  const int v = e ? atoi(e) : 0;
  return v > 0 ? v : 14;  // measured at 56 x 56: forward 0.75 -> 0.69 ms with two slabs and 21 items; 7 items lose
}

// Shape of the grid.  NS slabs of 16 channels per block share the hat products and the sampling tables, so more
// is better while every SM still gets a block; the band of output rows is as tall as shared memory allows beside
// the planes (its loads are paid once per unit), cut finer when there are too few units to fill the GPU.
// dy_rows = 1 when a band of dy (16 * NS channels) is staged too.
DcnPlan dcn_plan(const Geom& g, int ns_cap, int dy_rows) {
  DcnPlan pl;
  pl.BH = 0;
  if (!dcn_fast_shape(g)) return pl;
  const int NB = (g.Wo + 7) / 8;
  const int Wpo = g.Wo + (g.Wo & 1);
  const int HW16 = (g.HW + 15) & ~15;
  const size_t plane = (size_t)HW16 * 32;
  const int slabs = g.C / 16;
  for (int ns = 4; ns >= 1; ns >>= 1) {
    if (ns > ns_cap || slabs % ns) continue;
    if (ns > 1 && (long long)(slabs / ns) * g.N < 148) continue;
    auto need = [&](int bh, int& warps) {
      warps = bh * NB;
      if (warps > 16) warps = 16;
      if (warps < 2) warps = 2;
      const size_t smem = ns * plane + (size_t)(36 + dy_rows * 16 * ns) * band_pitch(bh, Wpo) * 2 + (size_t)warps * kPairTabWords * 4;
      const size_t red = dy_rows ? (size_t)warps * 16 * ns * 16 * 4 : 0;
      return smem < red ? red : smem;
    };
    int bh_max = 0, wv;
    for (int bh = 1; bh <= g.Ho; ++bh) {
      if (need(bh, wv) > kOnePerSm) break;
      bh_max = bh;
    }
    if (!bh_max || (ns > 1 && bh_max * NB < min_items() && bh_max < g.Ho)) continue;  // short bands: the per-unit cost eats the gain
    const int groups = slabs / ns;
    int bands = (g.Ho + bh_max - 1) / bh_max;
    const long long base_units = (long long)g.N * groups;
    if (base_units * bands < 148) {
      long long wantb = (148 + base_units - 1) / base_units;
      if (wantb > g.Ho) wantb = g.Ho;
      if (wantb > bands) bands = (int)wantb;
    }
    pl.NS = ns;
    pl.BH = (g.Ho + bands - 1) / bands;
    pl.bands = (g.Ho + pl.BH - 1) / pl.BH;
    pl.smem = need(pl.BH, pl.warps);
    const long long units = (long long)g.N * pl.bands;
    long long want = 148 / groups;  // one block per SM: a single wave over all channel groups
    if (want > units) want = units;
    if (want < 1) want = 1;
    pl.units_per_block = (int)((units + want - 1) / want);
    pl.blocks_x = (int)((units + pl.units_per_block - 1) / pl.units_per_block);
    pl.ws_bytes = (size_t)pl.blocks_x * g.C * 16 * sizeof(float);
    return pl;
  }
  return pl;
}

DDataPlan ddata_plan(const Geom& g) {
  DDataPlan pl;
  pl.warps = 0;
  if (!dcn_fast_shape(g)) return pl;
  const int groups = g.C / 16;
  if ((long long)g.N * groups < 96) return pl;  // whole samples per block: too few of them to fill the GPU
  const int NB = (g.Wo + 7) / 8;
  const int items = g.Ho * NB;
  pl.warps = items < 16 ? (items < 2 ? 2 : items) : 16;
  pl.smem = 128 + (size_t)((g.HW + 1) / 2) * 128 + 128 + (size_t)pl.warps * kPairTabWords * 4;

  if (pl.smem > kOnePerSm) {
    pl.warps = 0;
    return pl;
  }
  int want = 148 / groups;
  if (want > g.N) want = g.N;
  if (want < 1) want = 1;
  pl.samples_per_block = (g.N + want - 1) / want;
  pl.blocks_x = (g.N + pl.samples_per_block - 1) / pl.samples_per_block;
  return pl;
}

DCoordPlan dcoord_plan(const Geom& g, int ns_cap) {
  DCoordPlan pl;
  pl.BH = 0;
  if (!dcn_fast_shape(g)) return pl;
  const int NB = (g.Wo + 7) / 8;
  const int Wpo = g.Wo + (g.Wo & 1);
  const int HW16 = (g.HW + 15) & ~15;
  const size_t plane = (size_t)HW16 * 32;
  const int slabs = g.C / 16;
  for (int ns = 2; ns >= 1; ns >>= 1) {  // four slabs would spill the accumulators
    if (ns > ns_cap || slabs % ns) continue;
    if (ns > 1 && (long long)(slabs / ns) * g.N < 148) continue;
    const int cg = 16 * ns;
    auto need = [&](int bh, int& warps) {
      warps = bh * NB;
      if (warps > 16) warps = 16;
      if (warps < 2) warps = 2;
      return ns * plane + (size_t)(36 + cg) * band_pitch(bh, Wpo) * 2 + (size_t)16 * (cg + 8) * 2 + (size_t)cg * kBankPitch * 2 +
             (size_t)warps * kCoordWarpWords * 4;
    };
    int bh_max = 0, wv;
    for (int bh = 1; bh <= g.Ho; ++bh) {
      if (need(bh, wv) > kOnePerSm) break;
      bh_max = bh;
    }
    if (!bh_max || (ns > 1 && bh_max * NB < 28 && bh_max < g.Ho)) continue;
    const int groups = slabs / ns;
    int bands = (g.Ho + bh_max - 1) / bh_max;
    const long long base_units = (long long)g.N * groups;
    if (base_units * bands < 148) {
      long long wantb = (148 + base_units - 1) / base_units;
      if (wantb > g.Ho) wantb = g.Ho;
      if (wantb > bands) bands = (int)wantb;
    }
    pl.NS = ns;
    pl.groups = groups;
    pl.BH = (g.Ho + bands - 1) / bands;
    pl.bands = (g.Ho + pl.BH - 1) / pl.BH;
    pl.smem = need(pl.BH, pl.warps);
    const long long units = (long long)g.N * pl.bands;
    long long want = 148 / groups;
    if (want > units) want = units;
    if (want < 1) want = 1;
    pl.units_per_block = (int)((units + want - 1) / want);
    pl.blocks_x = (int)((units + pl.units_per_block - 1) / pl.units_per_block);
    pl.ws_bytes = groups > 1 ? (size_t)g.N * 36 * g.P * sizeof(float) : 0;
    return pl;
  }
  return pl;
}

int slab_cap() {  // DK_B200_DCN_SLABS = 1, 2 or 4 caps the channel slabs per block (tuning knob)
  static const int cap = [] {
    const char* e = tuning_env("DK_B200_DCN_SLABS");
    const int v = e ? atoi(e) : 0;
    return (v == 1 || v == 2 || v == 4) ? v : 4;
  }();
  return cap;
}

}  // namespace

size_t deform_filter_mma_workspace(const Geom& g) {
  const DcnPlan pl = dcn_plan(g, 4, 1);  // the largest any cap can ask for is the one with the most blocks
  size_t need = pl.BH ? pl.ws_bytes : 0;
  for (int cap = 1; cap <= 2; ++cap) {
    const DcnPlan p2 = dcn_plan(g, cap, 1);
    if (p2.BH && p2.ws_bytes > need) need = p2.ws_bytes;
  }
  return need;
}

int deform_filter_mma(const __half* dy, const __half* x, const __half* off, const __half* rot, __half* dw, const Geom& g,
                      void* ws, size_t ws_bytes, cudaStream_t s) {
  DcnPlan pl = dcn_plan(g, slab_cap(), 1);
  if (!pl.BH || pl.smem > (size_t)device_smem_optin() || g.C / (16 * pl.NS) > 65535) return DK_ERR_UNSUPPORTED;
  if (ws == nullptr || ws_bytes < pl.ws_bytes) return DK_ERR_WORKSPACE;
  pl.mode_dy = ptr_mode(dy);
  pl.mode_rot = ptr_mode(rot);
  pl.mode_off = ptr_mode(off);
  pl.vec = (g.HW & 7) == 0 && ptr_mode(x) == 2;
  float* partial = reinterpret_cast<float*>(ws);
  const dim3 grid(pl.blocks_x, g.C / (16 * pl.NS));
  auto launch = [&](auto kern) -> int {
    if (int e = enable_smem(kern, pl.smem)) return e;
    kern<<<grid, pl.warps * 32, pl.smem, s>>>(dy, x, off, rot, partial, g, pl);
    return check_launch();
  };
  int rc;
#define DK_PICK(K, SS, ZZ) \
  (pl.NS == 4 ? launch(K<SS, 4, ZZ>) : pl.NS == 2 ? launch(K<SS, 2, ZZ>) : launch(K<SS, 1, ZZ>))
  if (rot)
    rc = g.sH == 1 ? DK_PICK(mma_deform_filter_kernel, 1, false) : DK_PICK(mma_deform_filter_kernel, 2, false);
  else
    rc = g.sH == 1 ? DK_PICK(mma_deform_filter_kernel, 1, true) : DK_PICK(mma_deform_filter_kernel, 2, true);
  if (rc) return rc;
  const int n_out = g.C * g.cells;
  reduce_dcn_bank_partials_kernel<<<(n_out + 7) / 8, 256, 0, s>>>(partial, dw, g.C, g.cells, pl.blocks_x);
  return check_launch();
}

int deform_forward_mma(const __half* x, const __half* off, const __half* rot, const __half* w, __half* y, const Geom& g,
                       cudaStream_t s) {
  DcnPlan pl = dcn_plan(g, slab_cap(), 0);
  if (!pl.BH || pl.smem > (size_t)device_smem_optin() || g.C / (16 * pl.NS) > 65535) return DK_ERR_UNSUPPORTED;
  pl.mode_rot = ptr_mode(rot);
  pl.mode_off = ptr_mode(off);
  pl.mode_dy = 0;
  pl.vec = (g.HW & 7) == 0 && ptr_mode(x) == 2;
  const dim3 grid(pl.blocks_x, g.C / (16 * pl.NS));
  auto launch = [&](auto kern) -> int {
    if (int e = enable_smem(kern, pl.smem)) return e;
    kern<<<grid, pl.warps * 32, pl.smem, s>>>(x, off, rot, w, y, g, pl);
    return check_launch();
  };
  if (rot) return g.sH == 1 ? DK_PICK(mma_deform_fwd_kernel, 1, false) : DK_PICK(mma_deform_fwd_kernel, 2, false);
  return g.sH == 1 ? DK_PICK(mma_deform_fwd_kernel, 1, true) : DK_PICK(mma_deform_fwd_kernel, 2, true);
}

size_t deform_data_mma_workspace(const Geom& g) { return ddata_plan(g).warps ? (size_t)g.N * sizeof(int) : 0; }

int deform_data_mma(const __half* dy, const __half* off, const __half* rot, const __half* w, __half* dx, const Geom& g,
                    void* ws, size_t ws_bytes, cudaStream_t s) {
  DDataPlan pl = ddata_plan(g);
  if (!pl.warps || pl.smem > (size_t)device_smem_optin() || g.C / 16 > 65535) return DK_ERR_UNSUPPORTED;
  if ((size_t)g.HW * sizeof(int) > 48 * 1024) return DK_ERR_UNSUPPORTED;
  if (ws == nullptr || ws_bytes < (size_t)g.N * sizeof(int)) return DK_ERR_WORKSPACE;
  int* hits = reinterpret_cast<int*>(ws);
  if (g.sH == 1) dcn_hit_count_kernel<1><<<g.N, 1024, (size_t)g.HW * sizeof(int), s>>>(off, hits, g);
  else dcn_hit_count_kernel<2><<<g.N, 1024, (size_t)g.HW * sizeof(int), s>>>(off, hits, g);
  if (int rc = check_launch()) return rc;
  pl.pair_dy = (g.Wo & 1) == 0 && ptr_mode(dy) >= 1 && ptr_mode(dx) >= 1;
  const dim3 grid(pl.blocks_x, g.C / 16);
  auto launch = [&](auto kern) -> int {
    if (int e = enable_smem(kern, pl.smem)) return e;
    kern<<<grid, pl.warps * 32, pl.smem, s>>>(dy, off, rot, w, hits, dx, g, pl);
    return check_launch();
  };
  if (rot) return g.sH == 1 ? launch(mma_deform_data_kernel<1, false>) : launch(mma_deform_data_kernel<2, false>);
  return g.sH == 1 ? launch(mma_deform_data_kernel<1, true>) : launch(mma_deform_data_kernel<2, true>);
}

size_t deform_coords_mma_workspace(const Geom& g) {
  size_t need = 0;
  for (int cap = 1; cap <= 2; cap <<= 1) {
    const DCoordPlan pl = dcoord_plan(g, cap);
    if (pl.BH && pl.ws_bytes > need) need = pl.ws_bytes;
  }
  return need;
}

// Partial bank gradients of the fused call below: [blocks][C][16] floats; 0 = the shape is not covered.
size_t deform_coords_bank_workspace(const Geom& g) {
  size_t need = 0;
  for (int cap = 1; cap <= 2; cap <<= 1) {
    const DCoordPlan pl = dcoord_plan(g, cap);
    const size_t b = pl.BH ? (size_t)pl.blocks_x * g.C * 16 * sizeof(float) : 0;
    if (b > need) need = b;
  }
  return need;
}

// dw != nullptr (with both offset gradients wanted, or the image-space one when rot == nullptr): the bank gradient is
// computed in the same pass from the products dy * xs; *bank_done tells the caller that dw has been written.
int deform_coords_mma(const __half* dy, const __half* x, const __half* off, const __half* rot, const __half* w, __half* doff,
                      __half* drot, const Geom& g, void* ws, size_t ws_bytes, cudaStream_t s, __half* dw, void* bank_ws,
                      size_t bank_ws_bytes, bool* bank_done) {
  if (bank_done) *bank_done = false;
  if (!doff && !drot) return DK_OK;
  if (!rot && drot) return DK_ERR_BAD_ARGUMENT;
  DCoordPlan pl = dcoord_plan(g, slab_cap());
  if (!pl.BH || pl.smem > (size_t)device_smem_optin() || g.C / (16 * pl.NS) > 65535) return DK_ERR_UNSUPPORTED;
  if (pl.ws_bytes && (ws == nullptr || ws_bytes < pl.ws_bytes)) return DK_ERR_UNSUPPORTED;  // no scratch: the SIMT kernel
  const bool with_bank = dw != nullptr && bank_done != nullptr && doff != nullptr && (drot != nullptr || !rot) && bank_ws != nullptr &&
                         bank_ws_bytes >= (size_t)pl.blocks_x * g.C * 16 * sizeof(float) &&
                         (size_t)pl.warps * 16 * pl.NS * 16 * sizeof(float) <= pl.smem;
  pl.mode_dy = ptr_mode(dy);
  pl.mode_rot = ptr_mode(rot);
  pl.mode_off = ptr_mode(off);
  pl.vec = (g.HW & 7) == 0 && ptr_mode(x) == 2;
  float* partial = reinterpret_cast<float*>(ws);
  if (pl.ws_bytes) {
    const cudaError_t e = cudaMemsetAsync(partial, 0, pl.ws_bytes, s);
    if (e != cudaSuccess) {
      set_last_cuda_error(e);
      return DK_ERR_CUDA;
    }
  }
  const dim3 grid(pl.blocks_x, g.C / (16 * pl.NS));
  float* bank_partial = reinterpret_cast<float*>(bank_ws);
  if (with_bank && pl.warps > 12) pl.warps = 12;
  auto launch = [&](auto kern) -> int {
    if (int e = enable_smem(kern, pl.smem)) return e;
    kern<<<grid, pl.warps * 32, pl.smem, s>>>(dy, x, off, rot, w, doff, drot, partial, bank_partial, g, pl);
    return check_launch();
  };
  int rc;
#define DK_COORDS(SS, NN)                                                                                      \
  (!rot ? (with_bank ? launch(mma_deform_coords_kernel<SS, NN, true, false, true, true>)                       \
                     : launch(mma_deform_coords_kernel<SS, NN, true, false, true, false>))                     \
        : doff && drot ? (with_bank ? launch(mma_deform_coords_kernel<SS, NN, true, true, false, true>)        \
                                    : launch(mma_deform_coords_kernel<SS, NN, true, true, false, false>))      \
                       : doff ? launch(mma_deform_coords_kernel<SS, NN, true, false, false, false>)            \
                              : launch(mma_deform_coords_kernel<SS, NN, false, true, false, false>))
  if (g.sH == 1)
    rc = pl.NS == 2 ? DK_COORDS(1, 2) : DK_COORDS(1, 1);
  else
    rc = pl.NS == 2 ? DK_COORDS(2, 2) : DK_COORDS(2, 1);
#undef DK_COORDS
  if (rc) return rc;
  if (with_bank) {
    const int n_out = g.C * g.cells;
    reduce_dcn_bank_partials_kernel<<<(n_out + 7) / 8, 256, 0, s>>>(bank_partial, dw, g.C, g.cells, pl.blocks_x);
    if ((rc = check_launch())) return rc;
    *bank_done = true;
  }
  if (!pl.ws_bytes) return rc;
  const size_t plane18 = (size_t)18 * g.P, count = (size_t)g.N * plane18;
  const unsigned blocks = (unsigned)((count + 255) / 256);
  if (doff) round_coord_partials_kernel<<<blocks, 256, 0, s>>>(partial, doff, g.N, plane18, 0);
  if (drot) round_coord_partials_kernel<<<blocks, 256, 0, s>>>(partial, drot, g.N, plane18, 18);
  return check_launch();
}

}  // namespace dk
