// fp16 tensor-core paths of the DK + DCN operator: forward and bank gradient.
//
// y[c, p]      = sum over taps of K[c, p, tap] * xs[c, p, tap],          K = W * beta^T
// dW[c, cell]  = sum over (sample, pixel, tap) of dy[c, p] * xs[c, p, tap] * beta[(p, tap), cell]
// where beta are the hat products of the bank coordinate (see dk_local_mma.cu) and xs is the bilinear image
// sample at the tap's deformed position: four data-dependent reads per (pixel, tap, channel).  A block keeps the
// WHOLE input plane of its channels in shared memory, so those reads never leave the SM, and builds, three taps
// at a time, a table of (byte offset, coefficient) x 4 corners per (pixel, tap) that all its channels reuse.
// The two products with beta are mma.sync.m16n8k16 as for the local operator.
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
// The forward keeps its input planes as 32-bit words (channel j | channel j + 8 << 16), eight words per pixel
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
template <int S>
__device__ __forceinline__ void build_pair_table(unsigned* __restrict__ tab, const __half* __restrict__ oband, const Band& bo,
                                                 const Geom& g, int fh, int oh, int ow0, int lane) {
  if (lane < 24) {
    const int px = lane & 7, fw = lane >> 3;
    const int pc = ow0 + px;
    const int t = fh * 3 + fw;
    const __half* op = oband + (size_t)(2 * t) * bo.pitch_c + kSlack + oh * bo.Wp + pc - bo.org;
    const float ph = (float)(oh * S - 1 + fh) + __half2float(op[0]);
    const float pw = (float)(pc * S - 1 + fw) + __half2float(op[bo.pitch_c]);
    const bool used = pc < g.Wo && ph > -1.f && pw > -1.f && ph < (float)g.H && pw < (float)g.W;
    uint4 o4 = make_uint4(0, 0, 0, 0), c4 = make_uint4(0, 0, 0, 0);
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
      c4.x = (r0 && k0) ? pack2(hh * hw, hh * hw) : 0u;
      c4.y = (r0 && k1) ? pack2(hh * lw, hh * lw) : 0u;
      c4.z = (r1 && k0) ? pack2(lh * hw, lh * hw) : 0u;
      c4.w = (r1 && k1) ? pack2(lh * lw, lh * lw) : 0u;
    }
    uint4* e = reinterpret_cast<uint4*>(tab + fw * 80 + (px >> 1) * 20 + (px & 1) * 8);
    e[0] = o4;
    e[1] = c4;
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

struct DcnPlan {
  int NS, BH, warps, bands, units_per_block, blocks_x;
  int mode_rot, mode_off, mode_dy;
  bool vec;
  size_t smem, ws_bytes;
};

// y[c, p] = sum over taps of K[c, p, tap] * xs[c, p, tap]:  K = W * beta^T from one mma per tap (as in the local
// forward), xs sampled from the channel-pair planes.  A block owns 16 * NS channels and walks over units
// (sample, band of output rows); the planes are reloaded only when the sample changes.
template <int S, int NS>
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
  int cur_n = -1;
  for (int unit = u_begin; unit < u_end; ++unit) {
    const int n = unit / pl.bands;
    const int oh0 = (unit - n * pl.bands) * pl.BH;
    const Band br = make_band(oh0, pl.BH, g.Ho, g.Wo, pl.mode_rot);
    const Band bo = make_band(oh0, pl.BH, g.Ho, g.Wo, pl.mode_off);
    __syncthreads();  // readers of the previous unit are done
    load_band(rband, br, rot, n, 18, 0, 18, g.Ho, g.Wo);
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
      unsigned bf[9][2];
      beta_direct<S, false, false>(bf, rband, br, g, lc, sc44, oh, ow0, g.H, g.W, g.Wo, gq);
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
template <int S, int NS>
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
    load_band(rband, br, rot, n, 18, 0, 18, g.Ho, g.Wo);
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
      unsigned bw[9][2];  // beta as B fragments: [tap][cells 0-7 | cells 8-15]
      {
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
    if (!bh_max || (ns > 1 && bh_max * NB < 32 && bh_max < g.Ho)) continue;  // short bands: the per-unit cost eats the gain
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

int slab_cap() {  // DK_B200_DCN_SLABS = 1, 2 or 4 caps the channel slabs per block (tuning knob)
  static const int cap = [] {
    const char* e = getenv("DK_B200_DCN_SLABS");
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
  if (g.sH == 1)
    rc = pl.NS == 4 ? launch(mma_deform_filter_kernel<1, 4>) : pl.NS == 2 ? launch(mma_deform_filter_kernel<1, 2>)
                                                                        : launch(mma_deform_filter_kernel<1, 1>);
  else
    rc = pl.NS == 4 ? launch(mma_deform_filter_kernel<2, 4>) : pl.NS == 2 ? launch(mma_deform_filter_kernel<2, 2>)
                                                                        : launch(mma_deform_filter_kernel<2, 1>);
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
  if (g.sH == 1)
    return pl.NS == 4 ? launch(mma_deform_fwd_kernel<1, 4>) : pl.NS == 2 ? launch(mma_deform_fwd_kernel<1, 2>)
                                                                        : launch(mma_deform_fwd_kernel<1, 1>);
  return pl.NS == 4 ? launch(mma_deform_fwd_kernel<2, 4>) : pl.NS == 2 ? launch(mma_deform_fwd_kernel<2, 2>)
                                                                      : launch(mma_deform_fwd_kernel<2, 1>);
}

}  // namespace dk
