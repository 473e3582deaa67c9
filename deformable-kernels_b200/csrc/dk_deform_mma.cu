// fp16 tensor-core path of the DK + DCN bank gradient.
//
// dW[c, cell] = sum over (sample, pixel, tap) of dy[c,p] * xs[c,p,tap] * beta[(p,tap), cell], where xs is
// the bilinear image sample at the tap's deformed position and beta the hat products of the bank
// coordinate (see dk_local_mma.cu).  As for the local operator the sum over (pixel, tap) is an
// mma.sync.m16n8k16 with dK = dy * xs as the A operand; what is new is xs: four data-dependent
// reads per (pixel, tap, channel).  A block keeps the WHOLE input plane of its 16 channels in
// shared memory, so those reads never leave the SM, and builds, three taps at a time, a table of
// (byte offset, coefficient) x 4 corners per (pixel, tap) that every channel of the slab reuses.
//
// Covers fp16, 3x3, pad 1, dilation 1, stride 1 or 2, one rotation group, <= 16 bank cells,
// C % 16 == 0 and planes small enough for 16 of them to fit on chip (56 x 56 and below).
#include <cstdlib>

#include "dk_mma_common.cuh"

namespace dk {

using namespace mma;

namespace {

constexpr size_t kOnePerSm = 226 * 1024;

struct DFPlan {
  int BH, warps, bands, units_per_block, blocks_x;
  int mode_x, mode_dy, mode_rot, mode_off;
  size_t smem, ws_bytes;
};

constexpr int kTabWords = 24 * 8;  // 3 taps x 8 pixels x (4 byte offsets + 4 coefficients)

// image sample of one (pixel, tap) for one channel plane: sum of coefficient * value over the four corners
__device__ __forceinline__ float sample4(const __half* __restrict__ plane, const uint4 o, const uint4 cf) {
  const char* base = reinterpret_cast<const char*>(plane);
  float a = 0.f;
  fma_hh<0, 0>(a, (unsigned)*reinterpret_cast<const unsigned short*>(base + o.x), cf.x);
  fma_hh<0, 0>(a, (unsigned)*reinterpret_cast<const unsigned short*>(base + o.y), cf.y);
  fma_hh<0, 0>(a, (unsigned)*reinterpret_cast<const unsigned short*>(base + o.z), cf.z);
  fma_hh<0, 0>(a, (unsigned)*reinterpret_cast<const unsigned short*>(base + o.w), cf.w);
  return a;
}

__device__ __forceinline__ unsigned half_bits(float v) { return (unsigned)__half_as_ushort(__float2half_rn(v)); }

template <int S, int MAXT>
__global__ void __launch_bounds__(MAXT, 1) mma_deform_filter_kernel(const __half* __restrict__ dy, const __half* __restrict__ x,
                                                                   const __half* __restrict__ off, const __half* __restrict__ rot,
                                                                   float* __restrict__ partial, const Geom g, const DFPlan pl) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int c0 = blockIdx.y * 16;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int gq = lane >> 2, q = lane & 3;
  const int NB = (g.Wo + 7) >> 3;
  const int items = pl.BH * NB;
  const int Wpo = g.Wo + (g.Wo & 1);
  const Band bxp = make_band(0, g.H, g.H, g.W, pl.mode_x);  // the whole input plane
  const int ypitch = band_pitch(pl.BH, Wpo);

  __half* xpl = reinterpret_cast<__half*>(smem_raw);           // [16][bxp.pitch_c]
  __half* yband = xpl + (size_t)16 * bxp.pitch_c;               // [16][ypitch]
  __half* rband = yband + (size_t)16 * ypitch;                  // [18][ypitch]
  __half* oband = rband + (size_t)18 * ypitch;                  // [18][ypitch]
  unsigned* tab = reinterpret_cast<unsigned*>(oband + (size_t)18 * ypitch) + warp * kTabWords;
  const LaneCells lc = lane_cells(g, q);
  const bool sc44 = g.scH == 4 && g.scW == 4;

  float acc[2][4];
#pragma unroll
  for (int k = 0; k < 4; ++k) acc[0][k] = acc[1][k] = 0.f;

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
    if (n != cur_n) {
      load_band(xpl, bxp, x, n, g.C, c0, 16, g.H, g.W);
      cur_n = n;
    }
    load_band(yband, by, dy, n, g.C, c0, 16, g.Ho, g.Wo);
    load_band(rband, br, rot, n, 18, 0, 18, g.Ho, g.Wo);
    load_band(oband, bo, off, n, 18, 0, 18, g.Ho, g.Wo);
    cp_async_wait_all();
    __syncthreads();

    for (int item = warp; item < items; item += nwarps) {
      const int dr = item / NB;
      const int oh = oh0 + dr;
      if (oh >= g.Ho) break;
      const int ow0 = (item - dr * NB) << 3;
      unsigned bw[10][2];
      {
        unsigned bf[9][2];
        beta_direct<S, false, false>(bf, rband, br, g, lc, sc44, oh, ow0, g.H, g.W, g.Wo, gq);
#pragma unroll
        for (int t = 0; t < 9; ++t) {
          bw[t][0] = movmatrix_trans(bf[t][0]);
          bw[t][1] = movmatrix_trans(bf[t][1]);
        }
        bw[9][0] = bw[9][1] = 0u;
      }
      const int ow = ow0 + 2 * q;
      const int yoff = kSlack + oh * by.Wp + ow - by.org;
      const unsigned dy0 = *reinterpret_cast<const unsigned*>(yband + (size_t)gq * by.pitch_c + yoff);
      const unsigned dy1 = *reinterpret_cast<const unsigned*>(yband + (size_t)(gq + 8) * by.pitch_c + yoff);
      const __half* plA = xpl + (size_t)gq * bxp.pitch_c;
      const __half* plB = plA + (size_t)8 * bxp.pitch_c;
      unsigned dk0[10], dk1[10];
      dk0[9] = dk1[9] = 0u;
#pragma unroll
      for (int fh = 0; fh < 3; ++fh) {
        __syncwarp();
        if (lane < 24) {
          // sampling table of (pixel px, tap (fh, fw)): byte offsets and coefficients of the four image corners
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
            const int base = kSlack - bxp.org;
            const int h0c = max(h0, 0), h1c = min(h0 + 1, g.H - 1), w0c = max(w0, 0), w1c = min(w0 + 1, g.W - 1);
            o4.x = (unsigned)(base + h0c * bxp.Wp + w0c) * 2u;
            o4.y = (unsigned)(base + h0c * bxp.Wp + w1c) * 2u;
            o4.z = (unsigned)(base + h1c * bxp.Wp + w0c) * 2u;
            o4.w = (unsigned)(base + h1c * bxp.Wp + w1c) * 2u;
            c4.x = (r0 && k0) ? half_bits(hh * hw) : 0u;
            c4.y = (r0 && k1) ? half_bits(hh * lw) : 0u;
            c4.z = (r1 && k0) ? half_bits(lh * hw) : 0u;
            c4.w = (r1 && k1) ? half_bits(lh * lw) : 0u;
          }
          uint4* e = reinterpret_cast<uint4*>(tab + (fw * 8 + px) * 8);
          e[0] = o4;
          e[1] = c4;
        }
        __syncwarp();
#pragma unroll
        for (int fw = 0; fw < 3; ++fw) {
          const uint4* e0 = reinterpret_cast<const uint4*>(tab + (fw * 8 + 2 * q) * 8);
          const uint4 oA = e0[0], cA = e0[1], oB = e0[2], cB = e0[3];  // pixel 2q, pixel 2q + 1
          const float a0 = sample4(plA, oA, cA), a1 = sample4(plA, oB, cB);
          const float b0 = sample4(plB, oA, cA), b1 = sample4(plB, oB, cB);
          dk0[fh * 3 + fw] = hmul2u(dy0, pack2(a0, a1));
          dk1[fh * 3 + fw] = hmul2u(dy1, pack2(b0, b1));
        }
      }
#pragma unroll
      for (int j = 0; j < 5; ++j) {
        mma16816_acc(acc[0], dk0[2 * j], dk1[2 * j], dk0[2 * j + 1], dk1[2 * j + 1], bw[2 * j][0], bw[2 * j + 1][0]);
        mma16816_acc(acc[1], dk0[2 * j], dk1[2 * j], dk0[2 * j + 1], dk1[2 * j + 1], bw[2 * j][1], bw[2 * j + 1][1]);
      }
    }
  }
  // reduce the warps' accumulators and write this block's partial bank gradient [16 channels][16 cells]
  __syncthreads();
  float* red = reinterpret_cast<float*>(smem_raw);  // [nwarps][16][16]
  {
    float* r0 = red + ((size_t)warp * 16 + gq) * 16;
    float* r1 = r0 + 8 * 16;
    r0[2 * q] = acc[0][0]; r0[2 * q + 1] = acc[0][1];
    r1[2 * q] = acc[0][2]; r1[2 * q + 1] = acc[0][3];
    r0[8 + 2 * q] = acc[1][0]; r0[8 + 2 * q + 1] = acc[1][1];
    r1[8 + 2 * q] = acc[1][2]; r1[8 + 2 * q + 1] = acc[1][3];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 256; i += blockDim.x) {
    float sum = 0.f;
    for (int wv = 0; wv < nwarps; ++wv) sum += red[(size_t)wv * 256 + i];
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

// Warps per block: 14 keep the whole working set in registers; 24 (80 registers, a few spilled words)
// hide more of the shared-memory latency of the sampling reads.  DK_B200_DCN_FILT_WARPS overrides.
int df_max_warps() {
  static const int v = [] {
    const char* e = getenv("DK_B200_DCN_FILT_WARPS");
    const int w = e ? atoi(e) : 0;
    return (w >= 2 && w <= 24) ? w : 14;
  }();
  return v;
}

DFPlan df_plan(const Geom& g) {
  DFPlan pl;
  pl.BH = 0;
  if (!dcn_fast_shape(g)) return pl;
  const int NB = (g.Wo + 7) / 8;
  const int Wp = g.W + (g.W & 1), Wpo = g.Wo + (g.Wo & 1);
  const size_t xbytes = (size_t)16 * band_pitch(g.H, Wp) * 2;
  const int groups = g.C / 16;
  auto need = [&](int bh, int& warps) {
    warps = bh * NB;
    if (warps > df_max_warps()) warps = df_max_warps();
    if (warps < 2) warps = 2;
    size_t smem = xbytes + (size_t)(16 + 36) * band_pitch(bh, Wpo) * 2 + (size_t)warps * kTabWords * 4;
    const size_t red = (size_t)warps * 256 * 4;
    return smem < red ? red : smem;
  };
  // tallest band of output rows that fits beside the planes: the per-unit load latency is paid once per band
  int bh_max = 0, w;
  for (int bh = 1; bh <= g.Ho; ++bh) {
    if (need(bh, w) > kOnePerSm) break;
    bh_max = bh;
  }
  if (!bh_max) return pl;
  int bands = (g.Ho + bh_max - 1) / bh_max;
  // few samples: cut the rows finer so that every SM gets a unit
  const long long base_units = (long long)g.N * groups;
  if (base_units * bands < 148) {
    long long wantb = (148 + base_units - 1) / base_units;
    if (wantb > g.Ho) wantb = g.Ho;
    if (wantb > bands) bands = (int)wantb;
  }
  pl.BH = (g.Ho + bands - 1) / bands;
  pl.bands = (g.Ho + pl.BH - 1) / pl.BH;
  pl.smem = need(pl.BH, pl.warps);
  const long long units = (long long)g.N * pl.bands;
  // one block per SM (the planes fill its shared memory): a single wave over all channel groups
  long long want = 148 / groups;
  if (want > units) want = units;
  if (want < 1) want = 1;
  pl.units_per_block = (int)((units + want - 1) / want);
  pl.blocks_x = (int)((units + pl.units_per_block - 1) / pl.units_per_block);
  pl.ws_bytes = (size_t)pl.blocks_x * g.C * 16 * sizeof(float);
  return pl;
}

}  // namespace

size_t deform_filter_mma_workspace(const Geom& g) {
  const DFPlan pl = df_plan(g);
  return pl.BH ? pl.ws_bytes : 0;
}

int deform_filter_mma(const __half* dy, const __half* x, const __half* off, const __half* rot, __half* dw, const Geom& g,
                      void* ws, size_t ws_bytes, cudaStream_t s) {
  DFPlan pl = df_plan(g);
  if (!pl.BH || pl.smem > (size_t)device_smem_optin() || g.C / 16 > 65535) return DK_ERR_UNSUPPORTED;
  if (ws == nullptr || ws_bytes < pl.ws_bytes) return DK_ERR_WORKSPACE;
  pl.mode_x = ptr_mode(x);
  pl.mode_dy = ptr_mode(dy);
  pl.mode_rot = ptr_mode(rot);
  pl.mode_off = ptr_mode(off);
  float* partial = reinterpret_cast<float*>(ws);
  int rc;
  const dim3 grid(pl.blocks_x, g.C / 16);
  auto launch = [&](auto kern) -> int {
    if (int e = enable_smem(kern, pl.smem)) return e;
    kern<<<grid, pl.warps * 32, pl.smem, s>>>(dy, x, off, rot, partial, g, pl);
    return 0;
  };
  if (pl.warps <= 14)
    rc = g.sH == 1 ? launch(mma_deform_filter_kernel<1, 448>) : launch(mma_deform_filter_kernel<2, 448>);
  else
    rc = g.sH == 1 ? launch(mma_deform_filter_kernel<1, 768>) : launch(mma_deform_filter_kernel<2, 768>);
  if (rc) return rc;
  if ((rc = check_launch())) return rc;
  const int n_out = g.C * g.cells;
  reduce_dcn_bank_partials_kernel<<<(n_out + 7) / 8, 256, 0, s>>>(partial, dw, g.C, g.cells, pl.blocks_x);
  return check_launch();
}

}  // namespace dk
