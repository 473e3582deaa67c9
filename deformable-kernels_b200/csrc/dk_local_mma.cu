// fp16 fast path of the local deformable kernel on the tensor cores.
//
// Zero-extended bilinear sampling of a bank equals a contraction with hat functions:
//   B(W[c]; u, v) = sum_{a,b} W[c,a,b] * hat(u - a) * hat(v - b),   hat(t) = max(0, 1 - |t|)
// (two of the hats per axis are non-zero, all vanish when u <= -1 or u >= scope: the
// reference's validity rule, csrc/filter_sample_depthwise_cuda_kernel.cu:59).  The hat products
// beta[(pixel, tap), cell] do not depend on the channel, which turns the three expensive parts
// of the operator into small dense products over the 16 bank cells / 16 channels / 16 (pixel,
// tap) pairs, each one mma.sync.m16n8k16 (fp16 in, fp32 accumulate):
//   forward, grad-input   K[16 ch x 8 px]       = W[16 ch x 16 cells]  * beta^T[16 cells x 8 px]
//                         y[c,p] += x[c,p+tap] * K[c,p]                     (1 FMA per pixel, tap, channel)
//   grad-bank             dW[16 ch x 16 cells] += dK[16 ch x 16 (px,tap)] * beta[16 (px,tap) x 16 cells]
//   grad-offsets          G^T[16 cells x 8 px] += W^T[16 cells x 16 ch]  * dK[16 ch x 8 px]
//                         d(offset)[p,tap] = sum_cell G[p,tap,cell] * d(beta)/d(u or v)   (4 corners)
// with dK[c,(p,tap)] = dy[c,p] * x[c,p+tap].  The SIMT formulation needs four gathered bank
// values and five FMAs per (pixel, tap, channel) and is bound by instruction issue.
//
// Covers: fp16, 3x3 kernel, dilation 1, pad 1, stride 1 or 2 (equal in h and w), one rotation
// group, at most 16 bank cells, channels a multiple of 16.
// Everything else stays on the SIMT kernels of dk_local.cu.
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "dk_mma_common.cuh"

namespace dk {

using namespace mma;

namespace {

// Block shapes are searched once per (geometry, pass) and remembered: the latency-bound small calls would otherwise pay
// the search on every launch.  (Builds with -DDK_TUNING, whose knobs can change between calls, search every time.)
template <typename Plan, typename F>
Plan cached_plan(const Geom& g, int tag, F compute) {
#ifdef DK_TUNING
  (void)tag;
  return compute();
#else
  struct Entry {
    Geom g;
    int tag;
    Plan pl;
  };
  static std::mutex mu;
  static std::vector<Entry> cache;
  {
    std::lock_guard<std::mutex> lock(mu);
    for (const Entry& e : cache)
      if (e.tag == tag && std::memcmp(&e.g, &g, sizeof(Geom)) == 0) return e.pl;
  }
  const Plan pl = compute();
  std::lock_guard<std::mutex> lock(mu);
  if (cache.size() < 256) cache.push_back(Entry{g, tag, pl});
  return pl;
#endif
}

// ================================================================== forward / grad-input
struct ConvPlan {
  int BH, CG, groups, warps, bands;
  int mode_src, mode_rot;  // copy widths the base pointers allow
  bool pair_store;         // destination rows are even and the pointer is 4-byte aligned
  size_t smem;
};

// source rows a band of BH destination rows needs
__host__ __device__ inline int conv_band_rows(int bh, int S, bool transposed) {
  if (!transposed) return (bh - 1) * S + 3;
  return S == 1 ? bh + 2 : (bh >> 1) + 2;
}

template <int S, bool TRANSPOSED>
__global__ void __launch_bounds__(448, 2) mma_conv_kernel(const __half* __restrict__ src, const __half* __restrict__ rot,
                                                          const __half* __restrict__ w, __half* __restrict__ dst, const Geom g,
                                                          const ConvPlan pl) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int Hd = TRANSPOSED ? g.H : g.Ho, Wd = TRANSPOSED ? g.W : g.Wo;
  const int Hs = TRANSPOSED ? g.Ho : g.H, Ws = TRANSPOSED ? g.Wo : g.W;
  const int n = blockIdx.z;
  const int c0 = blockIdx.y * pl.CG;
  const int cnt = min(pl.CG, g.C - c0);
  const int d_row0 = blockIdx.x * pl.BH;
  const int RB = conv_band_rows(pl.BH, S, TRANSPOSED);
  const int src_row_lo = TRANSPOSED ? (S == 1 ? d_row0 - 1 : d_row0 >> 1) : d_row0 * S - 1;
  const Band bx = make_band(src_row_lo, RB, Hs, Ws, pl.mode_src);
  // offset planes: the rows of the output pixels whose offsets drive the band's taps
  const Band br = TRANSPOSED ? make_band(src_row_lo, RB, g.Ho, g.Wo, pl.mode_rot)
                             : make_band(d_row0, pl.BH, g.Ho, g.Wo, pl.mode_rot);

  __half* band = reinterpret_cast<__half*>(smem_raw);
  __half* rband = band + pl.CG * bx.pitch_c;                                 // [18][br.pitch_c]
  __half* bank = rband + 18 * br.pitch_c;                                    // [CG][kBankPitch]

  for (int i = threadIdx.x; i < cnt * 16; i += blockDim.x) {
    const int j = i >> 4, cell = i & 15;
    bank[j * kBankPitch + cell] = cell < g.cells ? __ldg(w + (size_t)(c0 + j) * g.cells + cell) : __float2half(0.f);
  }
  load_band(band, bx, src, n, g.C, c0, cnt, Hs, Ws);
  load_band(rband, br, rot, n, 18, 0, 18, g.Ho, g.Wo);
  cp_async_wait_all();
  __syncthreads();

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int gq = lane >> 2, q = lane & 3;
  const int NB = (Wd + 7) >> 3;
  const int items = pl.BH * NB;
  const bool dst_even = pl.pair_store;
  const LaneCells lc = lane_cells(g, q);
  const bool sc44 = g.scH == 4 && g.scW == 4;

  for (int item = warp; item < items; item += nwarps) {
    const int dr = item / NB;
    const int drow = d_row0 + dr;
    if (drow >= Hd) break;
    const int ow0 = (item - dr * NB) << 3;
    unsigned bf[9][2];
    beta_direct<S, TRANSPOSED>(bf, rband, br, g, lc, sc44, drow, ow0, Hs, Ws, Wd, gq);

    const int ow = ow0 + 2 * q;
    // TRANSPOSED with stride 2: pixel 0 (even column) takes tap column 1 from grad-output column ow/2,
    // pixel 1 takes tap columns 0 and 2 from columns ow/2 + 1 and ow/2; only tap rows of matching parity count.
    const int j0 = ow >> 1;
    const int wbase = (TRANSPOSED && S == 2) ? kSlack + (j0 & ~1) - bx.org
                                             : window_offset(bx, TRANSPOSED ? drow - 1 : drow * S - 1, ow, S);
    const unsigned* bkp = reinterpret_cast<const unsigned*>(bank + gq * kBankPitch) + q;
    const __half* x0 = band + gq * bx.pitch_c + wbase;
    const int xstep = 16 * bx.pitch_c, x8 = 8 * bx.pitch_c;
    const size_t dplane = (size_t)Hd * Wd;
    __half* y0 = dst + ((size_t)n * g.C + c0 + gq) * dplane + (size_t)drow * Wd + ow;
#pragma unroll 2
    for (int cb16 = 0; cb16 < cnt; cb16 += 16, bkp += 16 * kBankPitch / 2, x0 += xstep, y0 += 16 * dplane) {
      unsigned a[4];
      a[0] = bkp[0];
      a[1] = bkp[8 * kBankPitch / 2];
      a[2] = bkp[4];
      a[3] = bkp[8 * kBankPitch / 2 + 4];
      const __half* x1 = x0 + x8;
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      if (TRANSPOSED && S == 2) {
        const unsigned sel = (j0 & 1) ? 0x5432u : 0x3210u;  // -> (dy[j0], dy[j0 + 1]) in one word
#pragma unroll
        for (int fh = 0; fh < 3; ++fh) {
          const int tr = drow + 1 - fh;
          if (tr < 0 || (tr & 1)) continue;  // uniform over the warp
          const int orow = tr >> 1;
          const unsigned* p0 = reinterpret_cast<const unsigned*>(x0 + orow * bx.Wp);
          const unsigned* p1 = reinterpret_cast<const unsigned*>(x1 + orow * bx.Wp);
          const unsigned ab0 = __byte_perm(p0[0], p0[1], sel), ab1 = __byte_perm(p1[0], p1[1], sel);
          unsigned d[2];
          mma16816_h(d, a, bf[fh * 3 + 0][0], bf[fh * 3 + 0][1]);
          fma_hh<1, 1>(acc[1], ab0, d[0]);
          fma_hh<1, 1>(acc[3], ab1, d[1]);
          mma16816_h(d, a, bf[fh * 3 + 1][0], bf[fh * 3 + 1][1]);
          fma_hh<0, 0>(acc[0], ab0, d[0]);
          fma_hh<0, 0>(acc[2], ab1, d[1]);
          mma16816_h(d, a, bf[fh * 3 + 2][0], bf[fh * 3 + 2][1]);
          fma_hh<0, 1>(acc[1], ab0, d[0]);
          fma_hh<0, 1>(acc[3], ab1, d[1]);
        }
      } else {
#pragma unroll
        for (int fh = 0; fh < 3; ++fh) {
          const int rsel = TRANSPOSED ? 2 - fh : fh;
          const unsigned* p0 = reinterpret_cast<const unsigned*>(x0 + rsel * bx.Wp);
          const unsigned* p1 = reinterpret_cast<const unsigned*>(x1 + rsel * bx.Wp);
          const unsigned w0 = p0[0], w1 = p0[1], w2 = p0[2];
          const unsigned v0 = p1[0], v1 = p1[1], v2 = p1[2];
          unsigned d[3][2];
#pragma unroll
          for (int fw = 0; fw < 3; ++fw) mma16816_h(d[fw], a, bf[fh * 3 + fw][0], bf[fh * 3 + fw][1]);
          // tap column fw reads window half 1 + c (pixel 0) and 1 + S + c (pixel 1), c = fw (forward) or 2 - fw
          constexpr int C0 = TRANSPOSED ? 2 : 0, C1 = 1, C2 = TRANSPOSED ? 0 : 2;
          fma_win<1 + C0, 0>(acc[0], w0, w1, w2, d[0][0]);
          fma_win<1 + S + C0, 1>(acc[1], w0, w1, w2, d[0][0]);
          fma_win<1 + C0, 0>(acc[2], v0, v1, v2, d[0][1]);
          fma_win<1 + S + C0, 1>(acc[3], v0, v1, v2, d[0][1]);
          fma_win<1 + C1, 0>(acc[0], w0, w1, w2, d[1][0]);
          fma_win<1 + S + C1, 1>(acc[1], w0, w1, w2, d[1][0]);
          fma_win<1 + C1, 0>(acc[2], v0, v1, v2, d[1][1]);
          fma_win<1 + S + C1, 1>(acc[3], v0, v1, v2, d[1][1]);
          fma_win<1 + C2, 0>(acc[0], w0, w1, w2, d[2][0]);
          fma_win<1 + S + C2, 1>(acc[1], w0, w1, w2, d[2][0]);
          fma_win<1 + C2, 0>(acc[2], v0, v1, v2, d[2][1]);
          fma_win<1 + S + C2, 1>(acc[3], v0, v1, v2, d[2][1]);
        }
      }
      if (ow < Wd) {
        __half* y1 = y0 + 8 * dplane;
        if (dst_even) {
          *reinterpret_cast<__half2*>(y0) = __floats2half2_rn(acc[0], acc[1]);
          *reinterpret_cast<__half2*>(y1) = __floats2half2_rn(acc[2], acc[3]);
        } else {
          y0[0] = __float2half_rn(acc[0]);
          y1[0] = __float2half_rn(acc[2]);
          if (ow + 1 < Wd) {
            y0[1] = __float2half_rn(acc[1]);
            y1[1] = __float2half_rn(acc[3]);
          }
        }
      }
    }
  }
}

// shared memory per block that still lets two blocks share an SM (228 KB per SM, 1 KB reserved per block)
constexpr size_t kTwoPerSm = 113 * 1024;
constexpr size_t kOnePerSm = 226 * 1024;

bool fast_shape(const Geom& g) {
  if (g.kH != 3 || g.kW != 3 || g.dH != 1 || g.dW != 1 || g.pH != 1 || g.pW != 1) return false;
  if (g.sH != g.sW || (g.sH != 1 && g.sH != 2)) return false;
  if (g.G != 1 || g.cells > 16 || (g.C & 15) || g.N > 65535) return false;
  return true;
}

int pick_warps(int items, int maxw) {
  if (items <= 2) return 2;
  if (items < 4) return items;
  int bw = maxw, bwaste = 1 << 30;
  for (int wv = maxw; wv >= 4; --wv) {
    const int waste = ((items + wv - 1) / wv) * wv - items;
    if (waste < bwaste) { bwaste = waste; bw = wv; }
  }
  return bw;
}

// Share of the GPU's block slots that a grid of ctas blocks keeps busy, bpsm blocks resident per SM.  Up to three waves the
// last, partly filled one costs a whole wave; with more, blocks of later waves start as earlier ones finish and it costs
// about half its gap.
double wave_fill(long long ctas, int bpsm) {
  const long long slots = 148LL * bpsm;
  const double exact = (double)ctas / (double)slots;
  const double whole = (double)((ctas + slots - 1) / slots);
  return exact / (exact + (whole - exact) * (whole <= 3.0 ? 1.0 : 0.5));
}

// Shared memory of a forward / grad-input block.
size_t conv_smem(const Geom& g, bool transposed, int cg, int bh) {
  const int S = g.sH;
  const int Ws = transposed ? g.Wo : g.W;
  const int Wp = Ws + (Ws & 1), Wpo = g.Wo + (g.Wo & 1);
  const int rb = conv_band_rows(bh, S, transposed);
  return (size_t)cg * band_pitch(rb, Wp) * 2 + (size_t)18 * band_pitch(transposed ? rb : bh, Wpo) * 2 +
         (size_t)cg * kBankPitch * 2;
}

// Channel group, band height and warps per block are chosen together by an estimate of the time per output row.
ConvPlan conv_plan_search(const Geom& g, bool transposed) {
  ConvPlan pl;
  const int S = g.sH;
  const int Hd = transposed ? g.H : g.Ho, Wd = transposed ? g.W : g.Wo;
  const int NB = (Wd + 7) / 8;
  int cg_only = 0, cap = Hd;
  size_t budget = kTwoPerSm;
  if (const char* e = tuning_env("DK_B200_CONV_CG")) cg_only = atoi(e) > 0 ? atoi(e) : 0;        // tuning knobs
  if (const char* e = tuning_env("DK_B200_CONV_BH")) cap = atoi(e) > 0 ? atoi(e) : cap;
  if (const char* e = tuning_env("DK_B200_CONV_SMEM_KB")) budget = (size_t)atoi(e) * 1024;
  static const int kCgMax[] = {64, 96, 128, 192, 256, 320, 480};
  double best_cost = 1e30;
  pl.BH = 0;
  for (int ci = 0; ci < 7; ++ci) {
    const int cgmax = cg_only ? cg_only : kCgMax[ci];
    const int ngrp = (g.C + cgmax - 1) / cgmax;
    const int cg = (((g.C + ngrp - 1) / ngrp) + 15) & ~15;
    const int groups = (g.C + cg - 1) / cg;
    // Estimated time per output, in instructions per item and channel slab; only ratios matter:
    //   (hat products / slabs + work per slab) / (share of warp slots with an item x occupancy)   -- issue-bound part
    //   + halves staged per output (rows of the group's channels, the 18 offset planes)            -- not overlapped
    // over the share of block slots kept busy and the share of the last band's rows that exist.
    // Constants from timing block shapes on 112 x 112 ... 7 x 7 planes with 96 ... 960 channels: blocks whose item count
    // is a multiple of their warps at 28 resident warps per SM beat blocks with no idle warp slot but 14 resident warps
    // by 10 %.
    const double per_item = 250.0 / (cg / 16) + 220.0;
    const int Ws = transposed ? g.Wo : g.W;
    for (int bh = 1; bh <= Hd && bh <= cap; ++bh) {
      const size_t smem = conv_smem(g, transposed, cg, bh);
      if (smem > budget) break;
      const int items = bh * NB;
      if (items < 14 && bh < Hd && bh < cap) continue;  // a block's fixed costs (launch, bank copy, first load) want 14 items or more
      const int bands = (Hd + bh - 1) / bh;
      const long long ctas = (long long)bands * groups * g.N;
      const int rb = conv_band_rows(bh, S, transposed);
      const double staged = ((double)cg * rb * Ws + 18.0 * (transposed ? rb : bh) * g.Wo) / ((double)cg * bh * Wd);
      const double band_fill = (double)Hd / (bands * bh);
      const int wmax = items < 2 ? 2 : (items < 14 ? items : 14);
      for (int w = wmax; w >= 2 && w >= wmax / 2; --w) {
        int bpsm = (int)((228 * 1024) / (smem + 1024));
        if (bpsm > 28 / w) bpsm = 28 / w;  // 72 registers per thread: 28 warps per SM
        if (bpsm > 16) bpsm = 16;
        if (bpsm < 1) continue;
        const int rounds = (items + w - 1) / w;
        const double util = (double)items / (rounds * w);
        const int resident = bpsm * w;
        const double occ = resident >= 20 ? 1.0 : 0.6 + 0.02 * resident;
        const double cost = (per_item / (util * occ) + 46.0 * staged) / (wave_fill(ctas, bpsm) * band_fill);
        if (cost < best_cost) {
          best_cost = cost;
          pl.BH = bh;
          pl.CG = cg;
          pl.groups = groups;
          pl.warps = w;
        }
      }
    }
    if (cg_only) break;
  }
  if (!pl.BH) {  // no block shape fits the budget: the caller falls back to the SIMT kernels
    pl.CG = pl.groups = pl.warps = pl.bands = 0;
    pl.smem = 0;
    return pl;
  }
  pl.bands = (Hd + pl.BH - 1) / pl.BH;
  pl.smem = conv_smem(g, transposed, pl.CG, pl.BH);
  return pl;
}

ConvPlan conv_plan(const Geom& g, bool transposed) {
  return cached_plan<ConvPlan>(g, transposed ? 1 : 0, [&] { return conv_plan_search(g, transposed); });
}

template <int S, bool TRANSPOSED>
int launch_conv(const __half* src, const __half* rot, const __half* w, __half* dst, const Geom& g, cudaStream_t s) {
  ConvPlan pl = conv_plan(g, TRANSPOSED);
  if (!pl.BH || pl.smem > (size_t)device_smem_optin() || pl.groups > 65535) return DK_ERR_UNSUPPORTED;
  pl.mode_src = ptr_mode(src);
  pl.mode_rot = ptr_mode(rot);
  pl.pair_store = (((TRANSPOSED ? g.W : g.Wo) & 1) == 0) && ptr_mode(dst) >= 1;
  auto kern = mma_conv_kernel<S, TRANSPOSED>;
  int rc = enable_smem(kern, pl.smem);
  if (rc) return rc;
  kern<<<dim3(pl.bands, pl.groups, g.N), pl.warps * 32, pl.smem, s>>>(src, rot, w, dst, g, pl);
  return check_launch();
}

// ================================================================== grad-offsets and grad-bank
// Shared by both kernels: the products dK[c, (pixel pair, tap)] = dy[c, pixel pair] * x[c, pixel pair + tap]
// of the two channels (gq, gq+8 of a 16-channel slab) this thread holds in A fragments.
template <int S>
__device__ __forceinline__ void dk_products(unsigned (&dk0)[9], unsigned (&dk1)[9], const __half* __restrict__ x0, int xpitch8,
                                            int Wp, unsigned dy0, unsigned dy1) {
  const __half* x1 = x0 + xpitch8;
#pragma unroll
  for (int fh = 0; fh < 3; ++fh) {
    const unsigned* p0 = reinterpret_cast<const unsigned*>(x0 + fh * Wp);
    const unsigned* p1 = reinterpret_cast<const unsigned*>(x1 + fh * Wp);
    const unsigned w0 = p0[0], w1 = p0[1], w2 = p0[2];
    const unsigned v0 = p1[0], v1 = p1[1], v2 = p1[2];
#pragma unroll
    for (int fw = 0; fw < 3; ++fw) {
      dk0[fh * 3 + fw] = hmul2u(dy0, tap_pair<S>(w0, w1, w2, fw));
      dk1[fh * 3 + fw] = hmul2u(dy1, tap_pair<S>(v0, v1, v2, fw));
    }
  }
}

struct RotPlan {
  bool dy_direct;  // dy straight from global memory into registers (see FiltPlan)
  int BH, warps, bands;
  int CG, groups;  // channels per block; with more than one group the blocks write fp32 partial sums
  bool big;        // one block of up to 16 warps per SM instead of two of up to 8
  int mode_x, mode_dy, mode_rot;
  size_t smem, ws_bytes;
};
constexpr int kRotScratch = 3 * 16 * 8 * 4 + 72 * 8;  // G of three taps (aliases the beta table) + (u, v)

template <int S, int MAXT, int MINB, bool DYD>
__global__ void __launch_bounds__(MAXT, MINB) mma_rot_kernel(const __half* __restrict__ dy, const __half* __restrict__ x,
                                                         const __half* __restrict__ rot, const __half* __restrict__ w,
                                                         __half* __restrict__ drot, float* __restrict__ partial,
                                                         const Geom g, const RotPlan pl) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int n = blockIdx.y;
  const int oh0 = blockIdx.x * pl.BH;
  const int c0 = blockIdx.z * pl.CG;
  const int cnt = min(pl.CG, g.C - c0);
  const Band bx = make_band(oh0 * S - 1, (pl.BH - 1) * S + 3, g.H, g.W, pl.mode_x);
  const Band by = make_band(oh0, pl.BH, g.Ho, g.Wo, pl.mode_dy);
  const Band br = make_band(oh0, pl.BH, g.Ho, g.Wo, pl.mode_rot);
  const int pitchT = pl.CG + 8;  // halves per cell row of the transposed bank

  __half* xband = reinterpret_cast<__half*>(smem_raw);
  __half* yband = xband + (size_t)pl.CG * bx.pitch_c;
  __half* rband = yband + (DYD ? (size_t)0 : (size_t)pl.CG * by.pitch_c);  // [18][br.pitch_c]
  __half* bankT = rband + (size_t)18 * br.pitch_c;                         // [16 cells][CG + 8]
  unsigned char* scratch = reinterpret_cast<unsigned char*>(bankT + 16 * pitchT);

  for (int i = threadIdx.x; i < 16 * cnt; i += blockDim.x) {
    const int cell = i / cnt, c = i - cell * cnt;
    bankT[cell * pitchT + c] = cell < g.cells ? __ldg(w + (size_t)(c0 + c) * g.cells + cell) : __float2half(0.f);
  }
  load_band(xband, bx, x, n, g.C, c0, cnt, g.H, g.W);
  if (!DYD) load_band(yband, by, dy, n, g.C, c0, cnt, g.Ho, g.Wo);
  load_band(rband, br, rot, n, 18, 0, 18, g.Ho, g.Wo);
  cp_async_wait_all();
  __syncthreads();

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int gq = lane >> 2, q = lane & 3;
  const int NB = (g.Wo + 7) >> 3;
  const int items = pl.BH * NB;
  unsigned* T = reinterpret_cast<unsigned*>(scratch + (size_t)warp * kRotScratch);
  float* Gs = reinterpret_cast<float*>(T);                       // [3 taps][16 cells][8 px], after the fragments are read
  float2* uv = reinterpret_cast<float2*>(T + 3 * 16 * 8);        // [9 taps][8 px]
  __half* drot_n = drot + (size_t)n * 18 * g.P;
  float* part_n = partial + ((size_t)blockIdx.z * g.N + n) * 18 * g.P;

  for (int item = warp; item < items; item += nwarps) {
    const int dr = item / NB;
    const int oh = oh0 + dr;
    if (oh >= g.Ho) break;
    const int ow0 = (item - dr * NB) << 3;
    item_uv<S>(uv, rband, br, g, oh, ow0, lane);
    const int ow = ow0 + 2 * q;
    const int xoff = window_offset(bx, oh * S - 1, ow, S);
    const int yoff = kSlack + oh * by.Wp + ow - by.org;

    float G[9][4];
#pragma unroll
    for (int t = 0; t < 9; ++t) G[t][0] = G[t][1] = G[t][2] = G[t][3] = 0.f;

    // DYD: the slab's two dy words come from global memory, fetched one slab ahead
    const bool dy_in = ow < g.Wo;
    const unsigned* dp = reinterpret_cast<const unsigned*>(dy + ((size_t)n * g.C + c0 + gq) * g.P + (size_t)oh * g.Wo + ow);
    const size_t dstep8 = (size_t)8 * g.P / 2;  // words between channel rows gq and gq + 8
    unsigned ndy0 = 0u, ndy1 = 0u;
    if (DYD && dy_in) {
      ndy0 = __ldg(dp);
      ndy1 = __ldg(dp + dstep8);
    }
    for (int cb16 = 0; cb16 < cnt; cb16 += 16) {
      unsigned dy0, dy1;
      if (DYD) {
        dy0 = ndy0;
        dy1 = ndy1;
        if (dy_in && cb16 + 16 < cnt) {
          ndy0 = __ldg(dp + (size_t)(cb16 + 16) / 8 * dstep8);
          ndy1 = __ldg(dp + (size_t)(cb16 + 24) / 8 * dstep8);
        }
      } else {
        dy0 = *reinterpret_cast<const unsigned*>(yband + (size_t)(cb16 + gq) * by.pitch_c + yoff);
        dy1 = *reinterpret_cast<const unsigned*>(yband + (size_t)(cb16 + gq + 8) * by.pitch_c + yoff);
      }
      unsigned dk0[9], dk1[9];
      dk_products<S>(dk0, dk1, xband + (size_t)(cb16 + gq) * bx.pitch_c + xoff, 8 * bx.pitch_c, bx.Wp, dy0, dy1);
      // A = W^T slab: rows = cells (gq, gq+8), k = channels (2q,2q+1) and (2q+8,2q+9)
      const unsigned* wt0 = reinterpret_cast<const unsigned*>(bankT + gq * pitchT + cb16);
      const unsigned* wt1 = reinterpret_cast<const unsigned*>(bankT + (gq + 8) * pitchT + cb16);
      const unsigned a0 = wt0[q], a1 = wt1[q], a2 = wt0[q + 4], a3 = wt1[q + 4];
#pragma unroll
      for (int t = 0; t < 9; ++t) mma16816_acc(G[t], a0, a1, a2, a3, movmatrix_trans(dk0[t]), movmatrix_trans(dk1[t]));
    }

    // d(offset)[pixel, tap, dir] = sum over the four corner cells of G * d(coefficient)/d(u or v)
#pragma unroll
    for (int pass = 0; pass < 3; ++pass) {
      __syncwarp();
#pragma unroll
      for (int tt = 0; tt < 3; ++tt) {
        const int t = pass * 3 + tt;
        *reinterpret_cast<float2*>(Gs + (tt * 16 + gq) * 8 + 2 * q) = make_float2(G[t][0], G[t][1]);
        *reinterpret_cast<float2*>(Gs + (tt * 16 + gq + 8) * 8 + 2 * q) = make_float2(G[t][2], G[t][3]);
      }
      __syncwarp();
      if (lane < 24) {
        const int px = lane & 7, tt = lane >> 3;
        const int t = pass * 3 + tt;
        const float2 c = uv[t * 8 + px];
        float gu = 0.f, gv = 0.f;
        if (c.x < 1e29f) {
          const float fu = floorf(c.x), fv = floorf(c.y);
          const int h0 = (int)fu, w0 = (int)fv;
          const float lh = c.x - fu, lw = c.y - fv;
          const float hh = 1.f - lh, hw = 1.f - lw;
          const float* Gp = Gs + tt * 128 + px;
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
          const size_t o = (size_t)(2 * t) * g.P + oh * g.Wo + ow0 + px;
          if (pl.groups == 1) {
            drot_n[o] = __float2half_rn(gu);
            drot_n[o + g.P] = __float2half_rn(gv);
          } else {
            part_n[o] = gu;
            part_n[o + g.P] = gv;
          }
        }
      }
    }
    __syncwarp();
  }
}

// out[i] = sum over channel groups of partial[group][i], fixed order
__global__ void reduce_rot_partials_kernel(const float* __restrict__ partial, __half* __restrict__ out, size_t n_out,
                                           int groups) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_out) return;
  float s = 0.f;
  for (int k = 0; k < groups; ++k) s += partial[(size_t)k * n_out + i];
  out[i] = __float2half_rn(s);
}

// Plan of the grad-offsets kernel.  A block needs the bands of every channel it sums over, and
// the sum over channels must be complete before the four-corner contraction, so:
//   1. all channels in one block, two blocks (<= 8 warps) per SM, if that fits and fills the GPU;
//   2. else all channels in one block of up to 16 warps, one per SM (large planes);
//   3. else (small planes, many channels) split the channels into groups that each write an
//      fp32 partial sum, reduced by a second pass: cheap there because the offset tensor is
//      small next to the activations.
static bool rot_dy_direct(const Geom& g) {
  // even rows (the pixel pairs of dy are aligned words) and small planes: measured faster up to 28 x 28 outputs
  // (0.095 -> 0.080, 0.083 -> 0.056 ms), slower on the wide layers, whose blocks walk over many slabs per item
  bool on = (g.Wo & 1) == 0 && g.P <= 784;
  if (const char* e = tuning_env("DK_B200_ROT_DY_DIRECT")) on = on && atoi(e) != 0;  // comparison runs
  return on;
}
static size_t rot_smem(const Geom& g, int cg, int bh, int warps) {
  const int S = g.sH;
  const int Wp = g.W + (g.W & 1), Wpo = g.Wo + (g.Wo & 1);
  return (size_t)cg * (band_pitch((bh - 1) * S + 3, Wp) + (rot_dy_direct(g) ? 0 : band_pitch(bh, Wpo))) * 2 +
         (size_t)18 * band_pitch(bh, Wpo) * 2 +
         (size_t)16 * (cg + 8) * 2 + (size_t)warps * kRotScratch;
}

RotPlan rot_plan_search(const Geom& g) {
  RotPlan pl;
  const int NB = (g.Wo + 7) / 8;
  const long long min_ctas = 2 * 148;
  pl.BH = 0;
  pl.big = false;
  pl.groups = 1;
  pl.CG = g.C;
  pl.dy_direct = rot_dy_direct(g);
  // One block of up to 16 warps per SM with a taller band first: the halo rows of x weigh less and a block's load is
  // spread over more items (measured: C = 144 at 56 x 56 0.38 -> 0.22 ms, never slower on the sweep's layers).
  // DK_B200_ROT_BIG=0 tries two blocks per SM first (tuning knob).
  static const int first_attempt = [] {
    const char* e = tuning_env("DK_B200_ROT_BIG");
    return (e && atoi(e) == 0) ? 0 : 1;
  }();
  for (int k = 0; k < 2 && !pl.BH; ++k) {
    const int attempt = first_attempt ? 1 - k : k;
    const size_t budget = attempt == 0 ? kTwoPerSm : kOnePerSm;
    const int maxw = attempt == 0 ? 8 : 16;
    int tallest = 0;
    int cap = g.Ho;
    if (const char* e = tuning_env("DK_B200_ROT_BH")) cap = atoi(e) > 0 ? atoi(e) : cap;  // tuning knob
    for (int bh = 1; bh <= g.Ho && bh <= cap; ++bh) {
      if (rot_smem(g, g.C, bh, pick_warps(bh * NB, maxw)) > budget) break;
      tallest = bh;
      if (bh * NB >= 2 * maxw) break;
    }
    if (!tallest) continue;
    if (tallest * NB < 7 || (long long)((g.Ho + tallest - 1) / tallest) * g.N < min_ctas) continue;
    // Among the bands up to that height: time of a band = fixed part (latency of its loads, barriers) + rows staged
    // + rounds of items over the warps; nothing overlaps in a block that has the SM to itself.  Constants fitted to
    // 28 x 28 ... 112 x 112 planes (band heights 1-14), in instructions per warp.
    const double t_item = 250.0 + 220.0 * (g.C / 16);
    const double per_half = 0.0645;
    double best_cost = 1e30;
    for (int bh = 1; bh <= tallest; ++bh) {
      const int items = bh * NB;
      if (items < 7 && bh < tallest) continue;
      const int wfull = items < maxw ? items : maxw;
      const int rounds = (items + wfull - 1) / wfull;
      int w = (items + rounds - 1) / rounds;  // fewest warps that finish in as many rounds
      if (w < 2) w = 2;
      if (rot_smem(g, g.C, bh, w) > budget) continue;
      const int bands = (g.Ho + bh - 1) / bh;
      auto band_time = [&](int rows) {
        const double staged = per_half * ((double)g.C * ((rows - 1) * g.sH + 3) * g.W + (pl.dy_direct ? 18.0 : g.C + 18.0) * rows * g.Wo);
        return 1000.0 + staged + ((rows * NB + w - 1) / w) * t_item;
      };
      const double cost = ((bands - 1) * band_time(bh) + band_time(g.Ho - (bands - 1) * bh)) / g.Ho;
      if (cost < best_cost) {
        best_cost = cost;
        pl.BH = bh;
        pl.warps = w;
      }
    }
    pl.big = attempt == 1;
  }
  if (!pl.BH) {
    const int slabs = g.C / 16;
    int bh = (14 + NB - 1) / NB;
    if (bh > g.Ho) bh = g.Ho;
    for (; bh >= 1 && !pl.BH; --bh) {
      const int warps = pick_warps(bh * NB, 8);
      for (int groups = 1; groups <= slabs; ++groups) {
        const int cg = ((slabs + groups - 1) / groups) * 16;
        if ((g.C + cg - 1) / cg != groups) continue;
        if (rot_smem(g, cg, bh, warps) > kTwoPerSm) continue;
        const long long ctas = (long long)((g.Ho + bh - 1) / bh) * g.N * groups;
        if (ctas < min_ctas && cg > 32) continue;
        if (cg < 64 && bh > 1 && groups > 1) break;  // too little work per item: try a shorter band first
        pl.BH = bh;
        pl.warps = warps;
        pl.CG = cg;
        pl.groups = groups;
        break;
      }
    }
  }
  if (pl.BH) {
    pl.smem = rot_smem(g, pl.CG, pl.BH, pl.warps);
    pl.bands = (g.Ho + pl.BH - 1) / pl.BH;
    pl.ws_bytes = pl.groups > 1 ? (size_t)pl.groups * g.N * 18 * g.P * sizeof(float) : 0;
  }
  return pl;
}

RotPlan rot_plan(const Geom& g) {
  return cached_plan<RotPlan>(g, 2, [&] { return rot_plan_search(g); });
}

// ------------------------------------------------------------------ grad-bank
struct FiltPlan {
  bool dy_direct;  // dy goes from global memory straight into registers (each word is used once) instead of through a band
  bool dy_ring;    // ... or, rows of 8 n pixels: each warp copies its next item's dy (16 bytes per channel row) with cp.async
                   // into a two-slot ring of its own while it works on the current item
  bool big;  // six channel slabs per block, one block of up to 14 warps per SM
  int BH, CG, groups, warps, bands, units_per_block, blocks_x;
  int mode_x, mode_dy, mode_rot;
  size_t smem, ws_bytes;
};

// DYM: 0 = dy band in shared memory, 1 = dy words from global memory into registers, 2 = per-warp ring (see FiltPlan)
template <int S, int NS, int MAXT, int MINB, int DYM>
__global__ void __launch_bounds__(MAXT, MINB) mma_filter_kernel(const __half* __restrict__ dy, const __half* __restrict__ x,
                                                            const __half* __restrict__ rot, float* __restrict__ partial,
                                                            const Geom g, const FiltPlan pl) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int c0 = blockIdx.y * pl.CG;
  const int cnt = min(pl.CG, g.C - c0);
  const int nslab = cnt >> 4;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int gq = lane >> 2, q = lane & 3;
  const int NB = (g.Wo + 7) >> 3;
  const int items = pl.BH * NB;
  const int Wp = g.W + (g.W & 1), Wpo = g.Wo + (g.Wo & 1);
  const int xpitch = band_pitch((pl.BH - 1) * S + 3, Wp), ypitch = band_pitch(pl.BH, Wpo);

  __half* xband = reinterpret_cast<__half*>(smem_raw);
  __half* yband = xband + (size_t)pl.CG * xpitch;
  __half* rband = yband + (DYM ? (size_t)0 : (size_t)pl.CG * ypitch);  // [18][ypitch]
  __half* ring = rband + (size_t)18 * ypitch + (size_t)warp * (2 * pl.CG * 8);  // DYM == 2: [2 slots][CG rows][8 pixels]
  const LaneCells lc = lane_cells(g, q);
  const bool sc44 = g.scH == 4 && g.scW == 4;

  float acc[NS][2][4];  // up to NS slabs of 16 channels x (cells 0-7 | cells 8-15)
#pragma unroll
  for (int sidx = 0; sidx < NS; ++sidx)
#pragma unroll
    for (int k = 0; k < 4; ++k) acc[sidx][0][k] = acc[sidx][1][k] = 0.f;

  const int total_units = g.N * pl.bands;
  const int u_begin = blockIdx.x * pl.units_per_block;
  const int u_end = min(u_begin + pl.units_per_block, total_units);
  for (int unit = u_begin; unit < u_end; ++unit) {
    const int n = unit / pl.bands;
    const int oh0 = (unit - n * pl.bands) * pl.BH;
    const Band bx = make_band(oh0 * S - 1, (pl.BH - 1) * S + 3, g.H, g.W, pl.mode_x);
    const Band by = make_band(oh0, pl.BH, g.Ho, g.Wo, pl.mode_dy);
    const Band br = make_band(oh0, pl.BH, g.Ho, g.Wo, pl.mode_rot);
    __syncthreads();  // previous unit's readers are done
    load_band(xband, bx, x, n, g.C, c0, cnt, g.H, g.W);
    if (!DYM) load_band(yband, by, dy, n, g.C, c0, cnt, g.Ho, g.Wo);
    load_band(rband, br, rot, n, 18, 0, 18, g.Ho, g.Wo);
    // DYM == 2: 16 bytes of every channel row of item it_ go to ring slot slot_, one row per lane and step
    auto ring_fill = [&](int it_, int slot_) {
      const int r_ = it_ / NB;
      if (it_ < items && oh0 + r_ < g.Ho) {
        const __half* sp = dy + ((size_t)n * g.C + c0) * g.P + (size_t)(oh0 + r_) * g.Wo + ((it_ - r_ * NB) << 3);
        __half* dp = ring + slot_ * (pl.CG * 8);
        for (int c = lane; c < cnt; c += 32) cp_async16(dp + c * 8, sp + (size_t)c * g.P);
      }
      cp_async_commit();
    };
    if (DYM == 2) ring_fill(warp, 0);
    cp_async_wait_all();
    __syncthreads();
    int slot = 0;
    for (int item = warp; item < items; item += nwarps, slot ^= 1) {
      const int dr = item / NB;
      const int oh = oh0 + dr;
      if (oh >= g.Ho) break;
      const int ow0 = (item - dr * NB) << 3;
      if (DYM == 2) {
        __syncwarp();                        // the item before last has been read out of the other slot
        ring_fill(item + nwarps, slot ^ 1);  // next item (an empty group when there is none)
      }
      // dy of the item, fetched ahead of its use: every slab before the hat products (their latency hides behind those), or,
      // with more than four slabs, the first two now and each further one two slabs ahead (fewer registers held)
      constexpr int PRE = NS > 4 ? 2 : NS;
      unsigned dyw[NS][2];
      const int owl = ow0 + 2 * q;
      const __half* dp = dy + ((size_t)n * g.C + c0 + gq) * g.P + (size_t)oh * g.Wo + owl;
      auto fetch_dy = [&](int sidx) {
        dyw[sidx][0] = dyw[sidx][1] = 0u;
        if (sidx < nslab && owl < g.Wo) {
          dyw[sidx][0] = __ldg(reinterpret_cast<const unsigned*>(dp + (size_t)(sidx << 4) * g.P));
          dyw[sidx][1] = __ldg(reinterpret_cast<const unsigned*>(dp + (size_t)((sidx << 4) + 8) * g.P));
        }
      };
      if (DYM == 1) {
#pragma unroll
        for (int sidx = 0; sidx < PRE; ++sidx) fetch_dy(sidx);
      }
      unsigned bw[10][2];  // beta as B fragments of the grad-bank product: [tap][cells 0-7 | cells 8-15]
      {
        unsigned bf[9][2];
        beta_direct<S, false>(bf, rband, br, g, lc, sc44, oh, ow0, g.H, g.W, g.Wo, gq);
#pragma unroll
        for (int t = 0; t < 9; ++t) {
          bw[t][0] = movmatrix_trans(bf[t][0]);
          bw[t][1] = movmatrix_trans(bf[t][1]);
        }
        bw[9][0] = bw[9][1] = 0u;
      }
      const int ow = ow0 + 2 * q;
      const int xoff = window_offset(bx, oh * S - 1, ow, S);
      const int yoff = kSlack + oh * by.Wp + ow - by.org;
      const unsigned* rw = reinterpret_cast<const unsigned*>(ring + slot * (pl.CG * 8)) + gq * 4 + q;
      if (DYM == 2) {
        cp_async_wait_group<1>();  // everything but the copy of the next item has landed
        __syncwarp();
      }
#pragma unroll
      for (int sidx = 0; sidx < NS; ++sidx) {
        if (sidx < nslab) {
          const int cb16 = sidx << 4;
          unsigned dy0, dy1;
          if (DYM == 1) {
            dy0 = dyw[sidx][0];
            dy1 = dyw[sidx][1];
            if (sidx + PRE < NS) fetch_dy(sidx + PRE);
          } else if (DYM == 2) {
            dy0 = rw[sidx * 64];       // rows cb16 + gq and cb16 + gq + 8, four words per row
            dy1 = rw[sidx * 64 + 32];
          } else {
            dy0 = *reinterpret_cast<const unsigned*>(yband + (size_t)(cb16 + gq) * by.pitch_c + yoff);
            dy1 = *reinterpret_cast<const unsigned*>(yband + (size_t)(cb16 + gq + 8) * by.pitch_c + yoff);
          }
          unsigned dk0[10], dk1[10];
          {
            unsigned a9[9], b9[9];
            dk_products<S>(a9, b9, xband + (size_t)(cb16 + gq) * bx.pitch_c + xoff, 8 * bx.pitch_c, bx.Wp, dy0, dy1);
#pragma unroll
            for (int t = 0; t < 9; ++t) { dk0[t] = a9[t]; dk1[t] = b9[t]; }
            dk0[9] = dk1[9] = 0u;
          }
#pragma unroll
          for (int j = 0; j < 5; ++j) {  // k = 16 = 8 pixels x taps (2j, 2j+1)
            mma16816_acc(acc[sidx][0], dk0[2 * j], dk1[2 * j], dk0[2 * j + 1], dk1[2 * j + 1], bw[2 * j][0],
                         bw[2 * j + 1][0]);
            mma16816_acc(acc[sidx][1], dk0[2 * j], dk1[2 * j], dk0[2 * j + 1], dk1[2 * j + 1], bw[2 * j][1],
                         bw[2 * j + 1][1]);
          }
        }
      }
    }
  }
  // reduce the warps' accumulators and write this block's partial bank gradient [cnt][16]
  __syncthreads();
  float* red = reinterpret_cast<float*>(smem_raw);  // [nwarps][CG][16]
#pragma unroll
  for (int sidx = 0; sidx < NS; ++sidx) {
    if (sidx < nslab) {
      float* r0 = red + ((size_t)warp * pl.CG + (sidx << 4) + gq) * 16;
      float* r1 = r0 + 8 * 16;
      r0[2 * q] = acc[sidx][0][0]; r0[2 * q + 1] = acc[sidx][0][1];
      r1[2 * q] = acc[sidx][0][2]; r1[2 * q + 1] = acc[sidx][0][3];
      r0[8 + 2 * q] = acc[sidx][1][0]; r0[8 + 2 * q + 1] = acc[sidx][1][1];
      r1[8 + 2 * q] = acc[sidx][1][2]; r1[8 + 2 * q + 1] = acc[sidx][1][3];
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < cnt * 16; i += blockDim.x) {
    float sum = 0.f;
    for (int wv = 0; wv < nwarps; ++wv) sum += red[(size_t)wv * pl.CG * 16 + i];
    partial[((size_t)blockIdx.x * g.C + c0) * 16 + i] = sum;
  }
}

// out[c][cell] = sum over blocks of partial[block][c][16]; one warp per output, fixed summation tree
__global__ void reduce_bank_partials_kernel(const float* __restrict__ partial, __half* __restrict__ out, int C, int cells,
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

FiltPlan filt_plan_search(const Geom& g) {
  FiltPlan pl;
  const int S = g.sH;
  // Two shapes of block: up to four channel slabs and two blocks per SM, or six slabs in one block of up to
  // 14 warps per SM.  The second halves the hat-product work per slab; it pays on wide rows where the first
  // would be stuck with three slabs (measured: C = 96 at 112 x 112).
  int cg_small = (g.C % 64 == 0) ? 64 : (g.C % 48 == 0) ? 48 : (g.C % 32 == 0) ? 32 : 16;
  if (const char* e = tuning_env("DK_B200_FILT_CG")) {  // tuning knob: 16, 32, 48 or 64 channels per block
    const int v = atoi(e);
    if ((v == 16 || v == 32 || v == 48 || v == 64) && g.C % v == 0) cg_small = v;
  }
  const int cg_big = (g.C % 96 == 0) ? 96 : (g.C % 80 == 0) ? 80 : cg_small;
  pl.big = cg_big >= 2 * cg_small && (g.Wo + 7) / 8 >= 14;
  if (const char* e = tuning_env("DK_B200_FILT_BIG")) pl.big = atoi(e) != 0;  // tuning knob
  pl.CG = pl.big ? cg_big : cg_small;
  pl.groups = g.C / pl.CG;
  const int NB = (g.Wo + 7) / 8;
  const int Wp = g.W + (g.W & 1), Wpo = g.Wo + (g.Wo & 1);
  const size_t budget = pl.big ? kOnePerSm : kTwoPerSm;
  pl.BH = 0;
  // Every dy word is used exactly once, so staging it in shared memory only adds traffic on the path the kernel is bound
  // by; with even output rows it is read straight into registers and the room goes to a taller band (fewer halo rows
  // of x per output row).  DK_B200_FILT_DY_DIRECT=0 keeps the band (comparison runs).
  pl.dy_direct = (g.Wo & 1) == 0;
  if (const char* e = tuning_env("DK_B200_FILT_DY_DIRECT")) pl.dy_direct = pl.dy_direct && atoi(e) != 0;
  // Six-slab blocks on rows of 8 n pixels (16-byte pieces per item and channel row): their warps waited 2.5 issue slots
  // per instruction on the register loads of dy (two slabs of lookahead is all the registers allow), so each warp copies
  // the whole next item into a ring of its own instead: 0.58 -> 0.47 ms on C = 96 at 112 x 112.  The four-slab blocks
  // fetch all of an item's dy before its hat products and gain nothing (measured 0-7 % slower with the ring).
  // DK_B200_FILT_DY_RING=0 keeps the register path (comparison runs).
  pl.dy_ring = pl.big && pl.dy_direct && (g.Wo & 7) == 0 && (g.P & 7) == 0;
  if (const char* e = tuning_env("DK_B200_FILT_DY_RING")) pl.dy_ring = pl.dy_ring && atoi(e) != 0;
  // measured: taller bands pay at stride 1 once dy is out of shared memory (five rows of 112 with the ring: 0.468 -> 0.452 ms)
  int max_items = (pl.dy_direct && S == 1) ? (pl.dy_ring ? 70 : 56) : 24;
  if (const char* e = tuning_env("DK_B200_FILT_ITEMS")) max_items = atoi(e) > 0 ? atoi(e) : max_items;  // tuning knob
  auto shape = [&](int bh, int* warps) {
    *warps = pick_warps(bh * NB, pl.big ? 14 : 8);
    const size_t smem = (size_t)pl.CG * (band_pitch((bh - 1) * S + 3, Wp) + (pl.dy_direct ? 0 : band_pitch(bh, Wpo))) * 2 +
                        (size_t)18 * band_pitch(bh, Wpo) * 2 + (pl.dy_ring ? (size_t)*warps * 2 * pl.CG * 16 : 0);
    const size_t red = (size_t)*warps * pl.CG * 16 * 4;
    return smem < red ? red : smem;
  };
  for (int bh = 1; bh <= g.Ho; ++bh) {
    int warps;
    if (shape(bh, &warps) > budget) break;
    pl.BH = bh;
    if (bh * NB >= max_items) break;
  }
  if (!pl.BH) return pl;
  pl.bands = (g.Ho + pl.BH - 1) / pl.BH;
  pl.BH = (g.Ho + pl.bands - 1) / pl.bands;  // as many bands, all of (nearly) one height
  pl.smem = shape(pl.BH, &pl.warps);
  const long long units = (long long)g.N * pl.bands;
  // As many blocks as are resident at once (one wave): the kernel holds 128 registers per thread, so 16 warps per SM.
  // Measured 8-23 % faster than twice as many blocks on planes of 28 x 28 and smaller.
  long long per_sm = 16 / pl.warps;
  if (per_sm > (long long)((228 * 1024) / (pl.smem + 1024))) per_sm = (long long)((228 * 1024) / (pl.smem + 1024));
  if (per_sm < 1) per_sm = 1;
  if (const char* e = tuning_env("DK_B200_FILT_BLOCKS_PER_SM")) per_sm = atoi(e) > 0 ? atoi(e) : per_sm;  // tuning knob
  long long want = per_sm * 148 / pl.groups;
  if (want > units) want = units;
  if (want < 1) want = 1;
  pl.units_per_block = (int)((units + want - 1) / want);
  pl.blocks_x = (int)((units + pl.units_per_block - 1) / pl.units_per_block);
  pl.ws_bytes = (size_t)pl.blocks_x * g.C * 16 * sizeof(float);
  return pl;
}

FiltPlan filt_plan(const Geom& g) {
  return cached_plan<FiltPlan>(g, 3, [&] { return filt_plan_search(g); });
}

// ------------------------------------------------------------------ grad-offsets + grad-bank in one pass
//
// Both gradients consume the products dK = dy * x.  For the planes the row-ring kernels do not take (28 x 28 and
// smaller) this kernel forms them once per item instead of once in each of the two kernels above:
//   G^T[16 cells x 8 px] += W^T * dK   (per item, over the block's channels) -> four-corner derivative -> d(offsets)
//   dW[16 ch x 16 cells] += dK * beta  (in registers across the block's items) -> per-block partial sums
// A block owns a group of up to 96 channels and walks over (sample, row band) units; with more than one group the
// offset gradients leave as fp32 partial sums per group.  One pass per kernel row (three taps) keeps 12 instead of 36
// accumulators of G live.  4 x 4 scopes only (G of a tap goes through a 6 x 6 grid with a zero border in shared memory).
struct GwPlan {
  bool dy_direct;  // dy straight from global memory into registers (even output rows)
  bool big;        // one block of up to 16 warps per SM instead of two of up to 8
  int BH, CG, groups, warps, bands, units_per_block, blocks_x;
  int mode_x, mode_dy, mode_rot;
  size_t smem, dw_bytes, ws_bytes;
};
constexpr int kGwBandScratch = 3 * 36 * 8 * 4 + 24 * 8;  // per warp: G of three taps on the padded grid + their (u, v)

template <int S, int MAXT, int MINB, bool DYD>
__global__ void __launch_bounds__(MAXT, MINB) mma_gw_kernel(const __half* __restrict__ dy, const __half* __restrict__ x,
                                                        const __half* __restrict__ rot, const __half* __restrict__ w,
                                                        __half* __restrict__ drot, float* __restrict__ gpart,
                                                        float* __restrict__ partial, const Geom g, const GwPlan pl) {
  constexpr int NS = 6;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int c0 = blockIdx.y * pl.CG;
  const int cnt = pl.CG;  // the groups divide the channels evenly
  const int nslab = cnt >> 4;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int gq = lane >> 2, q = lane & 3;
  const int NB = (g.Wo + 7) >> 3;
  const int items = pl.BH * NB;
  const int Wp = g.W + (g.W & 1), Wpo = g.Wo + (g.Wo & 1);
  const int xpitch = band_pitch((pl.BH - 1) * S + 3, Wp), ypitch = band_pitch(pl.BH, Wpo);
  const int pitchT = pl.CG + 8;

  __half* xband = reinterpret_cast<__half*>(smem_raw);
  __half* yband = xband + (size_t)pl.CG * xpitch;
  __half* rband = yband + (DYD ? (size_t)0 : (size_t)pl.CG * ypitch);  // [18][ypitch]
  __half* bankT = rband + (size_t)18 * ypitch;                          // [16 cells][CG + 8]
  float* Gs = reinterpret_cast<float*>(bankT + 16 * pitchT) + (size_t)warp * (kGwBandScratch / 4);  // [3 taps][36 cells][8 px]
  float2* uv = reinterpret_cast<float2*>(Gs + 3 * 36 * 8);                                          // [3 taps][8 px]
  // 4 x 4 scope: the lane's cells 2q, 2q+1 (row q / 2) and 2q+8, 2q+9 (two rows further) share the columns 2 (q % 2), + 1
  const float cell_row = (float)(q >> 1), cell_col = (float)((q & 1) << 1);
  const float uh0 = 0.5f, uw0 = 0.5f;  // (scope - kernel) / 2 for a 4 x 4 scope and 3 x 3 taps

  for (int i = threadIdx.x; i < 16 * cnt; i += blockDim.x) {
    const int cell = i / cnt, c = i - cell * cnt;
    bankT[cell * pitchT + c] = __ldg(w + (size_t)(c0 + c) * 16 + cell);
  }
  {
    float* gz = reinterpret_cast<float*>(bankT + 16 * pitchT);  // the border cells of the G grids stay zero
    for (int i = threadIdx.x; i < nwarps * (kGwBandScratch / 4); i += blockDim.x) gz[i] = 0.f;
  }

  float acc[NS][2][4];  // bank gradient of up to NS slabs of 16 channels x (cells 0-7 | cells 8-15)
#pragma unroll
  for (int sidx = 0; sidx < NS; ++sidx)
#pragma unroll
    for (int k = 0; k < 4; ++k) acc[sidx][0][k] = acc[sidx][1][k] = 0.f;
  const __half* wtp = bankT + ((lane & 7) + ((lane >> 3) & 1) * 8) * pitchT + (lane >> 4) * 8;  // this lane's ldmatrix row
  const int pc6 = ((gq >> 2) + 1) * 6 + (gq & 3) + 1;  // cell gq in the padded grid; cell gq + 8 lies two rows further

  const int total_units = g.N * pl.bands;
  const int u_begin = blockIdx.x * pl.units_per_block;
  const int u_end = min(u_begin + pl.units_per_block, total_units);
  for (int unit = u_begin; unit < u_end; ++unit) {
    const int n = unit / pl.bands;
    const int oh0 = (unit - n * pl.bands) * pl.BH;
    const Band bx = make_band(oh0 * S - 1, (pl.BH - 1) * S + 3, g.H, g.W, pl.mode_x);
    const Band by = make_band(oh0, pl.BH, g.Ho, g.Wo, pl.mode_dy);
    const Band br = make_band(oh0, pl.BH, g.Ho, g.Wo, pl.mode_rot);
    __syncthreads();  // previous unit's readers are done
    load_band(xband, bx, x, n, g.C, c0, cnt, g.H, g.W);
    if (!DYD) load_band(yband, by, dy, n, g.C, c0, cnt, g.Ho, g.Wo);
    load_band(rband, br, rot, n, 18, 0, 18, g.Ho, g.Wo);
    cp_async_wait_all();
    __syncthreads();
    __half* drot_n = drot + (size_t)n * 18 * g.P;
    float* part_n = gpart + ((size_t)blockIdx.y * g.N + n) * 18 * g.P;
    for (int item = warp; item < items; item += nwarps) {
      const int dr = item / NB;
      const int oh = oh0 + dr;
      if (oh >= g.Ho) break;
      const int ow0 = (item - dr * NB) << 3;
      const int ow = ow0 + 2 * q, pc = ow0 + gq;
      // DYD: dy of the lane's pixel pair in every slab comes from global memory into registers, all loads in flight at once
      // and kept for the three kernel rows (fetching them again per kernel row, one slab ahead, measured 0.188 against
      // 0.150 ms on C = 192, 28 x 28); a pair beyond the row reads as zero
      unsigned dyw[NS][2];
      if (DYD) {
        const unsigned* dp = reinterpret_cast<const unsigned*>(dy + ((size_t)n * g.C + c0 + gq) * g.P + (size_t)oh * g.Wo + ow);
        const size_t dstep8 = (size_t)4 * g.P;  // words between channel rows gq and gq + 8
#pragma unroll
        for (int sidx = 0; sidx < NS; ++sidx) {
          dyw[sidx][0] = dyw[sidx][1] = 0u;
          if (sidx < nslab && ow < g.Wo) {
            dyw[sidx][0] = __ldg(dp + (size_t)(2 * sidx) * dstep8);
            dyw[sidx][1] = __ldg(dp + (size_t)(2 * sidx + 1) * dstep8);
          }
        }
      }
      const int xoff = window_offset(bx, oh * S - 1, ow, S);
      const int yoff = kSlack + oh * by.Wp + ow - by.org;
      const __half* rbase = rband + kSlack - br.org + oh * br.Wp + pc;
#pragma unroll
      for (int fh = 0; fh < 3; ++fh) {
        // hat products of the three taps of this kernel row, transposed into B fragments of dW += dK * beta; a tap
        // whose source position lies in the padding, or a pixel beyond the row, gets zeros and an invalid (u, v)
        const int sr = oh * S - 1 + fh;
        const bool rok = sr >= 0 && sr < g.H;
        unsigned bw[3][2];
#pragma unroll
        for (int fw = 0; fw < 3; ++fw) {
          const int t = fh * 3 + fw;
          const int sc = pc * S - 1 + fw;
          const bool ok = rok && pc < g.Wo && sc >= 0 && sc < g.W;
          const __half* rp = rbase + (size_t)(2 * t) * br.pitch_c;
          const float u = ((float)fh + __half2float(rp[0])) + uh0;
          const float v = ok ? ((float)fw + __half2float(rp[br.pitch_c])) + uw0 : 1e30f;
          const float du = u - cell_row, dv = v - cell_col;
          const float hh0 = hat(du), hh1 = hat(du - 2.f);
          const float hw0 = hat(dv), hw1 = hat(dv - 1.f);
          bw[fw][0] = movmatrix_trans(pack2(hh0 * hw0, hh0 * hw1));
          bw[fw][1] = movmatrix_trans(pack2(hh1 * hw0, hh1 * hw1));
          if (q == 0) uv[fw * 8 + gq] = make_float2(u, v);
        }
        float G[3][4];
#pragma unroll
        for (int t = 0; t < 3; ++t) G[t][0] = G[t][1] = G[t][2] = G[t][3] = 0.f;
#pragma unroll
        for (int sidx = 0; sidx < NS; ++sidx) {
          if (sidx < nslab) {
            const int cb16 = sidx << 4;
            unsigned dy0, dy1;
            if (DYD) {
              dy0 = dyw[sidx][0];
              dy1 = dyw[sidx][1];
            } else {
              dy0 = *reinterpret_cast<const unsigned*>(yband + (size_t)(cb16 + gq) * by.pitch_c + yoff);
              dy1 = *reinterpret_cast<const unsigned*>(yband + (size_t)(cb16 + gq + 8) * by.pitch_c + yoff);
            }
            const unsigned* p0 = reinterpret_cast<const unsigned*>(xband + (size_t)(cb16 + gq) * bx.pitch_c + xoff + fh * bx.Wp);
            const unsigned* p1 = p0 + 4 * bx.pitch_c;  // channel row gq + 8
            const unsigned w0 = p0[0], w1 = p0[1], w2 = p0[2];
            const unsigned v0 = p1[0], v1 = p1[1], v2 = p1[2];
            unsigned d0[3], d1[3];  // dK of channel rows gq and gq + 8 for the three taps
#pragma unroll
            for (int fw = 0; fw < 3; ++fw) {
              d0[fw] = hmul2u(dy0, tap_pair<S>(w0, w1, w2, fw));
              d1[fw] = hmul2u(dy1, tap_pair<S>(v0, v1, v2, fw));
            }
            // A = W^T slab: rows = the 16 cells, k = the slab's 16 channels
            unsigned a[4];
            {
              const unsigned sa = (unsigned)__cvta_generic_to_shared(wtp + cb16);
              asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                           : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3]) : "r"(sa));
            }
#pragma unroll
            for (int fw = 0; fw < 3; ++fw)
              mma16816_acc(G[fw], a[0], a[1], a[2], a[3], movmatrix_trans(d0[fw]), movmatrix_trans(d1[fw]));
            // k = 16 = 8 pixels x (tap 0 | tap 1), then 8 pixels x (tap 2 | nothing)
            mma16816_acc(acc[sidx][0], d0[0], d1[0], d0[1], d1[1], bw[0][0], bw[1][0]);
            mma16816_acc(acc[sidx][1], d0[0], d1[0], d0[1], d1[1], bw[0][1], bw[1][1]);
            mma16816_acc(acc[sidx][0], d0[2], d1[2], 0u, 0u, bw[2][0], 0u);
            mma16816_acc(acc[sidx][1], d0[2], d1[2], 0u, 0u, bw[2][1], 0u);
          }
        }
        // d(offset)[pixel, tap, dir] = sum over the four corner cells of G * d(coefficient)/d(u or v): floor-based, as in
        // mma_rot_kernel; the zero border of the grid stands for the corners outside the bank
        __syncwarp();
#pragma unroll
        for (int tt = 0; tt < 3; ++tt) {
          *reinterpret_cast<float2*>(Gs + (tt * 36 + pc6) * 8 + 2 * q) = make_float2(G[tt][0], G[tt][1]);
          *reinterpret_cast<float2*>(Gs + (tt * 36 + pc6 + 12) * 8 + 2 * q) = make_float2(G[tt][2], G[tt][3]);
        }
        __syncwarp();
        if (lane < 24) {
          const int px = lane & 7, tt = lane >> 3;
          const float2 c = uv[tt * 8 + px];
          const bool valid = c.x > -1.f && c.y > -1.f && c.x < 4.f && c.y < 4.f;
          const float uc = valid ? c.x : 0.f, vc = valid ? c.y : 0.f;  // floor in -1 .. 3: both corner rows inside the grid
          const float fu = floorf(uc), fv = floorf(vc);
          const float lh = uc - fu, lw = vc - fv;
          const float hh = 1.f - lh, hw = 1.f - lw;
          const float* Gp = Gs + (tt * 36 + ((int)fu + 1) * 6 + (int)fv + 1) * 8 + px;
          const float g00 = Gp[0], g01 = Gp[8], g10 = Gp[48], g11 = Gp[56];
          float gu = hw * (g10 - g00) + lw * (g11 - g01);
          float gv = hh * (g01 - g00) + lh * (g11 - g10);
          if (!valid) gu = gv = 0.f;
          if (ow0 + px < g.Wo) {
            const size_t o = (size_t)(2 * (fh * 3 + tt)) * g.P + oh * g.Wo + ow0 + px;
            if (pl.groups == 1) {
              drot_n[o] = __float2half_rn(gu);
              drot_n[o + g.P] = __float2half_rn(gv);
            } else {
              part_n[o] = gu;
              part_n[o + g.P] = gv;
            }
          }
        }
        __syncwarp();
      }
    }
  }
  // reduce the warps' bank-gradient accumulators and write this block's partial [cnt][16]
  __syncthreads();
  float* red = reinterpret_cast<float*>(smem_raw);  // [nwarps][CG][16]
#pragma unroll
  for (int sidx = 0; sidx < NS; ++sidx) {
    if (sidx < nslab) {
      float* r0 = red + ((size_t)warp * pl.CG + (sidx << 4) + gq) * 16;
      float* r1 = r0 + 8 * 16;
      r0[2 * q] = acc[sidx][0][0]; r0[2 * q + 1] = acc[sidx][0][1];
      r1[2 * q] = acc[sidx][0][2]; r1[2 * q + 1] = acc[sidx][0][3];
      r0[8 + 2 * q] = acc[sidx][1][0]; r0[8 + 2 * q + 1] = acc[sidx][1][1];
      r1[8 + 2 * q] = acc[sidx][1][2]; r1[8 + 2 * q + 1] = acc[sidx][1][3];
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < cnt * 16; i += blockDim.x) {
    float sum = 0.f;
    for (int wv = 0; wv < nwarps; ++wv) sum += red[(size_t)wv * pl.CG * 16 + i];
    partial[((size_t)blockIdx.x * g.C + c0) * 16 + i] = sum;
  }
}

// Channel groups of up to 96 channels (six slabs of bank-gradient accumulators: 128 registers); bands as tall as shared
// memory allows, two blocks of up to 8 warps per SM where a band with at least 16 items (or the whole plane) fits, else
// one block of up to 16 warps; as many blocks as are resident at once, each walking over its share of the units.
GwPlan gw_plan_search(const Geom& g) {
  GwPlan pl;
  pl.BH = 0;
  if (g.scH != 4 || g.scW != 4) return pl;
  // Measured on the sweep's layers (batch 128, against grad-offsets + grad-bank as two kernels): 14 x 14 outputs and below
  // 0.053 / 0.084 / 0.049 / 0.074 / 0.059 ms against 0.069 / 0.100 / 0.063 / 0.100 / 0.080; 28 x 28 outputs 0.150 against
  // 0.147 (there one block over all 192 channels does as well as two groups with partial sums), so those stay apart.
  if (g.P > 196 && !tuning_env("DK_B200_GW_ANY")) return pl;
  pl.CG = 0;
  for (int cg = 96; cg >= 48; cg -= 16)
    if (g.C % cg == 0) { pl.CG = cg; break; }
  if (!pl.CG) {
    if (g.C <= 96) pl.CG = g.C;
    else return pl;
  }
  pl.groups = g.C / pl.CG;
  const int S = g.sH;
  const int NB = (g.Wo + 7) / 8;
  const int Wp = g.W + (g.W & 1), Wpo = g.Wo + (g.Wo & 1);
  pl.dy_direct = (g.Wo & 1) == 0;
  if (const char* e = tuning_env("DK_B200_GW_DY_DIRECT")) pl.dy_direct = pl.dy_direct && atoi(e) != 0;  // comparison runs
  auto shape = [&](int bh, int warps) {
    const size_t smem = (size_t)pl.CG * (band_pitch((bh - 1) * S + 3, Wp) + (pl.dy_direct ? 0 : band_pitch(bh, Wpo))) * 2 +
                        (size_t)18 * band_pitch(bh, Wpo) * 2 + (size_t)16 * (pl.CG + 8) * 2 + (size_t)warps * kGwBandScratch;
    const size_t red = (size_t)warps * pl.CG * 16 * 4;
    return smem < red ? red : smem;
  };
  for (int attempt = 0; attempt < 2 && !pl.BH; ++attempt) {
    const int maxw = attempt == 0 ? 8 : 16;
    const size_t budget = attempt == 0 ? kTwoPerSm : kOnePerSm;
    int tallest = 0;
    for (int bh = 1; bh <= g.Ho; ++bh) {
      if (shape(bh, pick_warps(bh * NB, maxw)) > budget) break;
      tallest = bh;
      if (bh * NB >= 4 * maxw) break;
    }
    if (!tallest) continue;
    if (attempt == 0 && tallest < g.Ho && tallest * NB < 2 * maxw) continue;  // too short a band: one big block instead
    pl.BH = tallest;
    pl.big = attempt == 1;
  }
  if (!pl.BH) return pl;
  pl.bands = (g.Ho + pl.BH - 1) / pl.BH;
  pl.BH = (g.Ho + pl.bands - 1) / pl.bands;  // as many bands, all of (nearly) one height
  pl.warps = pick_warps(pl.BH * NB, pl.big ? 16 : 8);
  pl.smem = shape(pl.BH, pl.warps);
  const long long units = (long long)g.N * pl.bands;
  long long per_sm = pl.big ? 1 : 2;
  long long want = per_sm * 148 / pl.groups;
  if (want > units) want = units;
  if (want < 1) want = 1;
  pl.units_per_block = (int)((units + want - 1) / want);
  pl.blocks_x = (int)((units + pl.units_per_block - 1) / pl.units_per_block);
  pl.dw_bytes = (((size_t)pl.blocks_x * g.C * 16 * sizeof(float)) + 255) & ~(size_t)255;
  pl.ws_bytes = pl.dw_bytes + (pl.groups > 1 ? (size_t)pl.groups * g.N * 18 * g.P * sizeof(float) : 0);
  return pl;
}

GwPlan gw_plan(const Geom& g) {
  return cached_plan<GwPlan>(g, 4, [&] { return gw_plan_search(g); });
}

}  // namespace

// out[c][cell] = sum over blocks of partial[block][c][16]: the second stage of every tensor-core bank gradient
int launch_reduce_bank_partials(const float* partial, __half* out, int C, int cells, int nblocks, cudaStream_t s) {
  const int n_out = C * cells;
  reduce_bank_partials_kernel<<<(n_out + 7) / 8, 256, 0, s>>>(partial, out, C, cells, nblocks);
  return check_launch();
}

// out[i] = sum over channel groups of partial[group][i]: the second stage of the offset gradient when the channels are split
int launch_reduce_rot_partials(const float* partial, __half* out, size_t n_out, int groups, cudaStream_t s) {
  const size_t blocks = (n_out + 255) / 256;
  if (blocks > 0x7fffffffULL) return DK_ERR_UNSUPPORTED;
  reduce_rot_partials_kernel<<<(unsigned)blocks, 256, 0, s>>>(partial, out, n_out, groups);
  return check_launch();
}

// ------------------------------------------------------------------ entry points used by dk_local.cu
// Each returns DK_ERR_UNSUPPORTED when the shape is outside the fast path.

// Block shape the fp16 fast path would launch for `pass` (0 forward, 1 grad-input, 2 grad-offsets, 3 grad-bank), for
// tools and tests; no GPU is touched.  out = {band height, channels per block, channel groups, warps per block, bands,
// dynamic shared memory (bytes), blocks in the grid, workspace (bytes)}.
int local_mma_plan_query(const Geom& g, int pass, long long out[8]) {
  if (!fast_shape(g)) return DK_ERR_UNSUPPORTED;
  if (pass == 0 || pass == 1) {
    const ConvPlan pl = conv_plan(g, pass == 1);
    if (!pl.BH) return DK_ERR_UNSUPPORTED;
    const long long v[8] = {pl.BH, pl.CG, pl.groups, pl.warps, pl.bands, (long long)pl.smem, (long long)pl.bands * pl.groups * g.N, 0};
    for (int i = 0; i < 8; ++i) out[i] = v[i];
  } else if (pass == 2) {
    const RotPlan pl = rot_plan(g);
    if (!pl.BH) return DK_ERR_UNSUPPORTED;
    const long long v[8] = {pl.BH, pl.CG, pl.groups, pl.warps, pl.bands, (long long)pl.smem, (long long)pl.bands * pl.groups * g.N,
                            (long long)pl.ws_bytes};
    for (int i = 0; i < 8; ++i) out[i] = v[i];
  } else if (pass == 3) {
    const FiltPlan pl = filt_plan(g);
    if (!pl.BH) return DK_ERR_UNSUPPORTED;
    const long long v[8] = {pl.BH, pl.CG, pl.groups, pl.warps, pl.bands, (long long)pl.smem, (long long)pl.blocks_x * pl.groups,
                            (long long)pl.ws_bytes};
    for (int i = 0; i < 8; ++i) out[i] = v[i];
  } else {
    return DK_ERR_BAD_ARGUMENT;
  }
  return DK_OK;
}

int local_conv_mma(const __half* src, const __half* rot, const __half* w, __half* dst, const Geom& g, bool transposed,
                   cudaStream_t s) {
  if (!fast_shape(g)) return DK_ERR_UNSUPPORTED;
  if (transposed) return g.sH == 1 ? launch_conv<1, true>(src, rot, w, dst, g, s) : launch_conv<2, true>(src, rot, w, dst, g, s);
  if (g.sH == 1) return launch_conv<1, false>(src, rot, w, dst, g, s);
  return launch_conv<2, false>(src, rot, w, dst, g, s);
}

size_t local_rot_mma_workspace(const Geom& g) {
  if (!fast_shape(g)) return 0;
  const RotPlan pl = rot_plan(g);
  return pl.BH ? pl.ws_bytes : 0;
}

int local_rot_mma(const __half* dy, const __half* x, const __half* rot, const __half* w, __half* drot, const Geom& g,
                  void* ws, size_t ws_bytes, cudaStream_t s) {
  if (!fast_shape(g)) return DK_ERR_UNSUPPORTED;
  RotPlan pl = rot_plan(g);
  if (!pl.BH || pl.smem > (size_t)device_smem_optin() || pl.groups > 65535) return DK_ERR_UNSUPPORTED;
  if (pl.ws_bytes && (ws == nullptr || ws_bytes < pl.ws_bytes)) return DK_ERR_WORKSPACE;
  pl.mode_x = ptr_mode(x);
  pl.mode_dy = ptr_mode(dy);
  pl.mode_rot = ptr_mode(rot);
  if (pl.dy_direct && pl.mode_dy == 0) return DK_ERR_UNSUPPORTED;  // a dy pointer that is not 4-byte aligned: SIMT kernels
  int rc;
  const dim3 grid(pl.bands, g.N, pl.groups);
  float* partial = reinterpret_cast<float*>(ws);
#define DK_LAUNCH_ROT(SS, MAXT, MINB)                                                     \
  if (pl.dy_direct) DK_LAUNCH_ROT2(SS, MAXT, MINB, true) else DK_LAUNCH_ROT2(SS, MAXT, MINB, false)
#define DK_LAUNCH_ROT2(SS, MAXT, MINB, DD)                                                \
  {                                                                                       \
    auto kern = mma_rot_kernel<SS, MAXT, MINB, DD>;                                       \
    if ((rc = enable_smem(kern, pl.smem))) return rc;                                     \
    kern<<<grid, pl.warps * 32, pl.smem, s>>>(dy, x, rot, w, drot, partial, g, pl);       \
  }
  if (g.sH == 1) {
    if (pl.big) DK_LAUNCH_ROT(1, 512, 1) else DK_LAUNCH_ROT(1, 256, 2)
  } else {
    if (pl.big) DK_LAUNCH_ROT(2, 512, 1) else DK_LAUNCH_ROT(2, 256, 2)
  }
#undef DK_LAUNCH_ROT
#undef DK_LAUNCH_ROT2
  if ((rc = check_launch())) return rc;
  if (pl.groups > 1) {
    const size_t n_out = (size_t)g.N * 18 * g.P;
    const size_t blocks = (n_out + 255) / 256;
    if (blocks > 0x7fffffffULL) return DK_ERR_UNSUPPORTED;
    reduce_rot_partials_kernel<<<(unsigned)blocks, 256, 0, s>>>(partial, drot, n_out, pl.groups);
    rc = check_launch();
  }
  return rc;
}

size_t local_filter_mma_workspace(const Geom& g) {
  if (!fast_shape(g)) return 0;
  const FiltPlan pl = filt_plan(g);
  return pl.BH ? pl.ws_bytes : 0;
}

int local_filter_mma(const __half* dy, const __half* x, const __half* rot, __half* dw, const Geom& g, void* ws,
                     size_t ws_bytes, cudaStream_t s) {
  if (!fast_shape(g)) return DK_ERR_UNSUPPORTED;
  FiltPlan pl = filt_plan(g);
  if (!pl.BH || pl.smem > (size_t)device_smem_optin() || pl.groups > 65535) return DK_ERR_UNSUPPORTED;
  if (ws == nullptr || ws_bytes < pl.ws_bytes) return DK_ERR_WORKSPACE;
  pl.mode_x = ptr_mode(x);
  pl.mode_dy = ptr_mode(dy);
  pl.mode_rot = ptr_mode(rot);
  if (pl.dy_direct && pl.mode_dy == 0) return DK_ERR_UNSUPPORTED;  // a dy pointer that is not 4-byte aligned: SIMT kernels
  int rc;
  float* partial = reinterpret_cast<float*>(ws);
#define DK_LAUNCH_FILT(SS, NS, MAXT, MINB, DD)                                                        \
  {                                                                                                 \
    auto kern = mma_filter_kernel<SS, NS, MAXT, MINB, DD>;                                          \
    if ((rc = enable_smem(kern, pl.smem))) return rc;                                               \
    kern<<<dim3(pl.blocks_x, pl.groups), pl.warps * 32, pl.smem, s>>>(dy, x, rot, partial, g, pl);  \
  }
  const int dym = !pl.dy_direct ? 0 : (pl.dy_ring && pl.mode_dy == 2) ? 2 : 1;
#define DK_LAUNCH_FILT3(SS, NS, MAXT, MINB)                                \
  if (dym == 2) DK_LAUNCH_FILT(SS, NS, MAXT, MINB, 2)                      \
  else if (dym == 1) DK_LAUNCH_FILT(SS, NS, MAXT, MINB, 1)                 \
  else DK_LAUNCH_FILT(SS, NS, MAXT, MINB, 0)
  if (g.sH == 1) {
    if (pl.big) DK_LAUNCH_FILT3(1, 6, 448, 1) else DK_LAUNCH_FILT3(1, 4, 256, 2)
  } else {
    if (pl.big) DK_LAUNCH_FILT3(2, 6, 448, 1) else DK_LAUNCH_FILT3(2, 4, 256, 2)
  }
#undef DK_LAUNCH_FILT3
#undef DK_LAUNCH_FILT
  if ((rc = check_launch())) return rc;
  const int n_out = g.C * g.cells;
  reduce_bank_partials_kernel<<<(n_out + 7) / 8, 256, 0, s>>>(partial, dw, g.C, g.cells, pl.blocks_x);
  return check_launch();
}

// Workspace of local_gw_mma (per-block partial bank gradients, then the per-group partial offset gradients); 0 = not covered.
size_t local_gw_mma_workspace(const Geom& g) {
  if (!fast_shape(g)) return 0;
  const GwPlan pl = gw_plan(g);
  return pl.BH ? pl.ws_bytes : 0;
}

// grad-offsets and grad-bank of the local deformable kernel in one pass (band form; 4 x 4 scope)
int local_gw_mma(const __half* dy, const __half* x, const __half* rot, const __half* w, __half* drot, __half* dw, const Geom& g,
                 void* ws, size_t ws_bytes, cudaStream_t s) {
  if (!fast_shape(g)) return DK_ERR_UNSUPPORTED;
  GwPlan pl = gw_plan(g);
  if (!pl.BH || pl.smem > (size_t)device_smem_optin() || pl.groups > 65535) return DK_ERR_UNSUPPORTED;
  if (ws == nullptr || ws_bytes < pl.ws_bytes) return DK_ERR_WORKSPACE;
  pl.mode_x = ptr_mode(x);
  pl.mode_dy = ptr_mode(dy);
  pl.mode_rot = ptr_mode(rot);
  if (pl.dy_direct && pl.mode_dy == 0) return DK_ERR_UNSUPPORTED;  // a dy pointer that is not 4-byte aligned: separate kernels
  int rc;
  float* partial = reinterpret_cast<float*>(ws);
  float* gpart = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(ws) + pl.dw_bytes);
#define DK_LAUNCH_GW(SS, MAXT, MINB, DD)                                                                       \
  {                                                                                                          \
    auto kern = mma_gw_kernel<SS, MAXT, MINB, DD>;                                                           \
    if ((rc = enable_smem(kern, pl.smem))) return rc;                                                        \
    kern<<<dim3(pl.blocks_x, pl.groups), pl.warps * 32, pl.smem, s>>>(dy, x, rot, w, drot, gpart, partial, g, pl); \
  }
#define DK_LAUNCH_GW2(SS, MAXT, MINB) \
  if (pl.dy_direct) DK_LAUNCH_GW(SS, MAXT, MINB, true) else DK_LAUNCH_GW(SS, MAXT, MINB, false)
  if (g.sH == 1) {
    if (pl.big) DK_LAUNCH_GW2(1, 512, 1) else DK_LAUNCH_GW2(1, 256, 2)
  } else {
    if (pl.big) DK_LAUNCH_GW2(2, 512, 1) else DK_LAUNCH_GW2(2, 256, 2)
  }
#undef DK_LAUNCH_GW2
#undef DK_LAUNCH_GW
  if ((rc = check_launch())) return rc;
  if (pl.groups > 1) {
    const size_t n_out = (size_t)g.N * 18 * g.P;
    const size_t blocks = (n_out + 255) / 256;
    if (blocks > 0x7fffffffULL) return DK_ERR_UNSUPPORTED;
    reduce_rot_partials_kernel<<<(unsigned)blocks, 256, 0, s>>>(gpart, drot, n_out, pl.groups);
    if ((rc = check_launch())) return rc;
  }
  const int n_out = g.C * g.cells;
  reduce_bank_partials_kernel<<<(n_out + 7) / 8, 256, 0, s>>>(partial, dw, g.C, g.cells, pl.blocks_x);
  return check_launch();
}

}  // namespace dk
