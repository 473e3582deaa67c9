// Row-ring kernels of the local deformable kernel (fp16 storage, fp32 accumulation) for sm_100a.
//
// Same mathematics as dk_local_mma.cu -- the bilinear resampling of the bank is the contraction
//   K[c, p, tap] = sum_cell W[c, cell] * beta[p, tap, cell],   beta = hat(u - a) * hat(v - b)
// on mma.sync.m16n8k16, followed by y[c, p] += x[c, p + tap] * K[c, p, tap] on the CUDA cores --
// but a different way of moving the data.  A block walks down a contiguous range of output rows
// of ALL its channels.  A producer warp streams the source rows through rings of shared-memory
// slots (as many as shared memory holds: the depth need not be a power of two), one tiled TMA copy (cp.async.bulk.tensor) per row whose out-of-range elements the
// hardware fills with zeros: that supplies the convolution padding, so no tap needs a mask.  The
// consumer warps wait on a slot's mbarrier, never on each other: filling and computing overlap,
// each source row crosses HBM once and shared memory once, and all pitches are compile-time
// constants.  K comes out of the tensor cores rounded to fp16 (relative 2^-11, like the tensors
// themselves) and meets x in a mixed-precision FMA (fma.rn.f32.f16: the fp16 x fp16 product is exact,
// the sum is fp32), so the forward and grad-input passes need no fp16 -> fp32 conversions.  Measured
// on C = 96, 112 x 112, batch 128: 0.28 ms against 0.31 with K in fp32 and x widened by conversions;
// the error against the fp32 oracle is the same to three digits (the rounding of the output dominates).
//
// Kernels:
//   ring_conv_kernel   forward, and grad-input at stride 1 (the same stencil with the taps flipped)
//   ring_gw_kernel     grad-offsets and grad-bank in ONE pass: both consume dK = dy * x,
//                        G^T[16 cells x 8 px] += W^T * dK   -> four-corner derivative contraction -> d(offsets)
//                        dW[16 ch x 16 cells] += dK * beta  -> per-block partial sums, reduced in a fixed order
//
//   ring_convT2_kernel grad-input at stride 2: an item of 8 output pixels expands into a 2 x 16 patch of dx
//   ring_bwd_kernel    all three gradients from one stream of rows (least memory traffic; not the fastest, see below)
//
// Covers fp16, 3x3, pad 1, dilation 1, stride 1 or 2, one offset group, scope 4 x 4, channels a multiple
// of 16, input rows of 112 or 56 elements (fetched by TMA, which needs 16-byte row pitches) and of 28 elements
// (56-byte rows: up to four producer warps copy them in 8-byte cp.async pieces; at stride 2 only the grad-input
// kernel).  Other shapes stay on dk_local_mma.cu.
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "dk_ring.cuh"

namespace dk {

using namespace mma;
using namespace ring;

// second stages of the gradient reductions (dk_local_mma.cu):
// out[c][cell] = sum over blocks of partial[block][c][16];  out[i] = sum over channel groups of partial[group][i]
int launch_reduce_bank_partials(const float* partial, __half* out, int C, int cells, int nblocks, cudaStream_t s);
int launch_reduce_rot_partials(const float* partial, __half* out, size_t n_out, int groups, cudaStream_t s);

namespace {

constexpr int kErrTimeout = 1;

// Zero-initialised by the loader; set when a bounded wait ran out (see dk_ring.cuh).
__device__ int g_ring_error;

struct RingParams {
  int N, C;
  int Hs, Hd;      // rows of the source and of the destination plane
  int CG;          // channels per block (multiple of 16)
  int R, RR;       // slots in the source ring and in the per-destination-row rings
  int NP;          // producer warps (more than one only where no ring of the kernel is filled by TMA)
  int L;           // padded source rows per sample in the block's stream
  int rows_total;  // N * Hd
  int rows_per_block;
  int scH, scW, cells;
};

__device__ __forceinline__ LaneCells lane_cells_of(int scW, int cells, int q) {
  LaneCells lc;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int cell = 2 * q + (k & 1) + (k >> 1) * 8;
    lc.ok[k] = cell < cells;
    const int a = cell / scW;
    lc.ca[k] = (float)a;
    lc.cb[k] = (float)(cell - a * scW);
  }
  return lc;
}


// Hat products of pixel column gq of an item for one tap, as the B fragment of K = W * beta^T:
// b0 = cells (2q, 2q+1), b1 = cells (2q+8, 2q+9).  rp points at the tap's vertical offset of the
// pixel in a ring slot; the horizontal one lies WOP halves further.  (u, v) are returned.
template <int WOP, bool SC44>
__device__ __forceinline__ void beta_tap(unsigned (&b)[2], const __half* __restrict__ rp, float fh, float fw, const LaneCells& lc,
                                         float uh0, float uw0, float& u, float& v) {
  // same association as the reference: (tap index + offset) + (scope - kernel) / 2
  u = (fh + __half2float(rp[0])) + uh0;
  v = (fw + __half2float(rp[WOP])) + uw0;
  if (SC44) {  // 4 x 4 scope: the lane's four cells share two rows and two columns
    const float hh0 = hat(u - lc.ca[0]), hh1 = hat(u - lc.ca[2]);
    const float hw0 = hat(v - lc.cb[0]), hw1 = hat(v - lc.cb[1]);
    b[0] = pack2(hh0 * hw0, hh0 * hw1);
    b[1] = pack2(hh1 * hw0, hh1 * hw1);
  } else {
    float b4[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) b4[k] = lc.ok[k] ? hat(u - lc.ca[k]) * hat(v - lc.cb[k]) : 0.f;
    b[0] = pack2(b4[0], b4[1]);
    b[1] = pack2(b4[2], b4[3]);
  }
}

// Offset rows in a slot: 18 planes of WOP halves, 8 zero halves in front of each.
template <int Wr>
struct RotLayout {
  static constexpr int kWop = 8 + ((Wr + 7) / 8) * 8 + 8;
  static constexpr int kSlot = 18 * kWop;  // halves
  static constexpr int kPiece = (Wr % 8 == 0) ? 16 : ((Wr % 4 == 0) ? 8 : ((Wr % 2 == 0) ? 4 : 0));  // 0: element by element
  static constexpr int kPieces = kPiece ? Wr * 2 / kPiece : Wr;
};

template <int PIECE>
__device__ __forceinline__ void cp_piece(void* d, const void* s) {
  if (PIECE == 16) cp_async16(d, s);
  else if (PIECE == 8) cp_async8(d, s);
  else cp_async4(d, s);
}

// producer warp pw of np: row `row` of the 18 offset planes of sample n -> ring slot.  The slot's "full" barrier (count
// 32 * np) gets one arrival per lane: when that lane's cp.async copies have landed, or, for odd row widths that only allow
// element-wise copies, after the lane's plain stores.
template <int Wr>
__device__ __forceinline__ void fill_rot_row(__half* slot, const __half* __restrict__ rot, int n, int rows, int row, int lane,
                                             unsigned full_bar, int pw = 0, int np = 1) {
  using RL = RotLayout<Wr>;
  const size_t plane = (size_t)rows * Wr;
  const __half* sp = rot + (size_t)n * 18 * plane + (size_t)row * Wr;
  if (RL::kPiece) {
    if (RL::kPieces <= 16) {
      // a lane keeps its piece of the row and walks down the 18 planes, 32 / kPieces of them per step
      constexpr int PLS = 32 / (RL::kPieces <= 16 ? RL::kPieces : 1);
      const int sub = lane / RL::kPieces, pc = lane - sub * RL::kPieces;
      if (sub < PLS) {
        const int first = PLS * pw + sub, step = PLS * np;
        __half* d = slot + first * RL::kWop + 8 + pc * (RL::kPiece / 2);
        const __half* g = sp + first * plane + pc * (RL::kPiece / 2);
        for (int pl = first; pl < 18; pl += step) {
          cp_piece<RL::kPiece ? RL::kPiece : 4>(d, g);
          d += step * RL::kWop;
          g += step * plane;
        }
      }
    } else {
      for (int i = lane + 32 * pw; i < 18 * RL::kPieces; i += 32 * np) {
        const int pl = i / RL::kPieces, pc = i - pl * RL::kPieces;
        cp_piece<RL::kPiece ? RL::kPiece : 4>(slot + pl * RL::kWop + 8 + pc * (RL::kPiece / 2), sp + pl * plane + pc * (RL::kPiece / 2));
      }
    }
    cp_async_arrive_noinc(full_bar);
  } else {
    for (int base = 256 * pw; base < 18 * Wr; base += 256 * np) {  // eight independent loads per lane in flight
      __half v[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int i = base + k * 32 + lane, pl = i / Wr;
        if (i < 18 * Wr) v[k] = __ldg(sp + pl * plane + (i - pl * Wr));
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int i = base + k * 32 + lane, pl = i / Wr;
        if (i < 18 * Wr) slot[pl * RL::kWop + 8 + (i - pl * Wr)] = v[k];
      }
    }
    mbar_arrive(full_bar);
  }
}

// producer warp pw of np: row `row` of channels c0 .. c0+cg-1 of sample n of a [N][C][rows][Wd] tensor -> ring slot, for rows
// TMA cannot fetch (cp.async pieces of 16, 8 or 4 bytes, element-wise for odd widths); full barrier count 32 * np as above
template <int Wd>
__device__ __forceinline__ void fill_plane_row(__half* slot, const __half* __restrict__ src, int n, int C, int c0, int cg, int rows,
                                               int row, int lane, unsigned full_bar, int pw = 0, int np = 1) {
  using L = RowLayout<Wd>;
  const size_t plane = (size_t)rows * Wd;
  const __half* sp = src + ((size_t)n * C + c0) * plane + (size_t)row * Wd;
  if (L::kPiece) {
    constexpr int PB = L::kPiece ? L::kPiece : 4;
    constexpr int PIECES = Wd * 2 / PB;
    if (PIECES <= 16) {
      // a lane keeps its piece of the row and walks down the channels, 32 / PIECES of them per step: two additions per copy
      constexpr int CH = 32 / (PIECES <= 16 ? PIECES : 1);
      const int sub = lane / PIECES, pc = lane - sub * PIECES;
      if (sub < CH) {
        const int first = CH * pw + sub, step = CH * np;
        __half* d = slot + first * L::kInner + 8 + pc * (PB / 2);
        const __half* g = sp + first * plane + pc * (PB / 2);
#pragma unroll 4
        for (int ch = first; ch < cg; ch += step) {
          cp_piece<PB>(d, g);
          d += step * L::kInner;
          g += step * plane;
        }
      }
    } else {
      for (int i = lane + 32 * pw; i < cg * PIECES; i += 32 * np) {
        const int ch = i / PIECES, pc = i - ch * PIECES;
        cp_piece<PB>(slot + ch * L::kInner + 8 + pc * (PB / 2), sp + ch * plane + pc * (PB / 2));
      }
    }
    cp_async_arrive_noinc(full_bar);
  } else {
    for (int base = 256 * pw; base < cg * Wd; base += 256 * np) {  // eight independent loads per lane in flight
      __half v[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int i = base + k * 32 + lane, ch = i / Wd;
        if (i < cg * Wd) v[k] = __ldg(sp + ch * plane + (i - ch * Wd));
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int i = base + k * 32 + lane, ch = i / Wd;
        if (i < cg * Wd) slot[ch * L::kInner + 8 + (i - ch * Wd)] = v[k];
      }
    }
    mbar_arrive(full_bar);
  }
}

// producer warp pw of np: one source row of the block's channels into its ring slot, whatever the row width allows.  Rows
// outside the plane (row < 0 or >= rows) become zero rows: the TMA unit fills them by itself, the other paths store zeros.
// The slot's full barrier counts 1 (TMA: the expect_tx arrival of the first producer warp; the others have nothing to do) or
// 32 * np (one arrival per lane).
template <int Wd>
__device__ __forceinline__ void fill_src_row(__half* slot, unsigned slot_u32, unsigned slot_bytes, const CUtensorMap* tm,
                                             const __half* __restrict__ src, int n, int C, int c0, int cg, int rows, int row, int lane,
                                             unsigned full_bar, int pw = 0, int np = 1) {
  if (RowLayout<Wd>::kTma) {
    if (lane == 0 && pw == 0) {
      mbar_arrive_expect_tx(full_bar, slot_bytes);
      tma_load_3d(slot_u32, tm, -8, row, n * C + c0, full_bar);
    }
  } else if (row >= 0 && row < rows) {
    fill_plane_row<Wd>(slot, src, n, C, c0, cg, rows, row, lane, full_bar, pw, np);
  } else {
    for (int i = lane + 32 * pw; i < (int)(slot_bytes >> 4); i += 32 * np) reinterpret_cast<uint4*>(slot)[i] = make_uint4(0, 0, 0, 0);
    mbar_arrive(full_bar);
  }
}

// Four 8 x 8 tiles of 16-bit values in one instruction: lane l passes the address of row l % 8 of tile l / 8 (16 bytes, aligned)
// and receives, per tile, the fragment element pair (row lane / 4, columns 2 (lane % 4), + 1).
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* row) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(row);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}

// d = a * b with fp16 output (d[0] = row gq, columns (2q, 2q+1); d[1] = row gq + 8), without `volatile` so that the
// compiler may schedule it freely
__device__ __forceinline__ void mma_h_new(unsigned (&d)[2], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f16.f16.f16.f16 {%0,%1}, {%2,%3,%4,%5}, {%6,%7}, {%8,%8};\n"
      : "=r"(d[0]), "=r"(d[1])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(0u));
}
__device__ __forceinline__ void ring_fail(int lane) {
  if (lane == 0) atomicExch(&g_ring_error, kErrTimeout);
}

// Arrivals of one finished item on the three source-row fills k0 .. k0+2 it read.  A stream row is read by
// U = 3 (stride 1) or 2 (stride 2) destination rows; where a neighbour that would read it lies outside the
// sample or outside this block's range, the first / last row of the range arrives in its place, so that every
// fill of a slot collects exactly U * (items per row) arrivals and is only then overwritten.
template <int S>
__device__ __forceinline__ int release_count(int j, bool first, bool last) {
  if (S == 1) return 1 + (first ? 2 - j : 0) + (last ? j : 0);
  return (j == 1) ? 2 : 1 + (((j == 0 && first) || (j == 2 && last)) ? 1 : 0);
}

// One tap (fh fixed by the caller, fw = FW) of an item for one channel slab: K = W * beta^T on the tensor cores with fp16
// output (K[ch gq][px 2q, 2q+1] in kh[0], channel gq + 8 in kh[1]), then four mixed-precision FMAs (fp16 x fp16 products,
// exact, summed in fp32) with the source values of the lane's two pixels: half 1 + i of the six-half window, where
// i = fw (forward) or 2 - fw (transposed) for pixel 0 and i + S (or + 1) for pixel 1.
template <int S, bool TR, int FW>
__device__ __forceinline__ void tap_row(float (&acc)[4], const unsigned (&a)[4], const unsigned (&b)[2], unsigned w0, unsigned w1,
                                        unsigned w2, unsigned v0, unsigned v1, unsigned v2) {
  unsigned kh[2];
  mma_h_new(kh, a, b[0], b[1]);
  constexpr int I0 = 1 + (TR ? 2 - FW : FW), I1 = I0 + (TR ? 1 : S);
  fma_win<I0, 0>(acc[0], w0, w1, w2, kh[0]);
  fma_win<I1, 1>(acc[1], w0, w1, w2, kh[0]);
  fma_win<I0, 0>(acc[2], v0, v1, v2, kh[1]);
  fma_win<I1, 1>(acc[3], v0, v1, v2, kh[1]);
}

// The channel-slab loop of the forward / stride-1 grad-input stencil for one item: xr[fh] points at the lane's window
// (channel row gq, source column ow*S - 2) in the slot of source row fh, bkp at the lane's words of the bank copy, y0 at
// destination (channel gq, pixel ow); bf holds the hat products of the nine taps.
// npx = how many of the lane's two pixels exist (0, 1, 2); PAIRS = destination rows are even, so a pixel pair is one aligned word.
template <int S, int INNER, bool TR, bool PAIRS>
__device__ __forceinline__ void conv_slabs(const __half* const (&xr)[3], const __half* __restrict__ bkp, __half* __restrict__ y0,
                                           int nslab, size_t dplane, int npx, const unsigned (&bf)[9][2]) {
#pragma unroll 3
  for (int sb = 0; sb < nslab; ++sb) {
    unsigned a[4];  // A = the slab's 16 channels x 16 cells
    ldmatrix_x4(a, bkp + sb * 16 * kBankPitch);
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int fh = 0; fh < 3; ++fh) {
      // the six halves from source column ow*S - 2 on, of channel rows gq (w) and gq + 8 (v)
      const unsigned* p0 = reinterpret_cast<const unsigned*>(xr[fh] + sb * 16 * INNER);
      const unsigned* p1 = p0 + 8 * INNER / 2;
      const unsigned w0 = p0[0], w1 = p0[1], w2 = p0[2];
      const unsigned v0 = p1[0], v1 = p1[1], v2 = p1[2];
      tap_row<S, TR, 0>(acc, a, bf[fh * 3 + 0], w0, w1, w2, v0, v1, v2);
      tap_row<S, TR, 1>(acc, a, bf[fh * 3 + 1], w0, w1, w2, v0, v1, v2);
      tap_row<S, TR, 2>(acc, a, bf[fh * 3 + 2], w0, w1, w2, v0, v1, v2);
    }
    __half* ya = y0 + (size_t)sb * 16 * dplane;
    if (PAIRS) {
      if (npx) {
        *reinterpret_cast<__half2*>(ya) = __floats2half2_rn(acc[0], acc[1]);
        *reinterpret_cast<__half2*>(ya + 8 * dplane) = __floats2half2_rn(acc[2], acc[3]);
      }
    } else {
      if (npx > 0) {
        ya[0] = __float2half_rn(acc[0]);
        ya[8 * dplane] = __float2half_rn(acc[2]);
      }
      if (npx > 1) {
        ya[1] = __float2half_rn(acc[1]);
        ya[8 * dplane + 1] = __float2half_rn(acc[3]);
      }
    }
  }
}

// ================================================================== forward (TR = false) and grad-input at stride 1 (TR = true)
//
// Destination pixel (d, ow) of channel c:  sum over taps of src[c, d*S - 1 + fh, ow*S - 1 + fw] * K[c, (d, ow), tap]   (forward)
//                                          sum over taps of src[c, d + 1 - fh, ow + 1 - fw] * K[c, (d+1-fh, ow+1-fw), tap]  (TR)
// The block's source rows form one stream: sample after sample, per sample the L rows
// -1 .. (Hd-1)*S + 1 (rows outside the plane arrive as zeros).  Stream row T is fill T - T0 of the source ring.
template <int S, int W, bool TR>
struct ConvShape {
  static constexpr int kWd = TR ? W : (W - 1) / S + 1;  // destination width
  static constexpr int kWr = TR ? W : kWd;              // width of the offset planes
  static constexpr int kNB = (kWd + 7) / 8;             // items (8 destination pixels) per row
  static constexpr int kInner = RowLayout<W>::kInner;
  static constexpr bool kTma = RowLayout<W>::kTma;
};

__host__ __device__ inline size_t conv_ring_smem(int cg, int inner, int rot_slot, int R, int RR) {
  return (size_t)R * cg * inner * 2 + 32 + (size_t)RR * rot_slot * 2 + (size_t)cg * kBankPitch * 2 + (size_t)(2 * R + 2 * RR) * 8 +
         16 + 128;
}

template <int S, int W, bool TR, bool SC44, int MAXT>
__global__ void __launch_bounds__(MAXT, 1) ring_conv_kernel(const __grid_constant__ CUtensorMap tm_src, const __half* __restrict__ src,
                                                            const __half* __restrict__ rot, const __half* __restrict__ bankw,
                                                            __half* __restrict__ dst, const RingParams p) {
  using Sh = ConvShape<S, W, TR>;
  using RL = RotLayout<Sh::kWr>;
  constexpr int INNER = Sh::kInner, WOP = RL::kWop, NB = Sh::kNB, Wd = Sh::kWd;
  static_assert(!TR || S == 1, "the transposed form of this kernel is the stride-1 one");
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int R = p.R, RR = p.RR;
  const int CG = p.CG;
  const int c0 = blockIdx.y * CG;
  const int slot_halves = CG * INNER;

  __half* xring = reinterpret_cast<__half*>(smem_raw);
  __half* rring = xring + (size_t)R * slot_halves + 16;
  __half* bank = rring + (size_t)RR * RL::kSlot;
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(
      (reinterpret_cast<uintptr_t>(bank + (size_t)CG * kBankPitch) + 7) & ~(uintptr_t)7);
  Ring rx, rr;
  rx.full = smem_u32(bars); rx.empty = rx.full + 8 * R; rx.set_slots(p.R);
  rr.full = rx.empty + 8 * R; rr.empty = rr.full + 8 * RR; rr.set_slots(p.RR);
  rx.issued = rr.empty + 8 * RR; rr.issued = rx.issued + 4;

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int np = p.NP, ncw = (blockDim.x >> 5) - np;

  // ---- set-up: barriers, zeroed rings (pads and the tail must read as zero from the start), bank copy
  if (threadIdx.x == 0) {
    for (int i = 0; i < R; ++i) {
      mbar_init(rx.full + 8 * i, Sh::kTma ? 1 : 32 * np);
      mbar_init(rx.empty + 8 * i, (S == 1 ? 3 : 2) * NB);
    }
    for (int i = 0; i < RR; ++i) {
      mbar_init(rr.full + 8 * i, 32 * np);
      mbar_init(rr.empty + 8 * i, (TR ? 3 : 1) * NB);
    }
    int* cnt = reinterpret_cast<int*>(bars + 2 * R + 2 * RR);
    cnt[0] = cnt[1] = 0;
    fence_barrier_init();
  }
  {
    uint4* z = reinterpret_cast<uint4*>(smem_raw);
    const int nz = (int)((reinterpret_cast<unsigned char*>(bank) - smem_raw) >> 4);
    for (int i = threadIdx.x; i < nz; i += blockDim.x) z[i] = make_uint4(0, 0, 0, 0);
  }
  for (int i = threadIdx.x; i < CG * 16; i += blockDim.x) {
    const int j = i >> 4, cell = i & 15;
    bank[j * kBankPitch + cell] = cell < p.cells ? __ldg(bankw + (size_t)(c0 + j) * p.cells + cell) : __float2half(0.f);
  }
  fence_proxy_async();
  __syncthreads();

  const int g0 = blockIdx.x * p.rows_per_block;
  const int g1 = min(g0 + p.rows_per_block, p.rows_total);
  if (g0 >= g1) return;
  const int Hd = p.Hd, L = p.L;
  const int n_first = g0 / Hd;
  const int T0 = n_first * L + (g0 - n_first * Hd) * S;

  if (warp < np) {
    // ------------------------------------------------------------ producers
    const int pw = warp;
    if (lane == 0 && Sh::kTma) prefetch_tensormap(&tm_src);
    const unsigned slot_bytes = (unsigned)slot_halves * 2;
    const unsigned xring_u32 = smem_u32(xring);
    int T = T0;
    bool ok = true;
    for (int g = g0; g < g1 && ok; ++g) {
      const int n = g / Hd, d = g - n * Hd;
      if (!TR) {
        const int kr = g - g0;
        ok = rr.reclaim(kr, lane, pw == 0);
        if (ok) fill_rot_row<Sh::kWr>(rring + (size_t)rr.slot(kr) * RL::kSlot, rot, n, Hd, d, lane, rr.full + 8 * rr.slot(kr), pw, np);
      }
      const int Tend = n * L + d * S + 2;
      for (; T <= Tend && ok; ++T) {
        const int k = T - T0;
        const int r = T - n * L - 1;  // source row; -1 and >= Hs arrive as zero rows
        if (TR) {
          ok = rr.reclaim(k, lane, pw == 0);
          if (ok)
            fill_rot_row<Sh::kWr>(rring + (size_t)rr.slot(k) * RL::kSlot, rot, n, p.Hs, min(max(r, 0), p.Hs - 1), lane,
                                  rr.full + 8 * rr.slot(k), pw, np);
        }
        ok = ok && rx.reclaim(k, lane, pw == 0);
        if (ok)
          fill_src_row<W>(xring + (size_t)rx.slot(k) * slot_halves, xring_u32 + rx.slot(k) * slot_bytes, slot_bytes, &tm_src, src, n,
                          p.C, c0, CG, p.Hs, r, lane, rx.full + 8 * rx.slot(k), pw, np);
        __syncwarp();
      }
    }
    cp_async_wait_all();
    if (!ok) ring_fail(lane);
    return;
  }

  // -------------------------------------------------------------- consumers
  const int cw = warp - np;
  const int gq = lane >> 2, q = lane & 3;
  const LaneCells lc = lane_cells_of(p.scW, p.cells, q);
  const float uh0 = (float)(p.scH - 3) * 0.5f, uw0 = (float)(p.scW - 3) * 0.5f;
  const int nslab = CG >> 4;
  const size_t dplane = (size_t)Hd * Wd;
  const int items = (g1 - g0) * NB;

  for (int it = cw; it < items; it += ncw) {
    const int grow = it / NB, cb = it - grow * NB;
    const int g = g0 + grow;
    const int n = g / Hd, d = g - n * Hd;
    const int k0 = n * L + d * S - T0;
    const int ow0 = cb << 3;
    const int pg = ow0 + gq;
    bool ok = true;
    float u, v;

    // hat products of the item's 72 (pixel, tap) pairs
    unsigned bf[9][2];
    if (!TR) {
      ok = rr.wait_full(grow);
      const __half* rp = rring + (size_t)rr.slot(grow) * RL::kSlot + 8 + pg;
#pragma unroll
      for (int t = 0; t < 9; ++t) beta_tap<WOP, SC44>(bf[t], rp + 2 * t * WOP, (float)(t / 3), (float)(t % 3), lc, uh0, uw0, u, v);
    } else {
      ok = rr.wait_full(k0 + 2);
#pragma unroll
      for (int fh = 0; fh < 3; ++fh) {
        const int k = k0 + 2 - fh;  // offsets of destination row d + 1 - fh
        if (fh) ok = rr.wait_full(k) && ok;
        const __half* rp = rring + (size_t)rr.slot(k) * RL::kSlot + 8 + pg + 1;
#pragma unroll
        for (int fw = 0; fw < 3; ++fw)
          beta_tap<WOP, SC44>(bf[fh * 3 + fw], rp + 2 * (fh * 3 + fw) * WOP - fw, (float)fh, (float)fw, lc, uh0, uw0, u, v);
      }
    }
    const __half* xr[3];
    ok = rx.wait_full(k0 + 2) && ok;
#pragma unroll
    for (int fh = 0; fh < 3; ++fh) {
      const int k = k0 + (TR ? 2 - fh : fh);
      if (k != k0 + 2) ok = rx.wait_full(k) && ok;
      xr[fh] = xring + (size_t)rx.slot(k) * slot_halves + gq * INNER + (8 + (ow0 + 2 * q) * S - 2);
    }
    if (!ok) {
      ring_fail(lane);
      return;
    }

    const int ow = ow0 + 2 * q;
    const __half* bkp = bank + ((lane & 7) + ((lane >> 3) & 1) * 8) * kBankPitch + (lane >> 4) * 8;  // this lane's ldmatrix row
    __half* y0 = dst + ((size_t)n * p.C + c0 + gq) * dplane + (size_t)d * Wd + ow;
    conv_slabs<S, INNER, TR, (Wd % 2 == 0)>(xr, bkp, y0, nslab, dplane, ow + 1 < Wd ? 2 : (ow < Wd ? 1 : 0), bf);

    // done with the three source rows (and the offset rows)
    __syncwarp();
    if (lane == 0) {
      const bool first = (d == 0) || (g == g0), last = (d == Hd - 1) || (g == g1 - 1);
#pragma unroll
      for (int j = 0; j < 3; ++j) {
        const int m = release_count<S>(j, first, last);
        rx.release(k0 + j, m);
        if (TR) rr.release(k0 + j, m);
      }
      if (!TR) rr.release(grow, 1);
    }
  }
}

// The channel-slab loop of the stride-2 grad-input for one item: dr[da] points at the lane's dy pair (channel row gq,
// column b) in the slot of output row a + da, x0 at dx (channel gq, row 2a, column 2b); bf holds the hat products of
// the nine (pixel shift, tap) pairs, index 3 * vr + vc with (da, fh) = (0,1), (0,2), (1,0) for vr = 0, 1, 2 and (db, fw) alike.
// Four consecutive dx values of one row (the first ncols of them exist), as wide as the row pitch of W halves allows.
template <int W>
__device__ __forceinline__ void store4(__half* __restrict__ p, const float (&v)[4], int ncols) {
  if (W % 4 == 0) {
    if (ncols > 0) {
      const __half2 lo = __floats2half2_rn(v[0], v[1]), hi = __floats2half2_rn(v[2], v[3]);
      *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const unsigned*>(&lo), *reinterpret_cast<const unsigned*>(&hi));
    }
  } else if (W % 2 == 0) {
    if (ncols > 0) *reinterpret_cast<__half2*>(p) = __floats2half2_rn(v[0], v[1]);
    if (ncols > 2) *reinterpret_cast<__half2*>(p + 2) = __floats2half2_rn(v[2], v[3]);
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (i < ncols) p[i] = __float2half_rn(v[i]);
  }
}

template <int INNER, int W>
__device__ __forceinline__ void convT2_slabs(const __half* const (&dr)[2], const __half* __restrict__ bkp, __half* __restrict__ x0,
                                             int nslab, size_t dplane, bool row1, int ncols, const unsigned (&bf)[9][2]) {
#pragma unroll 3
  for (int sb = 0; sb < nslab; ++sb) {
    unsigned af[4];  // A = the slab's 16 channels x 16 cells
    ldmatrix_x4(af, bkp + sb * 16 * kBankPitch);
    // dy of channel rows gq (wa) and gq + 8 (wb): [da][word] = columns (b, b+1), (b+2, .)
    unsigned wa[2][2], wb[2][2];
#pragma unroll
    for (int da = 0; da < 2; ++da) {
      const unsigned* p0 = reinterpret_cast<const unsigned*>(dr[da] + sb * 16 * INNER);
      const unsigned* p1 = p0 + 8 * INNER / 2;
      wa[da][0] = p0[0]; wa[da][1] = p0[1]; wb[da][0] = p1[0]; wb[da][1] = p1[1];
    }
    float acc[2][2][4];  // [channel row][rr][dx columns 2b .. 2b+3]
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[0][0][i] = acc[0][1][i] = acc[1][0][i] = acc[1][1][i] = 0.f;
#pragma unroll
    for (int vr = 0; vr < 3; ++vr) {
      const int da = vr == 2 ? 1 : 0, rr_ = vr == 0 ? 0 : 1;
#pragma unroll
      for (int vc = 0; vc < 3; ++vc) {
        const int cc = vc == 0 ? 0 : 1;
        unsigned kh[2];
        mma_h_new(kh, af, bf[vr * 3 + vc][0], bf[vr * 3 + vc][1]);
        if (vc != 2) {  // db = 0: pixel 0 reads column b (word 0 low), pixel 1 column b + 1 (word 0 high)
          fma_hh<0, 0>(acc[0][rr_][cc], wa[da][0], kh[0]); fma_hh<1, 1>(acc[0][rr_][2 + cc], wa[da][0], kh[0]);
          fma_hh<0, 0>(acc[1][rr_][cc], wb[da][0], kh[1]); fma_hh<1, 1>(acc[1][rr_][2 + cc], wb[da][0], kh[1]);
        } else {        // db = 1: columns b + 1 (word 0 high) and b + 2 (word 1 low)
          fma_hh<1, 0>(acc[0][rr_][cc], wa[da][0], kh[0]); fma_hh<0, 1>(acc[0][rr_][2 + cc], wa[da][1], kh[0]);
          fma_hh<1, 0>(acc[1][rr_][cc], wb[da][0], kh[1]); fma_hh<0, 1>(acc[1][rr_][2 + cc], wb[da][1], kh[1]);
        }
      }
    }
    // dx columns 2b .. 2b+3 of rows 2a (and 2a+1 when it exists) for both channel rows
#pragma unroll
    for (int ch = 0; ch < 2; ++ch) {
      __half* xa = x0 + ((size_t)sb * 16 + ch * 8) * dplane;
      store4<W>(xa, acc[ch][0], ncols);
      if (row1) store4<W>(xa + W, acc[ch][1], ncols);
    }
  }
}

// ================================================================== grad-input at stride 2
//
// dx[2a + rr, 2b + cc] collects, from the output pixels (a + da, b + db) with da, db in {0, 1}, the taps
//   rows: rr = 0 <- (da 0, fh 1);  rr = 1 <- (da 0, fh 2) and (da 1, fh 0)        (columns alike with db, fw, cc)
// so an item of 8 output pixels (a, b0 .. b0+7) yields the 2 x 16 patch dx[2a .. 2a+1, 2 b0 .. 2 b0 + 15] from nine
// (pixel shift, tap) pairs, all of them useful: one mma and 4 FMAs per lane each, as in the forward pass.  The
// rows a and a + 1 of dy and of the offsets stream through two rings (row Ho of a sample is a zero row).
template <int W>  // W = width of dx
struct ConvT2Shape {
  static constexpr int kWo = (W - 1) / 2 + 1;
  static constexpr int kNB = (kWo + 7) / 8;
  static constexpr int kInner = RowLayout<kWo>::kInner;
  static constexpr bool kTma = RowLayout<kWo>::kTma;
};

template <int W, bool SC44, int MAXT>
__global__ void __launch_bounds__(MAXT, 1) ring_convT2_kernel(const __grid_constant__ CUtensorMap tm_dy, const __half* __restrict__ dy,
                                                              const __half* __restrict__ rot, const __half* __restrict__ bankw,
                                                              __half* __restrict__ dx, const RingParams p) {
  using Sh = ConvT2Shape<W>;
  using RL = RotLayout<Sh::kWo>;
  constexpr int INNER = Sh::kInner, WOP = RL::kWop, NB = Sh::kNB, Wo = Sh::kWo;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int R = p.R;  // both rings have R slots and share their fill numbers
  const int CG = p.CG;
  const int c0 = blockIdx.y * CG;
  const int slot_halves = CG * INNER;

  __half* dring = reinterpret_cast<__half*>(smem_raw);
  __half* rring = dring + (size_t)R * slot_halves + 64;
  __half* bank = rring + (size_t)R * RL::kSlot;
  const unsigned bars_off = (unsigned)((((size_t)R * slot_halves + 64 + (size_t)R * RL::kSlot + (size_t)CG * kBankPitch) * 2 + 7) & ~(size_t)7);
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem_raw + bars_off);
  Ring rd, rr;
  rd.full = smem_u32(bars); rd.empty = rd.full + 8 * R; rd.set_slots(p.R);
  rr.full = rd.empty + 8 * R; rr.empty = rr.full + 8 * R; rr.set_slots(p.R);
  rd.issued = rr.empty + 8 * R; rr.issued = rd.issued + 4;

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int np = p.NP, ncw = (blockDim.x >> 5) - np;

  if (threadIdx.x == 0) {
    for (int i = 0; i < R; ++i) {
      mbar_init(rd.full + 8 * i, Sh::kTma ? 1 : 32 * np);
      mbar_init(rd.empty + 8 * i, 2 * NB);
      mbar_init(rr.full + 8 * i, 32 * np);
      mbar_init(rr.empty + 8 * i, 2 * NB);
    }
    int* cnt = reinterpret_cast<int*>(bars + 4 * R);
    cnt[0] = cnt[1] = 0;
    fence_barrier_init();
  }
  {
    uint4* z = reinterpret_cast<uint4*>(smem_raw);
    const int nz = (int)((reinterpret_cast<unsigned char*>(bank) - smem_raw) >> 4);
    for (int i = threadIdx.x; i < nz; i += blockDim.x) z[i] = make_uint4(0, 0, 0, 0);
  }
  for (int i = threadIdx.x; i < CG * 16; i += blockDim.x) {
    const int j = i >> 4, cell = i & 15;
    bank[j * kBankPitch + cell] = cell < p.cells ? __ldg(bankw + (size_t)(c0 + j) * p.cells + cell) : __float2half(0.f);
  }
  fence_proxy_async();
  __syncthreads();

  const int Ho = p.Hs, H = p.Hd, L = p.L;  // L = Ho + 1 stream rows per sample
  const int g0 = blockIdx.x * p.rows_per_block;  // rows of the OUTPUT plane (a) that this block expands
  const int g1 = min(g0 + p.rows_per_block, p.rows_total);
  if (g0 >= g1) return;
  const int n_first = g0 / Ho;
  const int T0 = n_first * L + (g0 - n_first * Ho);

  if (warp < np) {
    // ------------------------------------------------------------ producers
    const int pw = warp;
    if (lane == 0 && Sh::kTma) prefetch_tensormap(&tm_dy);
    const unsigned slot_bytes = (unsigned)slot_halves * 2;
    const unsigned dring_u32 = smem_u32(dring);
    int T = T0;
    bool ok = true;
    for (int g = g0; g < g1 && ok; ++g) {
      const int n = g / Ho, a = g - n * Ho;
      const int Tend = n * L + a + 1;
      for (; T <= Tend && ok; ++T) {
        const int k = T - T0;
        const int r = T - n * L;  // row of dy and of the offsets; r = Ho is the zero row below the plane
        ok = rr.reclaim(k, lane, pw == 0);
        if (ok) fill_rot_row<Wo>(rring + (size_t)rr.slot(k) * RL::kSlot, rot, n, Ho, min(r, Ho - 1), lane, rr.full + 8 * rr.slot(k), pw, np);
        ok = ok && rd.reclaim(k, lane, pw == 0);
        if (ok)
          fill_src_row<Wo>(dring + (size_t)rd.slot(k) * slot_halves, dring_u32 + rd.slot(k) * slot_bytes, slot_bytes, &tm_dy, dy, n, p.C,
                           c0, CG, Ho, r, lane, rd.full + 8 * rd.slot(k), pw, np);
        __syncwarp();
      }
    }
    cp_async_wait_all();
    if (!ok) ring_fail(lane);
    return;
  }

  // -------------------------------------------------------------- consumers
  const int cw = warp - np;
  const int gq = lane >> 2, q = lane & 3;
  const LaneCells lc = lane_cells_of(p.scW, p.cells, q);
  const float uh0 = (float)(p.scH - 3) * 0.5f, uw0 = (float)(p.scW - 3) * 0.5f;
  const int nslab = CG >> 4;
  const size_t dplane = (size_t)H * W;
  const int items = (g1 - g0) * NB;

  for (int it = cw; it < items; it += ncw) {
    const int grow = it / NB, cb = it - grow * NB;
    const int g = g0 + grow;
    const int n = g / Ho, a = g - n * Ho;
    const int k0 = n * L + a - T0;
    const int b0 = cb << 3;
    const int pg = b0 + gq;
    bool ok = rr.wait_full(k0 + 1);
    ok = rr.wait_full(k0) && ok;
    float u, v;

    // hat products of the nine (pixel shift, tap) pairs: index vt = 3 * vr + vc, with (da, fh) = (0,1), (0,2), (1,0) for
    // vr = 0, 1, 2 and (db, fw) alike for vc
    unsigned bf[9][2];
#pragma unroll
    for (int vr = 0; vr < 3; ++vr) {
      const int da = vr == 2 ? 1 : 0, fh = vr == 2 ? 0 : vr + 1;
      const __half* rp = rring + (size_t)rr.slot(k0 + da) * RL::kSlot + 8 + pg;
#pragma unroll
      for (int vc = 0; vc < 3; ++vc) {
        const int db = vc == 2 ? 1 : 0, fw = vc == 2 ? 0 : vc + 1;
        beta_tap<WOP, SC44>(bf[vr * 3 + vc], rp + 2 * (fh * 3 + fw) * WOP + db, (float)fh, (float)fw, lc, uh0, uw0, u, v);
      }
    }
    ok = rd.wait_full(k0 + 1) && ok;
    ok = rd.wait_full(k0) && ok;
    if (!ok) {
      ring_fail(lane);
      return;
    }
    const int b = b0 + 2 * q;
    const __half* dr[2];
#pragma unroll
    for (int da = 0; da < 2; ++da) dr[da] = dring + (size_t)rd.slot(k0 + da) * slot_halves + gq * INNER + 8 + b;

    const __half* bkp = bank + ((lane & 7) + ((lane >> 3) & 1) * 8) * kBankPitch + (lane >> 4) * 8;  // this lane's ldmatrix row
    __half* x0 = dx + ((size_t)n * p.C + c0 + gq) * dplane + (size_t)(2 * a) * W + 2 * b;
    const bool row1 = 2 * a + 1 < H;
    convT2_slabs<INNER, W>(dr, bkp, x0, nslab, dplane, row1, min(max(W - 2 * b, 0), 4), bf);
    // every stream row is read by the output rows a - 1 and a; the first / last row of the range stands in for a missing neighbour
    __syncwarp();
    if (lane == 0) {
      const bool first = (a == 0) || (g == g0), last = (a == Ho - 1) || (g == g1 - 1);
      rd.release(k0, first ? 2 : 1);
      rr.release(k0, first ? 2 : 1);
      rd.release(k0 + 1, last ? 2 : 1);
      rr.release(k0 + 1, last ? 2 : 1);
    }
  }
}

// grad-offsets and grad-bank of one item (8 output pixels ow0 .. ow0+7 of one row): three passes, one per kernel row fh
// (three taps), which keeps 12 instead of 36 accumulators of G live and waits for a source row only when its pass starts.
//   rp    the item's offsets in the ring slot of its row (plane 0, pixel ow0 + gq)
//   dyr   the lane's dy pair (channel row gq, pixels ow0 + 2q, + 1) in the slot of that row
//   x rows: fills kx0 .. kx0 + 2 of ring rx (slots of xslot halves in xring)
//   acc   the warp's bank-gradient accumulators; Gs / uv the warp's scratch; drot_item -> d(offsets)[n, 0, oh, ow0], or, when
//         the block holds only a group of the channels, gpart_item -> the same element of the group's fp32 partial sums
// Returns false when a wait ran out.  The caller releases the rows afterwards.
template <int S, int W, int NS, bool SC44, bool PADG>
__device__ __forceinline__ bool gw_item(float (&acc)[NS][2][4], const Ring& rx, int kx0, const __half* __restrict__ xring, int xslot,
                                        const __half* __restrict__ rp, const __half* __restrict__ dyr,
                                        const __half* __restrict__ bankT, int pitchT, float* __restrict__ Gs,
                                        float2* __restrict__ uv, __half* __restrict__ drot_item, float* __restrict__ gpart_item,
                                        int P, int nslab, int ow0, const LaneCells& lc, float uh0, float uw0, int scH_rt,
                                        int scW_rt, int lane) {
  constexpr int Wo = (W - 1) / S + 1;
  constexpr int IX = RowLayout<W>::kInner, ID = RowLayout<Wo>::kInner, WOP = RotLayout<Wo>::kWop;
  const int gq = lane >> 2, q = lane & 3;
  const int ow = ow0 + 2 * q;
  const __half* wtp = bankT + ((lane & 7) + ((lane >> 3) & 1) * 8) * pitchT + (lane >> 4) * 8;  // this lane's ldmatrix row
#pragma unroll
  for (int fh = 0; fh < 3; ++fh) {
    // hat products of the three taps, transposed into B fragments of dW += dK * beta:
    // bw[fw][0] = (pixels 2q, 2q+1; cell gq), bw[fw][1] = cell gq + 8
    unsigned bw[3][2];
#pragma unroll
    for (int fw = 0; fw < 3; ++fw) {
      unsigned bb[2];
      float u, v;
      beta_tap<WOP, SC44>(bb, rp + 2 * (fh * 3 + fw) * WOP, (float)fh, (float)fw, lc, uh0, uw0, u, v);
      bw[fw][0] = movmatrix_trans(bb[0]);
      bw[fw][1] = movmatrix_trans(bb[1]);
      if (q == 0) uv[fw * 8 + gq] = make_float2(u, v);
    }
    if (!rx.wait_full(kx0 + fh)) return false;
    const __half* xr = xring + (size_t)rx.slot(kx0 + fh) * xslot + gq * IX + (8 + ow * S - 2);

    float G[3][4];
#pragma unroll
    for (int t = 0; t < 3; ++t) G[t][0] = G[t][1] = G[t][2] = G[t][3] = 0.f;

#pragma unroll
    for (int sidx = 0; sidx < NS; ++sidx) {
      if (sidx < nslab) {
        const unsigned dy0 = *reinterpret_cast<const unsigned*>(dyr + sidx * 16 * ID);
        const unsigned dy1 = *reinterpret_cast<const unsigned*>(dyr + sidx * 16 * ID + 8 * ID);
        const unsigned* p0 = reinterpret_cast<const unsigned*>(xr + sidx * 16 * IX);
        const unsigned* p1 = p0 + 8 * IX / 2;
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
        ldmatrix_x4(a, wtp + sidx * 16);
#pragma unroll
        for (int fw = 0; fw < 3; ++fw) mma16816_acc(G[fw], a[0], a[1], a[2], a[3], movmatrix_trans(d0[fw]), movmatrix_trans(d1[fw]));
        // k = 16 = 8 pixels x (tap 0 | tap 1), then 8 pixels x (tap 2 | nothing)
        mma16816_acc(acc[sidx][0], d0[0], d1[0], d0[1], d1[1], bw[0][0], bw[1][0]);
        mma16816_acc(acc[sidx][1], d0[0], d1[0], d0[1], d1[1], bw[0][1], bw[1][1]);
        mma16816_acc(acc[sidx][0], d0[2], d1[2], 0u, 0u, bw[2][0], 0u);
        mma16816_acc(acc[sidx][1], d0[2], d1[2], 0u, 0u, bw[2][1], 0u);
      }
    }

    // d(offset)[pixel, tap, dir] = sum over the four corner cells of G * d(coefficient)/d(u or v).  Floor-based, so at an
    // integer coordinate it is the right-hand derivative and at the upper edge the derivative into the zero extension
    // (csrc/filter_sample_depthwise_cuda_kernel.cu:137-158); zero when the tap samples outside the bank (:131-135).
    // PADG (4 x 4 scope): G goes into a 6 x 6 grid per (tap, pixel) whose border cells stay zero from the start of the
    // kernel, so the four corners are read without range checks (3.6 instead of 1.7 KB of scratch per warp).
    __syncwarp();
    constexpr int GC = PADG ? 36 : 16;  // cells per tap in the scratch grid
    if (SC44 && PADG) {
      const int pc = ((gq >> 2) + 1) * 6 + (gq & 3) + 1;  // cell gq in the padded grid; cell gq + 8 lies two rows further
#pragma unroll
      for (int tt = 0; tt < 3; ++tt) {
        *reinterpret_cast<float2*>(Gs + (tt * 36 + pc) * 8 + 2 * q) = make_float2(G[tt][0], G[tt][1]);
        *reinterpret_cast<float2*>(Gs + (tt * 36 + pc + 12) * 8 + 2 * q) = make_float2(G[tt][2], G[tt][3]);
      }
    } else {
#pragma unroll
      for (int tt = 0; tt < 3; ++tt) {
        *reinterpret_cast<float2*>(Gs + (tt * GC + gq) * 8 + 2 * q) = make_float2(G[tt][0], G[tt][1]);
        *reinterpret_cast<float2*>(Gs + (tt * GC + gq + 8) * 8 + 2 * q) = make_float2(G[tt][2], G[tt][3]);
      }
    }
    __syncwarp();
    if (lane < 24) {
      const int px = lane & 7, tt = lane >> 3;
      const float2 c = uv[tt * 8 + px];
      const int scH = SC44 ? 4 : scH_rt, scW = SC44 ? 4 : scW_rt;
      const bool valid = c.x > -1.f && c.y > -1.f && c.x < (float)scH && c.y < (float)scW;
      float gu, gv;
      if (SC44 && PADG) {
        const float uc = valid ? c.x : 0.f, vc = valid ? c.y : 0.f;  // floor in -1 .. 3: both corner rows inside the grid
        const float fu = floorf(uc), fv = floorf(vc);
        const float lh = uc - fu, lw = vc - fv;
        const float hh = 1.f - lh, hw = 1.f - lw;
        const float* Gp = Gs + (tt * 36 + ((int)fu + 1) * 6 + (int)fv + 1) * 8 + px;
        const float g00 = Gp[0], g01 = Gp[8], g10 = Gp[48], g11 = Gp[56];
        gu = hw * (g10 - g00) + lw * (g11 - g01);
        gv = hh * (g01 - g00) + lh * (g11 - g10);
      } else {
        const float fu = floorf(c.x), fv = floorf(c.y);
        const float lh = c.x - fu, lw = c.y - fv;
        const float hh = 1.f - lh, hw = 1.f - lw;
        // corner rows h0, h0+1 and columns w0, w0+1, clamped into the bank for the loads; a corner outside counts as 0
        const int h0 = (int)fmaxf(fminf(fu, (float)scH), -2.f), w0 = (int)fmaxf(fminf(fv, (float)scW), -2.f);
        const bool r0 = h0 >= 0 && h0 < scH, r1 = h0 + 1 >= 0 && h0 + 1 < scH;
        const bool c0 = w0 >= 0 && w0 < scW, c1 = w0 + 1 >= 0 && w0 + 1 < scW;
        const int ra = min(max(h0, 0), scH - 1) * scW, rb = min(max(h0 + 1, 0), scH - 1) * scW;
        const int ca = min(max(w0, 0), scW - 1), cb2 = min(max(w0 + 1, 0), scW - 1);
        const float* Gp = Gs + tt * (GC * 8) + px;
        const float g00 = (r0 && c0) ? Gp[(ra + ca) * 8] : 0.f, g01 = (r0 && c1) ? Gp[(ra + cb2) * 8] : 0.f;
        const float g10 = (r1 && c0) ? Gp[(rb + ca) * 8] : 0.f, g11 = (r1 && c1) ? Gp[(rb + cb2) * 8] : 0.f;
        gu = hw * (g10 - g00) + lw * (g11 - g01);
        gv = hh * (g01 - g00) + lh * (g11 - g10);
      }
      if (!valid) gu = gv = 0.f;
      if (ow0 + px < Wo) {
        const int off = (2 * (fh * 3 + tt)) * P + px;
        if (gpart_item != nullptr) {
          gpart_item[off] = gu;
          gpart_item[off + P] = gv;
        } else {
          drot_item[off] = __float2half_rn(gu);
          drot_item[off + P] = __float2half_rn(gv);
        }
      }
    }
    __syncwarp();
  }
  return true;
}

// End of a block of the bank-gradient kernels: the consumer warps (cw = 0 .. ncw-1; all of them must call this) sum their
// accumulators through shared memory (red: [ncw][CG][16] floats, reusing the rings, which are idle by now) and write the
// block's partial sums out[CG][16].
template <int NS>
__device__ __forceinline__ void reduce_bank_accumulators(const float (&acc)[NS][2][4], float* __restrict__ red, float* __restrict__ out,
                                                         int CG, int nslab, int cw, int ncw, int lane) {
  const int gq = lane >> 2, q = lane & 3;
  asm volatile("bar.sync 1, %0;\n" ::"r"(ncw * 32) : "memory");
#pragma unroll
  for (int sidx = 0; sidx < NS; ++sidx) {
    if (sidx < nslab) {
      float* r0 = red + ((size_t)cw * CG + (sidx << 4) + gq) * 16;
      float* r1 = r0 + 8 * 16;
      r0[2 * q] = acc[sidx][0][0]; r0[2 * q + 1] = acc[sidx][0][1];
      r1[2 * q] = acc[sidx][0][2]; r1[2 * q + 1] = acc[sidx][0][3];
      r0[8 + 2 * q] = acc[sidx][1][0]; r0[8 + 2 * q + 1] = acc[sidx][1][1];
      r1[8 + 2 * q] = acc[sidx][1][2]; r1[8 + 2 * q + 1] = acc[sidx][1][3];
    }
  }
  asm volatile("bar.sync 1, %0;\n" ::"r"(ncw * 32) : "memory");
  for (int i = cw * 32 + lane; i < CG * 16; i += ncw * 32) {
    float sum = 0.f;
    for (int wv = 0; wv < ncw; ++wv) sum += red[(size_t)wv * CG * 16 + i];
    out[i] = sum;
  }
}

// ================================================================== grad-offsets + grad-bank in one pass
//
// Item = 8 output pixels (oh, ow0 .. ow0+7).  The warp that owns it runs over all channel slabs of the
// block: dK = dy * x (fp16 pairs), G += W^T * dK (all channels, complete inside the item), dW[slab] += dK * beta
// (kept in registers across the warp's items).  x rows stream as in the forward kernel; the rows of dy and of
// the offsets have their own rings, one fill per output row.
template <int S, int W>
struct GwShape {
  static constexpr int kWo = (W - 1) / S + 1;
  static constexpr int kNB = (kWo + 7) / 8;
  static constexpr int kInnerX = RowLayout<W>::kInner;
  static constexpr int kInnerD = RowLayout<kWo>::kInner;
  static constexpr bool kDyTma = RowLayout<kWo>::kTma;
};
constexpr int kGwScratch = 3 * 36 * 8 * 4 + 24 * 8;  // per warp: G of three taps x eight pixels on a 6 x 6 cell grid (zero border), and their bank coordinates (u, v)
constexpr int kBwdScratch = 3 * 16 * 8 * 4 + 24 * 8;  // the one-pass kernel, short of shared memory, keeps the 16 cells unpadded

__host__ __device__ inline size_t gw_ring_smem(int cg, int inner_x, int inner_d, int rot_slot, int R, int RR, int warps) {
  const size_t rings = (size_t)R * cg * inner_x * 2 + 128 + (size_t)RR * cg * inner_d * 2 + 128 + (size_t)RR * rot_slot * 2;
  const size_t red = (size_t)warps * cg * 16 * 4;  // the bank-gradient reduction at the end reuses the rings
  return (rings > red ? rings : red) + 16 + (size_t)16 * (cg + 8) * 2 + (size_t)warps * kGwScratch + (size_t)(2 * R + 4 * RR) * 8 +
         16 + 128;
}

template <int S, int W, int NS, bool SC44, int MAXT>
__global__ void __launch_bounds__(MAXT, 1) ring_gw_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_dy,
                                                          const __half* __restrict__ x, const __half* __restrict__ dy,
                                                          const __half* __restrict__ rot, const __half* __restrict__ bankw,
                                                          __half* __restrict__ drot, float* __restrict__ gpart,
                                                          float* __restrict__ partial, const RingParams p) {
  using Sh = GwShape<S, W>;
  using RL = RotLayout<Sh::kWo>;
  constexpr int IX = Sh::kInnerX, ID = Sh::kInnerD, NB = Sh::kNB, Wo = Sh::kWo;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int R = p.R, RR = p.RR;
  const int CG = p.CG;  // = 16 * (slabs <= NS): every channel, or (gpart != null) group blockIdx.y of them
  const int c0 = blockIdx.y * CG;
  const int xslot = CG * IX, dslot = CG * ID;
  const int np = p.NP, ncw = (blockDim.x >> 5) - np;
  const int pitchT = CG + 8;

  __half* xring = reinterpret_cast<__half*>(smem_raw);
  __half* dring = xring + (size_t)R * xslot + 64;  // 128 bytes of zeros behind each ring; TMA destinations stay 128-byte aligned
  __half* rring = dring + (size_t)RR * dslot + 64;
  // everything is addressed as smem_raw + offset, so that the compiler keeps using shared-memory loads and stores
  const unsigned rings_bytes = (unsigned)(((size_t)R * xslot + 64 + (size_t)RR * dslot + 64 + (size_t)RR * RL::kSlot) * 2);
  const unsigned red_bytes = (unsigned)ncw * CG * 16 * 4;
  const unsigned after = ((rings_bytes > red_bytes ? rings_bytes : red_bytes) + 15u) & ~15u;
  __half* bankT = reinterpret_cast<__half*>(smem_raw + after);  // [16 cells][CG + 8]
  const unsigned scratch_off = after + 16 * pitchT * 2;
  unsigned char* scratch = smem_raw + scratch_off;
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem_raw + ((scratch_off + (unsigned)ncw * kGwScratch + 7u) & ~7u));
  Ring rx, rd, rr;
  rx.full = smem_u32(bars); rx.empty = rx.full + 8 * R; rx.set_slots(p.R);
  rd.full = rx.empty + 8 * R; rd.empty = rd.full + 8 * RR; rd.set_slots(p.RR);
  rr.full = rd.empty + 8 * RR; rr.empty = rr.full + 8 * RR; rr.set_slots(p.RR);
  rx.issued = rr.empty + 8 * RR; rd.issued = rx.issued + 4; rr.issued = rx.issued + 8;

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  if (threadIdx.x == 0) {
    for (int i = 0; i < R; ++i) {
      mbar_init(rx.full + 8 * i, RowLayout<W>::kTma ? 1 : 32 * np);
      mbar_init(rx.empty + 8 * i, (S == 1 ? 3 : 2) * NB);
    }
    for (int i = 0; i < RR; ++i) {
      mbar_init(rd.full + 8 * i, Sh::kDyTma ? 1 : 32 * np);
      mbar_init(rd.empty + 8 * i, NB);
      mbar_init(rr.full + 8 * i, 32 * np);
      mbar_init(rr.empty + 8 * i, NB);
    }
    int* cnt = reinterpret_cast<int*>(bars + 2 * R + 4 * RR);
    cnt[0] = cnt[1] = cnt[2] = 0;
    fence_barrier_init();
  }
  {
    uint4* z = reinterpret_cast<uint4*>(smem_raw);
    const int nz = (int)(rings_bytes >> 4);
    for (int i = threadIdx.x; i < nz; i += blockDim.x) z[i] = make_uint4(0, 0, 0, 0);
    uint4* zs = reinterpret_cast<uint4*>(scratch);  // the border cells of the warps' G grids are never written again
    for (int i = threadIdx.x; i < ncw * (kGwScratch >> 4); i += blockDim.x) zs[i] = make_uint4(0, 0, 0, 0);
  }
  for (int i = threadIdx.x; i < 16 * CG; i += blockDim.x) {
    const int cell = i / CG, c = i - cell * CG;
    bankT[cell * pitchT + c] = cell < p.cells ? __ldg(bankw + (size_t)(c0 + c) * p.cells + cell) : __float2half(0.f);
  }
  fence_proxy_async();
  __syncthreads();

  const int g0 = blockIdx.x * p.rows_per_block;
  const int g1 = min(g0 + p.rows_per_block, p.rows_total);
  const int Ho = p.Hd, L = p.L;
  const int n_first = g0 < g1 ? g0 / Ho : 0;
  const int T0 = n_first * L + (g0 - n_first * Ho) * S;

  if (warp < np) {
    // ------------------------------------------------------------ producers
    const int pw = warp;
    if (g0 >= g1) return;
    if (lane == 0) {
      if (RowLayout<W>::kTma) prefetch_tensormap(&tm_x);
      if (Sh::kDyTma) prefetch_tensormap(&tm_dy);
    }
    const unsigned xbytes = (unsigned)xslot * 2, dbytes = (unsigned)dslot * 2;
    const unsigned xring_u32 = smem_u32(xring), dring_u32 = smem_u32(dring);
    int T = T0;
    bool ok = true;
    for (int g = g0; g < g1 && ok; ++g) {
      const int n = g / Ho, oh = g - n * Ho;
      const int kr = g - g0;
      ok = rr.reclaim(kr, lane, pw == 0);
      if (ok) fill_rot_row<Wo>(rring + (size_t)rr.slot(kr) * RL::kSlot, rot, n, Ho, oh, lane, rr.full + 8 * rr.slot(kr), pw, np);
      ok = ok && rd.reclaim(kr, lane, pw == 0);
      if (ok)
        fill_src_row<Wo>(dring + (size_t)rd.slot(kr) * dslot, dring_u32 + rd.slot(kr) * dbytes, dbytes, &tm_dy, dy, n, p.C, c0, CG, Ho,
                         oh, lane, rd.full + 8 * rd.slot(kr), pw, np);
      const int Tend = n * L + oh * S + 2;
      for (; T <= Tend && ok; ++T) {
        const int k = T - T0;
        ok = rx.reclaim(k, lane, pw == 0);
        if (ok)
          fill_src_row<W>(xring + (size_t)rx.slot(k) * xslot, xring_u32 + rx.slot(k) * xbytes, xbytes, &tm_x, x, n, p.C, c0, CG, p.Hs,
                          T - n * L - 1, lane, rx.full + 8 * rx.slot(k), pw, np);
        __syncwarp();
      }
    }
    cp_async_wait_all();
    if (!ok) ring_fail(lane);
    return;
  }

  // -------------------------------------------------------------- consumers
  const int cw = warp - np;
  const int gq = lane >> 2, q = lane & 3;
  const LaneCells lc = lane_cells_of(p.scW, p.cells, q);
  const float uh0 = (float)(p.scH - 3) * 0.5f, uw0 = (float)(p.scW - 3) * 0.5f;
  const int nslab = CG >> 4;
  const int items = g0 < g1 ? (g1 - g0) * NB : 0;
  const int P = Ho * Wo;
  float* Gs = reinterpret_cast<float*>(scratch + (size_t)cw * kGwScratch);  // [3 taps][36 cells][8 px]
  float2* uv = reinterpret_cast<float2*>(Gs + 3 * 36 * 8);                    // [3 taps][8 px]

  float acc[NS][2][4];  // bank gradient of up to NS slabs of 16 channels x (cells 0-7 | cells 8-15)
#pragma unroll
  for (int sidx = 0; sidx < NS; ++sidx)
#pragma unroll
    for (int k = 0; k < 4; ++k) acc[sidx][0][k] = acc[sidx][1][k] = 0.f;

  for (int it = cw; it < items; it += ncw) {
    const int grow = it / NB, cb = it - grow * NB;
    const int g = g0 + grow;
    const int n = g / Ho, oh = g - n * Ho;
    const int k0 = n * L + oh * S - T0;
    const int ow0 = cb << 3;
    const int pg = ow0 + gq;
    bool ok = rr.wait_full(grow);
    ok = rd.wait_full(grow) && ok;
    const int ow = ow0 + 2 * q;
    const __half* rp = rring + (size_t)rr.slot(grow) * RL::kSlot + 8 + pg;
    const __half* dyr = dring + (size_t)rd.slot(grow) * dslot + gq * ID + 8 + ow;
    __half* drot_item = drot + (size_t)n * 18 * P + oh * Wo + ow0;

    float* gpart_item = gpart != nullptr ? gpart + ((size_t)blockIdx.y * p.N + n) * 18 * P + oh * Wo + ow0 : nullptr;
    ok = gw_item<S, W, NS, SC44, true>(acc, rx, k0, xring, xslot, rp, dyr, bankT, pitchT, Gs, uv, drot_item, gpart_item, P, nslab, ow0, lc,
                                 uh0, uw0, p.scH, p.scW, lane) && ok;
    // the rows are no longer needed
    __syncwarp();
    if (lane == 0 && ok) {
      const bool first = (oh == 0) || (g == g0), last = (oh == Ho - 1) || (g == g1 - 1);
#pragma unroll
      for (int j = 0; j < 3; ++j) rx.release(k0 + j, release_count<S>(j, first, last));
      rd.release(grow, 1);
      rr.release(grow, 1);
    }
    if (!ok) {
      ring_fail(lane);
      break;
    }
  }

  // ---- bank gradient: sum the consumer warps' accumulators (the rings are free now) and write this block's partial
  reduce_bank_accumulators<NS>(acc, reinterpret_cast<float*>(smem_raw), partial + ((size_t)blockIdx.x * p.C + c0) * 16, CG, nslab, cw, ncw, lane);
}

// ================================================================== the whole backward in one pass
//
// grad-input, grad-offsets and grad-bank of one item by the same warp, back to back, from ONE stream of rows: every
// row of dy, of the offsets and of x crosses HBM and shared memory once for all three gradients.  Stride 1: the item at
// row j needs the rows j-1 .. j+1 of dy and of the offsets (grad-input, taps flipped) and of x (the products dy * x),
// i.e. the same three fills of all three rings.  Stride 2: grad-input expands output row j into dx rows 2j, 2j+1 from
// the rows j, j+1 of dy / offsets, the other two gradients read row j of those and rows 2j-1 .. 2j+1 of x.
template <int S, int W>
struct BwdShape {
  static constexpr int kWo = (W - 1) / S + 1;
  static constexpr int kNB = (kWo + 7) / 8;
  static constexpr int kInnerX = RowLayout<W>::kInner;
  static constexpr int kInnerD = RowLayout<kWo>::kInner;
  static constexpr bool kDyTma = RowLayout<kWo>::kTma;
  static constexpr int kUsersD = S == 1 ? 3 : 2;  // destination rows that read one row of dy / offsets
};

__host__ __device__ inline size_t bwd_ring_smem(int cg, int inner_x, int inner_d, int rot_slot, int Rx, int Rd, int warps) {
  const size_t rings = ((size_t)Rx * cg * inner_x + 64 + (size_t)Rd * cg * inner_d + 64 + (size_t)Rd * rot_slot) * 2;
  const size_t red = (size_t)warps * cg * 16 * 4;  // the bank-gradient reduction at the end reuses the rings
  return (rings > red ? rings : red) + 16 + (size_t)cg * kBankPitch * 2 + (size_t)16 * (cg + 8) * 2 + (size_t)warps * kBwdScratch +
         (size_t)(2 * Rx + 4 * Rd) * 8 + 16 + 128;
}

template <int S, int W, int NS, bool SC44, int MAXT>
__global__ void __launch_bounds__(MAXT, 1) ring_bwd_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_dy,
                                                           const __half* __restrict__ dy, const __half* __restrict__ rot,
                                                           const __half* __restrict__ bankw, __half* __restrict__ dx,
                                                           __half* __restrict__ drot, float* __restrict__ partial,
                                                           const RingParams p) {
  using Sh = BwdShape<S, W>;
  using RL = RotLayout<Sh::kWo>;
  constexpr int IX = Sh::kInnerX, ID = Sh::kInnerD, WOP = RL::kWop, NB = Sh::kNB, Wo = Sh::kWo;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int Rx = p.R, Rd = p.RR;
  const int CG = p.CG;  // every channel
  const int xslot = CG * IX, dslot = CG * ID;
  const int np = p.NP, ncw = (blockDim.x >> 5) - np;
  const int pitchT = CG + 8;

  __half* xring = reinterpret_cast<__half*>(smem_raw);
  __half* dring = xring + (size_t)Rx * xslot + 64;
  __half* rring = dring + (size_t)Rd * dslot + 64;
  const unsigned rings_bytes = (unsigned)(((size_t)Rx * xslot + 64 + (size_t)Rd * dslot + 64 + (size_t)Rd * RL::kSlot) * 2);
  const unsigned red_bytes = (unsigned)ncw * CG * 16 * 4;
  const unsigned after = ((rings_bytes > red_bytes ? rings_bytes : red_bytes) + 15u) & ~15u;
  __half* bank = reinterpret_cast<__half*>(smem_raw + after);                             // [CG][kBankPitch], for K = W * beta
  __half* bankT = bank + (size_t)CG * kBankPitch;                                         // [16 cells][CG + 8], for G = W^T * dK
  const unsigned scratch_off = after + (unsigned)(CG * kBankPitch + 16 * pitchT) * 2;
  unsigned char* scratch = smem_raw + scratch_off;
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem_raw + ((scratch_off + (unsigned)ncw * kBwdScratch + 7u) & ~7u));
  Ring rx, rd, rr;
  rx.full = smem_u32(bars); rx.empty = rx.full + 8 * Rx; rx.set_slots(p.R);
  rd.full = rx.empty + 8 * Rx; rd.empty = rd.full + 8 * Rd; rd.set_slots(p.RR);
  rr.full = rd.empty + 8 * Rd; rr.empty = rr.full + 8 * Rd; rr.set_slots(p.RR);
  rx.issued = rr.empty + 8 * Rd; rd.issued = rx.issued + 4; rr.issued = rx.issued + 8;

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  if (threadIdx.x == 0) {
    for (int i = 0; i < Rx; ++i) {
      mbar_init(rx.full + 8 * i, 1);
      mbar_init(rx.empty + 8 * i, (S == 1 ? 3 : 2) * NB);
    }
    for (int i = 0; i < Rd; ++i) {
      mbar_init(rd.full + 8 * i, Sh::kDyTma ? 1 : 32 * np);
      mbar_init(rd.empty + 8 * i, Sh::kUsersD * NB);
      mbar_init(rr.full + 8 * i, 32 * np);
      mbar_init(rr.empty + 8 * i, Sh::kUsersD * NB);
    }
    int* cnt = reinterpret_cast<int*>(bars + 2 * Rx + 4 * Rd);
    cnt[0] = cnt[1] = cnt[2] = 0;
    fence_barrier_init();
  }
  {
    uint4* z = reinterpret_cast<uint4*>(smem_raw);
    const int nz = (int)(rings_bytes >> 4);
    for (int i = threadIdx.x; i < nz; i += blockDim.x) z[i] = make_uint4(0, 0, 0, 0);
  }
  for (int i = threadIdx.x; i < 16 * CG; i += blockDim.x) {
    const int c = i >> 4, cell = i & 15;
    const __half v = cell < p.cells ? __ldg(bankw + (size_t)c * p.cells + cell) : __float2half(0.f);
    bank[c * kBankPitch + cell] = v;
    bankT[cell * pitchT + c] = v;
  }
  fence_proxy_async();
  __syncthreads();

  const int g0 = blockIdx.x * p.rows_per_block;
  const int g1 = min(g0 + p.rows_per_block, p.rows_total);
  const int Ho = p.Hs, H = p.Hd;        // rows of dy / offsets and of x / dx
  const int Lx = p.L;                   // stream rows of x per sample
  const int Ld = S == 1 ? Lx : Ho + 1;  // ... of dy and the offsets
  const int n_first = g0 < g1 ? g0 / Ho : 0;
  const int d_first = g0 - n_first * Ho;
  const int Tx0 = n_first * Lx + d_first * S;
  const int Td0 = n_first * Ld + d_first;

  if (warp < np) {
    // ------------------------------------------------------------ producers
    const int pw = warp;
    if (g0 >= g1) return;
    if (lane == 0) {
      prefetch_tensormap(&tm_x);
      if (Sh::kDyTma) prefetch_tensormap(&tm_dy);
    }
    const unsigned xbytes = (unsigned)xslot * 2, dbytes = (unsigned)dslot * 2;
    const unsigned xring_u32 = smem_u32(xring), dring_u32 = smem_u32(dring);
    int Tx = Tx0, Td = Td0;
    bool ok = true;
    for (int g = g0; g < g1 && ok; ++g) {
      const int n = g / Ho, j = g - n * Ho;
      const int Td_end = n * Ld + j + (S == 1 ? 2 : 1);
      for (; Td <= Td_end && ok; ++Td) {
        const int k = Td - Td0;
        const int r = Td - n * Ld - (S == 1 ? 1 : 0);  // row of dy / offsets; -1 and Ho are zero rows
        ok = rr.reclaim(k, lane, pw == 0);
        if (ok) fill_rot_row<Wo>(rring + (size_t)rr.slot(k) * RL::kSlot, rot, n, Ho, min(max(r, 0), Ho - 1), lane, rr.full + 8 * rr.slot(k), pw, np);
        ok = ok && rd.reclaim(k, lane, pw == 0);
        if (ok) {
          if (Sh::kDyTma) {
            if (lane == 0 && pw == 0) {
              mbar_arrive_expect_tx(rd.full + 8 * rd.slot(k), dbytes);
              tma_load_3d(dring_u32 + rd.slot(k) * dbytes, &tm_dy, -8, r, n * p.C, rd.full + 8 * rd.slot(k));
            }
          } else {
            __half* slot = dring + (size_t)rd.slot(k) * dslot;
            if (r >= 0 && r < Ho) {
              fill_plane_row<Wo>(slot, dy, n, p.C, 0, CG, Ho, r, lane, rd.full + 8 * rd.slot(k), pw, np);
            } else {  // a zero row: plain stores, then the same arrivals
              for (int i = lane + 32 * pw; i < dslot / 8; i += 32 * np) reinterpret_cast<uint4*>(slot)[i] = make_uint4(0, 0, 0, 0);
              mbar_arrive(rd.full + 8 * rd.slot(k));
            }
          }
        }
        __syncwarp();
      }
      const int Tx_end = n * Lx + j * S + 2;
      for (; Tx <= Tx_end && ok; ++Tx) {
        const int k = Tx - Tx0;
        ok = rx.reclaim(k, lane, pw == 0);
        if (lane == 0 && ok && pw == 0) {
          mbar_arrive_expect_tx(rx.full + 8 * rx.slot(k), xbytes);
          tma_load_3d(xring_u32 + rx.slot(k) * xbytes, &tm_x, -8, Tx - n * Lx - 1, n * p.C, rx.full + 8 * rx.slot(k));
        }
        __syncwarp();
      }
    }
    cp_async_wait_all();
    if (!ok) ring_fail(lane);
    return;
  }

  // -------------------------------------------------------------- consumers
  const int cw = warp - np;
  const int gq = lane >> 2, q = lane & 3;
  const LaneCells lc = lane_cells_of(p.scW, p.cells, q);
  const float uh0 = (float)(p.scH - 3) * 0.5f, uw0 = (float)(p.scW - 3) * 0.5f;
  const int nslab = CG >> 4;
  const int items = g0 < g1 ? (g1 - g0) * NB : 0;
  const int P = Ho * Wo;
  const size_t xplane = (size_t)H * W;
  float* Gs = reinterpret_cast<float*>(scratch + (size_t)cw * kBwdScratch);  // [3 taps][16 cells][8 px]
  float2* uv = reinterpret_cast<float2*>(Gs + 3 * 16 * 8);                    // [3 taps][8 px]
  const __half* bkp = bank + ((lane & 7) + ((lane >> 3) & 1) * 8) * kBankPitch + (lane >> 4) * 8;  // this lane's ldmatrix row

  float acc[NS][2][4];  // bank gradient of up to NS slabs of 16 channels x (cells 0-7 | cells 8-15)
#pragma unroll
  for (int sidx = 0; sidx < NS; ++sidx)
#pragma unroll
    for (int k = 0; k < 4; ++k) acc[sidx][0][k] = acc[sidx][1][k] = 0.f;

  bool failed = false;
  for (int it = cw; it < items; it += ncw) {
    const int grow = it / NB, cb = it - grow * NB;
    const int g = g0 + grow;
    const int n = g / Ho, j = g - n * Ho;
    const int kx0 = n * Lx + j * S - Tx0;
    const int kd0 = n * Ld + j - Td0;
    const int ow0 = cb << 3;
    const int pg = ow0 + gq;
    const int ow = ow0 + 2 * q;
    bool ok = true;
    float u, v;

    // ---- grad-input
    {
      unsigned bf[9][2];
      if (S == 1) {
        // dx[j, ow] = sum over taps of dy[j + 1 - fh, ow + 1 - fw] * K[(j + 1 - fh, ow + 1 - fw), tap]
        ok = rr.wait_full(kd0 + 2);
#pragma unroll
        for (int fh = 0; fh < 3; ++fh) {
          const int k = kd0 + 2 - fh;
          if (fh) ok = rr.wait_full(k) && ok;
          const __half* rq = rring + (size_t)rr.slot(k) * RL::kSlot + 8 + pg + 1;
#pragma unroll
          for (int fw = 0; fw < 3; ++fw)
            beta_tap<WOP, SC44>(bf[fh * 3 + fw], rq + 2 * (fh * 3 + fw) * WOP - fw, (float)fh, (float)fw, lc, uh0, uw0, u, v);
        }
        const __half* dr[3];
        ok = rd.wait_full(kd0 + 2) && ok;
#pragma unroll
        for (int fh = 0; fh < 3; ++fh) {
          const int k = kd0 + 2 - fh;
          if (fh) ok = rd.wait_full(k) && ok;
          dr[fh] = dring + (size_t)rd.slot(k) * dslot + gq * ID + (8 + ow - 2);
        }
        if (!ok) {
          failed = true;
          break;
        }
        __half* x0 = dx + ((size_t)n * p.C + gq) * xplane + (size_t)j * W + ow;
        conv_slabs<1, ID, true, true>(dr, bkp, x0, nslab, xplane, ow < W ? 2 : 0, bf);
      } else {
        ok = rr.wait_full(kd0 + 1);
        ok = rr.wait_full(kd0) && ok;
#pragma unroll
        for (int vr = 0; vr < 3; ++vr) {
          const int da = vr == 2 ? 1 : 0, fh = vr == 2 ? 0 : vr + 1;
          const __half* rq = rring + (size_t)rr.slot(kd0 + da) * RL::kSlot + 8 + pg;
#pragma unroll
          for (int vc = 0; vc < 3; ++vc) {
            const int db = vc == 2 ? 1 : 0, fw = vc == 2 ? 0 : vc + 1;
            beta_tap<WOP, SC44>(bf[vr * 3 + vc], rq + 2 * (fh * 3 + fw) * WOP + db, (float)fh, (float)fw, lc, uh0, uw0, u, v);
          }
        }
        ok = rd.wait_full(kd0 + 1) && ok;
        ok = rd.wait_full(kd0) && ok;
        if (!ok) {
          failed = true;
          break;
        }
        const __half* dr[2];
#pragma unroll
        for (int da = 0; da < 2; ++da) dr[da] = dring + (size_t)rd.slot(kd0 + da) * dslot + gq * ID + 8 + ow;
        __half* x0 = dx + ((size_t)n * p.C + gq) * xplane + (size_t)(2 * j) * W + 2 * ow;
        convT2_slabs<ID, W>(dr, bkp, x0, nslab, xplane, 2 * j + 1 < H, min(max(W - 2 * ow, 0), 4), bf);
      }
    }

    // ---- grad-offsets and grad-bank: row j of dy and of the offsets, rows j*S - 1 .. j*S + 1 of x
    {
      const int kr = S == 1 ? kd0 + 1 : kd0;
      const __half* rp = rring + (size_t)rr.slot(kr) * RL::kSlot + 8 + pg;
      const __half* dyr = dring + (size_t)rd.slot(kr) * dslot + gq * ID + 8 + ow;
      __half* drot_item = drot + (size_t)n * 18 * P + j * Wo + ow0;
      ok = gw_item<S, W, NS, SC44, false>(acc, rx, kx0, xring, xslot, rp, dyr, bankT, pitchT, Gs, uv, drot_item, nullptr, P, nslab, ow0, lc,
                                   uh0, uw0, p.scH, p.scW, lane);
      if (!ok) {
        failed = true;
        break;
      }
    }

    // every row the item read goes back to the producer
    __syncwarp();
    if (lane == 0) {
      const bool first = (j == 0) || (g == g0), last = (j == Ho - 1) || (g == g1 - 1);
#pragma unroll
      for (int i = 0; i < 3; ++i) {
        const int m = release_count<S>(i, first, last);
        rx.release(kx0 + i, m);
        if (S == 1) {
          rd.release(kd0 + i, m);
          rr.release(kd0 + i, m);
        }
      }
      if (S == 2) {
        rd.release(kd0, first ? 2 : 1);
        rr.release(kd0, first ? 2 : 1);
        rd.release(kd0 + 1, last ? 2 : 1);
        rr.release(kd0 + 1, last ? 2 : 1);
      }
    }
  }
  if (failed) ring_fail(lane);

  // ---- bank gradient: sum the consumer warps' accumulators (the rings are free now) and write this block's partial
  reduce_bank_accumulators<NS>(acc, reinterpret_cast<float*>(smem_raw), partial + (size_t)blockIdx.x * CG * 16, CG, nslab, cw, ncw, lane);
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver's tensor-map encoder, looked up through the runtime (the library links no driver library).
EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      ptr = nullptr;
    (void)cudaGetLastError();
    return reinterpret_cast<EncodeTiledFn>(ptr);
  }();
  return fn;
}

// fp16 planes [planes][rows][width] viewed as a rank-3 tensor; one box = `box_w` halves of one row of
// `box_planes` consecutive planes.  Elements outside the tensor are delivered as zeros.
bool make_row_map(CUtensorMap* tm, const __half* base, int width, int rows, long long planes, int box_w, int box_planes) {
  EncodeTiledFn enc = encode_tiled();
  if (!enc) return false;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (width & 7) || box_w > 256 || box_planes > 256 || (box_w & 7)) return false;
  const cuuint64_t dims[3] = {(cuuint64_t)width, (cuuint64_t)rows, (cuuint64_t)planes};
  const cuuint64_t strides[2] = {(cuuint64_t)width * 2, (cuuint64_t)width * rows * 2};
  const cuuint32_t box[3] = {(cuuint32_t)box_w, 1u, (cuuint32_t)box_planes};
  const cuuint32_t estr[3] = {1u, 1u, 1u};
  return enc(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<__half*>(base), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Input widths the kernels are instantiated for; scope 4 x 4.  The kernels themselves take any width: rows that are not
// multiples of 16 bytes come by cp.async pieces (28-wide rows: 8 bytes each, shared by several producer warps), odd ones
// element by element.  Which widths are routed here was decided by measurement on B200 (batch 128) against the band kernels
// of dk_local_mma.cu; the figures are at DK_RING_FOR_WIDE below.
#define DK_RING_FOR_WIDTH(WIDTH, CALL)        \
  switch (WIDTH) {                            \
    case 112: { constexpr int W = 112; CALL; } \
    case 56: { constexpr int W = 56; CALL; }   \
    case 28: { constexpr int W = 28; CALL; }   \
    default: return DK_ERR_UNSUPPORTED;       \
  }

// The widths whose stride-2 forward and offsets + bank passes run here.  28-wide planes at stride 2 have 14 x 14 outputs,
// two items per row of which one is three quarters empty: measured on B200 (C = 192, batch 128) the band kernels win the
// forward pass 0.027 to 0.034 ms and the offsets + bank pass 0.054 to 0.074; the ring kernel wins grad-input 0.025 to 0.041.
// At stride 1 the ring kernels win all three (0.052 / 0.054 / 0.123 against 0.059 / 0.057 / 0.145).  14-wide planes were
// measured too: the band kernels win everything there.
#define DK_RING_FOR_WIDE(WIDTH, CALL)         \
  switch (WIDTH) {                            \
    case 112: { constexpr int W = 112; CALL; } \
    case 56: { constexpr int W = 56; CALL; }   \
    default: return DK_ERR_UNSUPPORTED;       \
  }

bool ring_shape(const Geom& g) {
  if (g.kH != 3 || g.kW != 3 || g.dH != 1 || g.dW != 1 || g.pH != 1 || g.pW != 1) return false;
  if (g.sH != g.sW || (g.sH != 1 && g.sH != 2)) return false;
  if (g.G != 1 || g.scH != 4 || g.scW != 4 || (g.C & 15)) return false;
  if ((long long)g.N * (g.H + 2) > 0x3fffffff) return false;  // stream row indices are 32-bit
  return g.W == 112 || g.W == 56 || g.W == 28;
}

void spread_rows(long long rows, int groups, int* blocks_x, int* rows_per_block) {
  long long bx = device_sm_count() / groups;
  if (bx < 1) bx = 1;
  if (bx > rows) bx = rows;
  *rows_per_block = (int)((rows + bx - 1) / bx);
  *blocks_x = (int)((rows + *rows_per_block - 1) / *rows_per_block);
}

// ring depth for `rows` rows in flight: 4 .. 32 slots
int ring_slots(int rows) { return rows < 4 ? 4 : (rows > 32 ? 32 : rows); }
// the same, rounded up to a power of two: what a ring is given when shared memory is plentiful
int ring_slots_generous(int rows) {
  int r = 4;
  while (r < 32 && r < rows) r *= 2;
  return r;
}

// value of a tuning knob (an integer from the environment when the library is built with -DDK_TUNING), else `dflt`
int tuning_int(const char* name, int dflt, int lo, int hi) {
  const char* e = tuning_env(name);
  if (e == nullptr) return dflt;
  const int v = atoi(e);
  return v >= lo && v <= hi ? v : dflt;
}

constexpr int kConvWarps = 24;  // producer(s) + consumers of 80 registers (the register file is allocated per 128 threads)
constexpr int kConvMaxT = 768;

struct ConvRingPlan {
  bool ok;
  int CG, groups, R, RR, warps, np, blocks_x, rows_per_block;
  size_t smem;
};

// Channels per block, ring depths and grid of the forward / stride-1 grad-input kernel.  The consumers work on
// ceil(warps / items per row) + 1 destination rows at a time; the rings are made deep enough for those rows plus the
// producer's lookahead where shared memory allows, and the channels are split into as few groups as give at least eight
// (or all wanted) slots.
template <int S, int W, bool TR>
ConvRingPlan conv_ring_plan(const Geom& g) {
  using Sh = ConvShape<S, W, TR>;
  using RL = RotLayout<Sh::kWr>;
  ConvRingPlan pl;
  pl.ok = false;
  const size_t budget = (size_t)device_smem_optin();
  // Rows TMA cannot fetch arrive in cp.async pieces of 8 or 4 bytes (1344 of them for a row of 192 channels x 28 elements);
  // four warps share them there.  Measured on B200, C = 192, 28 x 28, batch 128, 1 / 2 / 4 producer warps of 24: forward
  // 0.056 / 0.052 / 0.050 ms, grad-input 0.056 / 0.050 / 0.049; the stride-2 grad-input kernel 0.027 / 0.024 / 0.023.
  pl.np = Sh::kTma ? 1 : tuning_int("DK_B200_RING_NP", 4, 1, 8);
  const int rows_busy = (kConvWarps - pl.np + Sh::kNB - 1) / Sh::kNB + 1;
  // source rows of the destination rows being worked on, plus one destination row of lookahead for the producer
  const int want = tuning_int("DK_B200_CONV_R", ring_slots_generous(rows_busy * S + 3), 4, 32);
  const int want_rr = TR ? want : ring_slots_generous(rows_busy + 1);
  // the fewest channel groups (the hat products of an item are shared by the block's channels) that give the wanted depth
  // or at least eight slots
  for (int groups = 1; groups <= g.C / 16 && !pl.ok; ++groups) {
    if (g.C % (16 * groups)) continue;
    const int cg = g.C / groups;
    if (cg > 256) continue;
    for (int R = want; R >= (want < 8 ? want : 8) && !pl.ok; --R) {
      // the offset rows are small: their ring gives way, down to the rows in use, before the source ring does
      const int rr_hi = TR ? R : (want_rr < R ? want_rr : R), rr_lo = TR ? R : (rows_busy + 1 < rr_hi ? rows_busy + 1 : rr_hi);
      for (int RR = rr_hi; RR >= rr_lo && !pl.ok; --RR) {
        const size_t smem = conv_ring_smem(cg, Sh::kInner, RL::kSlot, R, RR);
        if (smem > budget) continue;
        pl.ok = true;
        pl.CG = cg;
        pl.groups = groups;
        pl.R = R;
        pl.RR = RR;
        pl.smem = smem;
      }
    }
  }
  if (!pl.ok || pl.groups > 65535) {
    pl.ok = false;
    return pl;
  }
  spread_rows((long long)g.N * (TR ? g.H : g.Ho), pl.groups, &pl.blocks_x, &pl.rows_per_block);
  pl.warps = kConvWarps;
  return pl;
}

template <int S, int W, bool TR>
int launch_conv_ring(const __half* src, const __half* rot, const __half* w, __half* dst, const Geom& g, cudaStream_t s) {
  using Sh = ConvShape<S, W, TR>;
  const ConvRingPlan pl = conv_ring_plan<S, W, TR>(g);
  if (!pl.ok) return DK_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(rot) & 15) || (reinterpret_cast<uintptr_t>(src) & 15) || (reinterpret_cast<uintptr_t>(dst) & 3))
    return DK_ERR_UNSUPPORTED;
  const int Hs = TR ? g.Ho : g.H, Hd = TR ? g.H : g.Ho;
  CUtensorMap tm;
  if (Sh::kTma) {
    if (!make_row_map(&tm, src, W, Hs, (long long)g.N * g.C, Sh::kInner, pl.CG)) return DK_ERR_UNSUPPORTED;
  } else {
    memset(&tm, 0, sizeof(tm));
  }
  RingParams p;
  p.N = g.N; p.C = g.C; p.Hs = Hs; p.Hd = Hd;
  p.CG = pl.CG; p.R = pl.R; p.RR = pl.RR; p.NP = pl.np;
  if (tuning_env("DK_B200_PLAN_PRINT")) fprintf(stderr, "conv ring S=%d W=%d TR=%d C=%d: CG=%d R=%d RR=%d smem=%zu\n", S, W, (int)TR, g.C, pl.CG, pl.R, pl.RR, pl.smem);
  p.L = (Hd - 1) * S + 3;
  p.rows_total = g.N * Hd;
  p.rows_per_block = pl.rows_per_block;
  p.scH = g.scH; p.scW = g.scW; p.cells = g.cells;
  int warps = pl.warps;
  if (const char* e = tuning_env("DK_B200_RING_WARPS")) warps = atoi(e) > pl.np && atoi(e) <= kConvWarps ? atoi(e) : warps;
  auto kern = ring_conv_kernel<S, W, TR, true, kConvMaxT>;
  int rc = enable_smem(kern, pl.smem);
  if (rc) return rc;
  kern<<<dim3(pl.blocks_x, pl.groups), warps * 32, pl.smem, s>>>(tm, src, rot, w, dst, p);
  return check_launch();
}

__host__ __device__ inline size_t convT2_ring_smem(int cg, int inner, int rot_slot, int R) {
  return ((size_t)R * cg * inner + 64 + (size_t)R * rot_slot + (size_t)cg * kBankPitch) * 2 + 8 + (size_t)4 * R * 8 + 16 + 128;
}

constexpr int kConvT2Warps = 20;  // 640 threads of 96 registers

struct ConvT2RingPlan {
  bool ok;
  int CG, groups, R, warps, np, blocks_x, rows_per_block;
  size_t smem;
};

// Channels per block, ring depth (the dy ring and the offsets ring share their fill numbers) and grid of the stride-2
// grad-input kernel: as few channel groups as give the wanted depth or at least eight slots.
template <int W>
ConvT2RingPlan convT2_ring_plan(const Geom& g) {
  using Sh = ConvT2Shape<W>;
  using RL = RotLayout<Sh::kWo>;
  ConvT2RingPlan pl;
  pl.ok = false;
  const size_t budget = (size_t)device_smem_optin();
  const int want = tuning_int("DK_B200_CONVT2_R", ring_slots_generous((kConvT2Warps - 1 + Sh::kNB - 1) / Sh::kNB + 1 + 2), 4, 32);
  for (int gr = 1; gr <= g.C / 16 && !pl.ok; ++gr) {
    if (g.C % (16 * gr) || g.C / gr > 256) continue;
    for (int r = want; r >= (want < 8 ? want : 8) && !pl.ok; --r) {
      const size_t need = convT2_ring_smem(g.C / gr, Sh::kInner, RL::kSlot, r);
      if (need > budget) continue;
      pl.ok = true;
      pl.CG = g.C / gr;
      pl.groups = gr;
      pl.R = r;
      pl.smem = need;
    }
  }
  if (!pl.ok || pl.groups > 65535) {
    pl.ok = false;
    return pl;
  }
  pl.warps = kConvT2Warps;
  pl.np = Sh::kTma ? 1 : tuning_int("DK_B200_RING_NP", 4, 1, 8);  // see conv_ring_plan
  spread_rows((long long)g.N * g.Ho, pl.groups, &pl.blocks_x, &pl.rows_per_block);
  return pl;
}

template <int W>
int launch_convT2_ring(const __half* dy, const __half* rot, const __half* w, __half* dx, const Geom& g, cudaStream_t s) {
  using Sh = ConvT2Shape<W>;
  if ((reinterpret_cast<uintptr_t>(rot) & 15) || (reinterpret_cast<uintptr_t>(dx) & 7) || (reinterpret_cast<uintptr_t>(dy) & 15))
    return DK_ERR_UNSUPPORTED;
  const ConvT2RingPlan pl = convT2_ring_plan<W>(g);
  if (!pl.ok) return DK_ERR_UNSUPPORTED;
  CUtensorMap tm;
  if (Sh::kTma) {
    if (!make_row_map(&tm, dy, Sh::kWo, g.Ho, (long long)g.N * g.C, Sh::kInner, pl.CG)) return DK_ERR_UNSUPPORTED;
  } else {
    memset(&tm, 0, sizeof(tm));
  }
  RingParams p;
  p.N = g.N; p.C = g.C; p.Hs = g.Ho; p.Hd = g.H;
  p.CG = pl.CG; p.R = pl.R; p.RR = pl.R; p.NP = pl.np;
  if (tuning_env("DK_B200_PLAN_PRINT")) fprintf(stderr, "convT2 ring W=%d C=%d: CG=%d R=%d smem=%zu\n", W, g.C, pl.CG, pl.R, pl.smem);
  p.L = g.Ho + 1;
  p.rows_total = g.N * g.Ho;
  p.rows_per_block = pl.rows_per_block;
  p.scH = g.scH; p.scW = g.scW; p.cells = g.cells;
  auto kern = ring_convT2_kernel<W, true, 640>;
  int rc = enable_smem(kern, pl.smem);
  if (rc) return rc;
  kern<<<dim3(pl.blocks_x, pl.groups), pl.warps * 32, pl.smem, s>>>(tm, dy, rot, w, dx, p);
  return check_launch();
}

struct GwRingPlan {
  bool ok;
  int CG, groups, R, RR, warps, np, blocks_x, rows_per_block, ns;
  size_t smem, dw_bytes, ws_bytes;
};

// The fused offsets + bank pass keeps the bank gradient of all its channels in registers: up to 96 channels (128 registers,
// 16 warps) or, undivided, up to 144 (168 registers, 12 warps).  More channels are split into groups of up to 96 whose
// blocks write fp32 partial offset gradients [group][N][18][P], summed by a second small kernel.
template <int S, int W>
GwRingPlan gw_ring_plan(const Geom& g) {
  using Sh = GwShape<S, W>;
  using RL = RotLayout<Sh::kWo>;
  GwRingPlan pl;
  pl.ok = false;
  int groups = 1;
  if (g.C > 144) {
    groups = (g.C + 95) / 96;
    while (groups <= g.C / 16 && (g.C % (16 * groups) || g.C / groups > 96)) ++groups;
    if (groups > g.C / 16) return pl;
  }
  pl.groups = groups;
  pl.CG = g.C / groups;
  pl.ns = pl.CG <= 96 ? 6 : 9;
  // 128 or 168 registers per thread allow 16 or 12 warps.  On 28-wide planes 12 warps measured faster than 16 (0.123 against
  // 0.130 ms, C = 192), and more producer warps changed nothing here (this pass is not short of rows), so there is one.
  pl.np = tuning_int("DK_B200_GW_NP", 1, 1, 8);
  pl.warps = tuning_int("DK_B200_GW_WARPS", pl.ns == 6 ? (W == 28 ? 12 : 16) : 12, pl.np + 1, pl.ns == 6 ? 16 : 12);
  const size_t budget = (size_t)device_smem_optin();
  const int rows_busy = (pl.warps - pl.np + Sh::kNB - 1) / Sh::kNB + 1;
  // x rows of the destination rows being worked on plus one destination row of lookahead; dy / offset rows likewise.
  // Shared memory rarely holds both, so the pair that serves the largest share of both wants is taken.
  const int want = ring_slots((rows_busy + 1) * S + 2), want_rr = ring_slots(rows_busy + 1);
  long long best = -1;
  for (int R = 4; R <= want; ++R)
    for (int RR = 2; RR <= want_rr && RR <= R; ++RR) {
      const size_t smem = gw_ring_smem(pl.CG, Sh::kInnerX, Sh::kInnerD, RL::kSlot, R, RR, pl.warps - pl.np);
      if (smem > budget) continue;
      const int served = R * want_rr < RR * want ? R * want_rr : RR * want;  // min(R / want, RR / want_rr), cross-multiplied
      const long long score = (long long)served * 64 + R + RR;
      if (score <= best) continue;
      best = score;
      pl.ok = true;
      pl.R = R;
      pl.RR = RR;
      pl.smem = smem;
    }
  if (pl.ok) {
    const int R = tuning_int("DK_B200_GW_R", pl.R, 4, 32), RR = tuning_int("DK_B200_GW_RR", pl.RR, 2, 32);
    const size_t smem = gw_ring_smem(pl.CG, Sh::kInnerX, Sh::kInnerD, RL::kSlot, R, RR, pl.warps - pl.np);
    if (smem <= budget) {
      pl.R = R;
      pl.RR = RR;
      pl.smem = smem;
    }
  }
  if (!pl.ok || pl.groups > 65535) {
    pl.ok = false;
    return pl;
  }
  spread_rows((long long)g.N * g.Ho, pl.groups, &pl.blocks_x, &pl.rows_per_block);
  pl.dw_bytes = ((size_t)pl.blocks_x * g.C * 16 * sizeof(float) + 255) & ~(size_t)255;
  pl.ws_bytes = pl.dw_bytes + (pl.groups > 1 ? (size_t)pl.groups * g.N * 18 * g.P * sizeof(float) : 0);
  return pl;
}

template <int S, int W>
int launch_gw_ring(const __half* dy, const __half* x, const __half* rot, const __half* w, __half* drot, __half* dw, const Geom& g,
                   void* ws, size_t ws_bytes, cudaStream_t s) {
  using Sh = GwShape<S, W>;
  const GwRingPlan pl = gw_ring_plan<S, W>(g);
  if (!pl.ok) return DK_ERR_UNSUPPORTED;
  if (ws == nullptr || ws_bytes < pl.ws_bytes) return DK_ERR_WORKSPACE;
  if ((reinterpret_cast<uintptr_t>(rot) & 15) || (reinterpret_cast<uintptr_t>(dy) & 15) || (reinterpret_cast<uintptr_t>(x) & 15))
    return DK_ERR_UNSUPPORTED;
  CUtensorMap tmx, tmd;
  memset(&tmx, 0, sizeof(tmx));
  memset(&tmd, 0, sizeof(tmd));
  if (RowLayout<W>::kTma && !make_row_map(&tmx, x, W, g.H, (long long)g.N * g.C, Sh::kInnerX, pl.CG)) return DK_ERR_UNSUPPORTED;
  if (Sh::kDyTma && !make_row_map(&tmd, dy, Sh::kWo, g.Ho, (long long)g.N * g.C, Sh::kInnerD, pl.CG)) return DK_ERR_UNSUPPORTED;
  RingParams p;
  p.N = g.N; p.C = g.C; p.Hs = g.H; p.Hd = g.Ho;
  p.CG = pl.CG; p.R = pl.R; p.RR = pl.RR; p.NP = pl.np;
  if (tuning_env("DK_B200_PLAN_PRINT")) fprintf(stderr, "gw ring S=%d W=%d C=%d: CG=%d R=%d RR=%d warps=%d smem=%zu\n", S, W, g.C, pl.CG, pl.R, pl.RR, pl.warps, pl.smem);
  p.L = (g.Ho - 1) * S + 3;
  p.rows_total = g.N * g.Ho;
  p.rows_per_block = pl.rows_per_block;
  p.scH = g.scH; p.scW = g.scW; p.cells = g.cells;
  float* partial = reinterpret_cast<float*>(ws);
  float* gpart = pl.groups > 1 ? reinterpret_cast<float*>(reinterpret_cast<char*>(ws) + pl.dw_bytes) : nullptr;
  const dim3 grid(pl.blocks_x, pl.groups);
  int rc;
  if (pl.ns == 6) {
    auto kern = ring_gw_kernel<S, W, 6, true, 512>;
    if ((rc = enable_smem(kern, pl.smem))) return rc;
    kern<<<grid, pl.warps * 32, pl.smem, s>>>(tmx, tmd, x, dy, rot, w, drot, gpart, partial, p);
  } else {
    auto kern = ring_gw_kernel<S, W, 9, true, 384>;
    if ((rc = enable_smem(kern, pl.smem))) return rc;
    kern<<<grid, pl.warps * 32, pl.smem, s>>>(tmx, tmd, x, dy, rot, w, drot, gpart, partial, p);
  }
  if ((rc = check_launch())) return rc;
  if (pl.groups > 1 && (rc = launch_reduce_rot_partials(gpart, drot, (size_t)g.N * 18 * g.P, pl.groups, s))) return rc;
  return launch_reduce_bank_partials(partial, dw, g.C, g.cells, pl.blocks_x, s);
}

struct BwdRingPlan {
  bool ok;
  int Rx, Rd, warps, np, blocks_x, rows_per_block, ns;
  size_t smem, ws_bytes;
};

template <int S, int W>
BwdRingPlan bwd_ring_plan(const Geom& g) {
  using Sh = BwdShape<S, W>;
  using RL = RotLayout<Sh::kWo>;
  BwdRingPlan pl;
  pl.ok = false;
  pl.ns = g.C <= 96 ? 6 : 9;
  if (g.C > 144) return pl;  // the bank-gradient accumulators of all channels live in registers
  // 128 or 168 registers per thread allow 16 or 12 warps.  Where the dy rows come in cp.async pieces two producer warps share
  // them (C = 144, 56 x 56, stride 2: 0.142 ms with 2 + 10 warps, 0.146 with 1 + 10, 0.147 with 1 + 11).
  pl.np = tuning_int("DK_B200_BWD_NP", Sh::kDyTma ? 1 : 2, 1, 4);
  const int max_warps = pl.ns == 6 ? 16 : (pl.np > 1 ? 12 : 11);
  const size_t budget = (size_t)device_smem_optin();
  // Four slots is the least that lets the producer run one row ahead.  Each consumer warp owns 1.7 KB of scratch, so where
  // shared memory is short a few warps fewer are launched rather than falling back to two passes.  With the warps settled,
  // the x ring takes what is left: the source rows of the destination rows being worked on, plus the lookahead.
  const int forced_warps = tuning_int("DK_B200_BWD_WARPS", 0, 2, 12);
  for (int warps = forced_warps ? forced_warps : max_warps; warps >= (forced_warps ? forced_warps : max_warps - 8) && warps >= 2 && !pl.ok; --warps) {
    const int rows_busy = (warps - pl.np + Sh::kNB - 1) / Sh::kNB + 1;
    const int want_x = ring_slots((rows_busy + 1) * S + 2), want_d = ring_slots(rows_busy + 2);
    long long best = -1;
    for (int Rx = 4; Rx <= want_x; ++Rx)
      for (int Rd = 4; Rd <= want_d && Rd <= Rx; ++Rd) {
        const size_t smem = bwd_ring_smem(g.C, Sh::kInnerX, Sh::kInnerD, RL::kSlot, Rx, Rd, warps - pl.np);
        if (smem > budget) continue;
        const int served = Rx * want_d < Rd * want_x ? Rx * want_d : Rd * want_x;
        const long long score = (long long)served * 64 + Rx + Rd;
        if (score <= best) continue;
        best = score;
        pl.ok = true;
        pl.Rx = Rx;
        pl.Rd = Rd;
        pl.warps = warps;
        pl.smem = smem;
      }
  }
  if (pl.ok) {
    const int Rx = tuning_int("DK_B200_BWD_RX", pl.Rx, 4, 32), Rd = tuning_int("DK_B200_BWD_RD", pl.Rd, 4, 32);
    const size_t smem = bwd_ring_smem(g.C, Sh::kInnerX, Sh::kInnerD, RL::kSlot, Rx, Rd, pl.warps - pl.np);
    if (smem <= budget) {
      pl.Rx = Rx;
      pl.Rd = Rd;
      pl.smem = smem;
    }
  }
  if (!pl.ok) return pl;
  spread_rows((long long)g.N * g.Ho, 1, &pl.blocks_x, &pl.rows_per_block);
  pl.ws_bytes = (size_t)pl.blocks_x * g.C * 16 * sizeof(float);
  return pl;
}

template <int S, int W>
int launch_bwd_ring(const __half* dy, const __half* x, const __half* rot, const __half* w, __half* dx, __half* drot, __half* dw,
                    const Geom& g, void* ws, size_t ws_bytes, cudaStream_t s) {
  using Sh = BwdShape<S, W>;
  const BwdRingPlan pl = bwd_ring_plan<S, W>(g);
  if (!pl.ok) return DK_ERR_UNSUPPORTED;
  if (ws == nullptr || ws_bytes < pl.ws_bytes) return DK_ERR_WORKSPACE;
  if ((reinterpret_cast<uintptr_t>(rot) & 15) || (reinterpret_cast<uintptr_t>(dy) & 15) || (reinterpret_cast<uintptr_t>(dx) & 7))
    return DK_ERR_UNSUPPORTED;
  CUtensorMap tmx, tmd;
  if (!make_row_map(&tmx, x, W, g.H, (long long)g.N * g.C, Sh::kInnerX, g.C)) return DK_ERR_UNSUPPORTED;
  if (Sh::kDyTma) {
    if (!make_row_map(&tmd, dy, Sh::kWo, g.Ho, (long long)g.N * g.C, Sh::kInnerD, g.C)) return DK_ERR_UNSUPPORTED;
  } else {
    tmd = tmx;
  }
  RingParams p;
  p.N = g.N; p.C = g.C; p.Hs = g.Ho; p.Hd = g.H;
  p.CG = g.C; p.R = pl.Rx; p.RR = pl.Rd; p.NP = pl.np;
  if (tuning_env("DK_B200_PLAN_PRINT")) fprintf(stderr, "bwd ring S=%d W=%d C=%d: Rx=%d Rd=%d warps=%d smem=%zu\n", S, W, g.C, pl.Rx, pl.Rd, pl.warps, pl.smem);
  p.L = (g.Ho - 1) * S + 3;
  p.rows_total = g.N * g.Ho;
  p.rows_per_block = pl.rows_per_block;
  p.scH = g.scH; p.scW = g.scW; p.cells = g.cells;
  float* partial = reinterpret_cast<float*>(ws);
  int rc;
  if (pl.ns == 6) {
    auto kern = ring_bwd_kernel<S, W, 6, true, 512>;
    if ((rc = enable_smem(kern, pl.smem))) return rc;
    kern<<<pl.blocks_x, pl.warps * 32, pl.smem, s>>>(tmx, tmd, dy, rot, w, dx, drot, partial, p);
  } else {
    auto kern = ring_bwd_kernel<S, W, 9, true, 384>;
    if ((rc = enable_smem(kern, pl.smem))) return rc;
    kern<<<pl.blocks_x, pl.warps * 32, pl.smem, s>>>(tmx, tmd, dy, rot, w, dx, drot, partial, p);
  }
  if ((rc = check_launch())) return rc;
  return launch_reduce_bank_partials(partial, dw, g.C, g.cells, pl.blocks_x, s);
}

}  // namespace

// Plan of the row-ring kernel that a pass of the local deformable kernel would launch (host only).  pass: 4 forward,
// 5 grad-input, 6 grad-offsets + grad-bank, 7 the one-pass backward.  out = {slots of the source ring (x; dy for the
// stride-2 grad-input), slots of the per-row rings (offsets; dy where x is the source), warps per block, producer warps
// among them, channels per block, channel groups, dynamic shared memory in bytes, blocks in the grid}.
bool bwd_ring_shape(const Geom& g);

int local_ring_plan_query(const Geom& g, int pass, long long out[8]) {
  if (!ring_shape(g)) return DK_ERR_UNSUPPORTED;
  auto put = [&](long long r, long long rr, long long warps, long long np, long long cg, long long groups, size_t smem,
                 long long blocks) {
    const long long v[8] = {r, rr, warps, np, cg, groups, (long long)smem, blocks};
    for (int i = 0; i < 8; ++i) out[i] = v[i];
    return DK_OK;
  };
  if (pass == 4 || (pass == 5 && g.sH == 1)) {
    ConvRingPlan pl;
    pl.ok = false;
    auto plan = [&]() -> int {
      if (pass == 5) DK_RING_FOR_WIDTH(g.W, return ((pl = conv_ring_plan<1, W, true>(g)).ok))
      if (g.sH == 1) DK_RING_FOR_WIDTH(g.W, return ((pl = conv_ring_plan<1, W, false>(g)).ok))
      DK_RING_FOR_WIDE(g.W, return ((pl = conv_ring_plan<2, W, false>(g)).ok))
    };
    plan();
    if (!pl.ok) return DK_ERR_UNSUPPORTED;
    return put(pl.R, pl.RR, pl.warps, pl.np, pl.CG, pl.groups, pl.smem, (long long)pl.blocks_x * pl.groups);
  }
  if (pass == 5) {
    ConvT2RingPlan pl;
    pl.ok = false;
    auto plan = [&]() -> int { DK_RING_FOR_WIDTH(g.W, return ((pl = convT2_ring_plan<W>(g)).ok)) };
    plan();
    if (!pl.ok) return DK_ERR_UNSUPPORTED;
    return put(pl.R, pl.R, pl.warps, pl.np, pl.CG, pl.groups, pl.smem, (long long)pl.blocks_x * pl.groups);
  }
  if (pass == 6) {
    GwRingPlan pl;
    pl.ok = false;
    auto plan = [&]() -> int {
      if (g.sH == 1) DK_RING_FOR_WIDTH(g.W, return ((pl = gw_ring_plan<1, W>(g)).ok))
      DK_RING_FOR_WIDE(g.W, return ((pl = gw_ring_plan<2, W>(g)).ok))
    };
    plan();
    if (!pl.ok) return DK_ERR_UNSUPPORTED;
    return put(pl.R, pl.RR, pl.warps, pl.np, pl.CG, pl.groups, pl.smem, (long long)pl.blocks_x * pl.groups);
  }
  if (pass == 7) {
    if (!bwd_ring_shape(g)) return DK_ERR_UNSUPPORTED;
    BwdRingPlan pl;
    if (g.W == 112) pl = g.sH == 1 ? bwd_ring_plan<1, 112>(g) : bwd_ring_plan<2, 112>(g);
    else pl = g.sH == 1 ? bwd_ring_plan<1, 56>(g) : bwd_ring_plan<2, 56>(g);
    if (!pl.ok) return DK_ERR_UNSUPPORTED;
    return put(pl.Rx, pl.Rd, pl.warps, pl.np, g.C, 1, pl.smem, pl.blocks_x);
  }
  return DK_ERR_BAD_ARGUMENT;
}

// Code of the last bounded wait that ran out in a ring kernel on the current device (0 = none);
// synchronises with the device.  For tests and diagnosis.
int ring_error_status() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_ring_error, sizeof(int)) != cudaSuccess) return -1;
  return v;
}

// forward (transposed = false) or grad-input (transposed = true); DK_ERR_UNSUPPORTED = not a ring shape
int local_conv_ring(const __half* src, const __half* rot, const __half* w, __half* dst, const Geom& g, bool transposed,
                    cudaStream_t s) {
  if (!ring_shape(g)) return DK_ERR_UNSUPPORTED;
  if (!transposed) {
    if (g.sH == 1) DK_RING_FOR_WIDTH(g.W, return (launch_conv_ring<1, W, false>(src, rot, w, dst, g, s)))
    DK_RING_FOR_WIDE(g.W, return (launch_conv_ring<2, W, false>(src, rot, w, dst, g, s)))
  }
  if (g.sH == 1) DK_RING_FOR_WIDTH(g.W, return (launch_conv_ring<1, W, true>(src, rot, w, dst, g, s)))
  DK_RING_FOR_WIDTH(g.W, return (launch_convT2_ring<W>(src, rot, w, dst, g, s)))
}

// Workspace of local_gw_ring (per-block partial bank gradients, and partial offset gradients when the channels are split
// into groups); 0 = the shape is not covered.
size_t local_gw_ring_workspace(const Geom& g) {
  if (!ring_shape(g)) return 0;
  GwRingPlan pl;
  pl.ok = false;
  auto plan = [&]() -> int {
    if (g.sH == 1) DK_RING_FOR_WIDTH(g.W, return ((pl = gw_ring_plan<1, W>(g)).ok))
    DK_RING_FOR_WIDE(g.W, return ((pl = gw_ring_plan<2, W>(g)).ok))
  };
  plan();
  return pl.ok ? pl.ws_bytes : 0;
}

// Measured on B200 (batch 128, ms, one pass against grad-input + offsets / bank pass): C=96 112x112 stride 1 1.03 / 0.84,
// stride 2 0.29 / 0.26; C=144 56x56 stride 1 0.36 / 0.33, stride 2 0.172 / 0.184.  One pass moves every tensor once, but
// its grad-input half runs at the register count and warp count the offsets / bank half needs (12-15 warps of 128-168
// registers instead of 20 of 80), and on the 112-wide layers shared memory allows only 12 warps.  So it is the default
// only on the narrow stride-2 shape where it won; dk_sample_depthwise_backward_one_pass asks for it explicitly.
bool local_bwd_ring_preferred(const Geom& g) {
  if (tuning_env("DK_B200_NO_ONE_PASS")) return false;
  return ring_shape(g) && g.W == 56 && g.sH == 2 && g.C <= 144;
}

bool bwd_ring_shape(const Geom& g) { return ring_shape(g) && (g.W == 112 || g.W == 56); }

// Workspace of local_bwd_ring (the per-block partial bank gradients); 0 = the shape is not covered.
size_t local_bwd_ring_workspace(const Geom& g) {
  if (!bwd_ring_shape(g)) return 0;
  BwdRingPlan pl;
  if (g.W == 112) pl = g.sH == 1 ? bwd_ring_plan<1, 112>(g) : bwd_ring_plan<2, 112>(g);
  else pl = g.sH == 1 ? bwd_ring_plan<1, 56>(g) : bwd_ring_plan<2, 56>(g);
  return pl.ok ? pl.ws_bytes : 0;
}

// all three gradients in one pass over dy, x and the offsets
int local_bwd_ring(const __half* dy, const __half* x, const __half* rot, const __half* w, __half* dx, __half* drot, __half* dw,
                   const Geom& g, void* ws, size_t ws_bytes, cudaStream_t s) {
  if (!bwd_ring_shape(g) || dx == nullptr || drot == nullptr || dw == nullptr) return DK_ERR_UNSUPPORTED;
  if (g.W == 112)
    return g.sH == 1 ? launch_bwd_ring<1, 112>(dy, x, rot, w, dx, drot, dw, g, ws, ws_bytes, s)
                     : launch_bwd_ring<2, 112>(dy, x, rot, w, dx, drot, dw, g, ws, ws_bytes, s);
  return g.sH == 1 ? launch_bwd_ring<1, 56>(dy, x, rot, w, dx, drot, dw, g, ws, ws_bytes, s)
                   : launch_bwd_ring<2, 56>(dy, x, rot, w, dx, drot, dw, g, ws, ws_bytes, s);
}

// grad-offsets and grad-bank in one pass
int local_gw_ring(const __half* dy, const __half* x, const __half* rot, const __half* w, __half* drot, __half* dw, const Geom& g,
                  void* ws, size_t ws_bytes, cudaStream_t s) {
  if (!ring_shape(g) || drot == nullptr || dw == nullptr) return DK_ERR_UNSUPPORTED;
  if (g.sH == 1) DK_RING_FOR_WIDTH(g.W, return (launch_gw_ring<1, W>(dy, x, rot, w, drot, dw, g, ws, ws_bytes, s)))
  DK_RING_FOR_WIDE(g.W, return (launch_gw_ring<2, W>(dy, x, rot, w, drot, dw, g, ws, ws_bytes, s)))
}

}  // namespace dk
