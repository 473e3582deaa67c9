// Building blocks of the fp16 tensor-core kernels (dk_local_mma.cu).
//
// Conventions.  lane = 4*gq + q (gq = lane >> 2 in 0..7, q = lane & 3).  An "item" is a block
// of 8 horizontally adjacent destination pixels ow0 .. ow0+7 of one row; in accumulator
// fragments a thread owns the pixel pair (ow0 + 2q, ow0 + 2q + 1), in B fragments of the
// kernel GEMM it supplies pixel ow0 + gq.  A "band" is the set of source rows a block of
// destination rows needs, kept in shared memory as fp16 in the global row layout.
#pragma once

#include "dk_common.cuh"

namespace dk {
namespace mma {

constexpr int kSlack = 8;       // zeroed halves in front of each channel's band
constexpr int kBankPitch = 24;  // halves per channel row of the bank copy (12 words: conflict-free A loads)
constexpr int kBetaWords = 3 * 8 * 8;  // per-warp table for three taps: [tap][pixel][8 words of two cells], swizzled

// d = a * b (+ c): m16n8k16, fp16 inputs, fp32 accumulate.
__device__ __forceinline__ void mma16816(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
}
__device__ __forceinline__ void mma16816_acc(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                             unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// d = a * b with fp16 output: d[0] = row gq, columns (2q, 2q+1); d[1] = row gq + 8.
__device__ __forceinline__ void mma16816_h(unsigned (&d)[2], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f16.f16.f16.f16 {%0,%1}, {%2,%3,%4,%5}, {%6,%7}, {%8,%8};\n"
      : "=r"(d[0]), "=r"(d[1])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(0u));
}
// acc += half HA of a * half HB of b, product and sum in fp32 (sm_100 mixed-precision FMA)
template <int HA, int HB>
__device__ __forceinline__ void fma_hh(float& acc, unsigned a, unsigned b) {
  if (HA == 0 && HB == 0)
    asm("{\n .reg .b16 al, ah, bl, bh;\n mov.b32 {al, ah}, %1;\n mov.b32 {bl, bh}, %2;\n fma.rn.f32.f16 %0, al, bl, %0;\n}\n"
        : "+f"(acc) : "r"(a), "r"(b));
  else if (HA == 0 && HB == 1)
    asm("{\n .reg .b16 al, ah, bl, bh;\n mov.b32 {al, ah}, %1;\n mov.b32 {bl, bh}, %2;\n fma.rn.f32.f16 %0, al, bh, %0;\n}\n"
        : "+f"(acc) : "r"(a), "r"(b));
  else if (HA == 1 && HB == 0)
    asm("{\n .reg .b16 al, ah, bl, bh;\n mov.b32 {al, ah}, %1;\n mov.b32 {bl, bh}, %2;\n fma.rn.f32.f16 %0, ah, bl, %0;\n}\n"
        : "+f"(acc) : "r"(a), "r"(b));
  else
    asm("{\n .reg .b16 al, ah, bl, bh;\n mov.b32 {al, ah}, %1;\n mov.b32 {bl, bh}, %2;\n fma.rn.f32.f16 %0, ah, bh, %0;\n}\n"
        : "+f"(acc) : "r"(a), "r"(b));
}
// acc += (half IDX of the 6-half window held in w0, w1, w2) * (half KH of k)
template <int IDX, int KH>
__device__ __forceinline__ void fma_win(float& acc, unsigned w0, unsigned w1, unsigned w2, unsigned k) {
  fma_hh<(IDX & 1), KH>(acc, IDX < 2 ? w0 : (IDX < 4 ? w1 : w2), k);
}

// transpose of an 8x8 block of 16-bit values held one row per 4 lanes (standard fragment layout)
__device__ __forceinline__ unsigned movmatrix_trans(unsigned a) {
  unsigned d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(d) : "r"(a));
  return d;
}

__device__ __forceinline__ float lo2f(unsigned w) { return __low2float(*reinterpret_cast<const __half2*>(&w)); }
__device__ __forceinline__ float hi2f(unsigned w) { return __high2float(*reinterpret_cast<const __half2*>(&w)); }
__device__ __forceinline__ unsigned hmul2u(unsigned a, unsigned b) {
  __half2 r = __hmul2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
  return *reinterpret_cast<unsigned*>(&r);
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  const unsigned sa = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(sa), "l"(gmem));
}
__device__ __forceinline__ void cp_async4(void* smem, const void* gmem) {
  const unsigned sa = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(sa), "l"(gmem));
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;\n" ::: "memory"); }
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
// wait until at most N of this thread's committed groups are still in flight
template <int N>
__device__ __forceinline__ void cp_async_wait_group() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

// The pair (source value of pixel 0, source value of pixel 1) for tap column fw, cut out of the
// 6-half window [ow*S-2, ow*S+3] held in three words: halves 1+fw and 1+S+fw.
template <int S>
__device__ __forceinline__ unsigned tap_pair(unsigned w0, unsigned w1, unsigned w2, int fw) {
  if (S == 1) {
    if (fw == 0) return __byte_perm(w0, w1, 0x5432);  // (w0.hi, w1.lo)
    if (fw == 1) return w1;
    return __byte_perm(w1, w2, 0x5432);               // (w1.hi, w2.lo)
  } else {
    if (fw == 0) return __byte_perm(w0, w1, 0x7632);  // (w0.hi, w1.hi)
    if (fw == 1) return __byte_perm(w1, w2, 0x5410);  // (w1.lo, w2.lo)
    return __byte_perm(w1, w2, 0x7632);               // (w1.hi, w2.hi)
  }
}

// ---------------------------------------------------------------- band loader
struct Band {
  int row_lo;   // first source row held
  int RB;       // rows held
  int Wp;       // row pitch in shared memory (halves, even)
  int pitch_c;  // channel pitch (halves), = 8 (mod 16): conflict-free across the 8 channels of a fragment
  int mode;     // 2 = 16-byte vectors, 1 = 4-byte pairs, 0 = scalars
  int org;      // element (row, col) of local channel j sits at j*pitch_c + kSlack + row*Wp + col - org
};

__host__ __device__ inline int band_pitch(int RB, int Wp) {
  const int need = RB * Wp + kSlack + 16;
  int pitch = ((need + 7) & ~15) + 8;
  if (pitch < need) pitch += 16;
  return pitch;
}
__host__ __device__ inline int band_mode(int plane, int Ws) {
  return ((plane & 7) == 0 && (Ws & 1) == 0) ? 2 : ((Ws & 1) == 0 ? 1 : 0);
}
// maxmode caps the copy width by the alignment of the tensor's base pointer (see ptr_mode).
__device__ __forceinline__ Band make_band(int row_lo, int RB, int Hs, int Ws, int maxmode) {
  Band b;
  b.row_lo = row_lo;
  b.RB = RB;
  b.Wp = Ws + (Ws & 1);
  b.pitch_c = band_pitch(RB, b.Wp);
  b.mode = min(band_mode(Hs * Ws, Ws), maxmode);
  b.org = (b.mode == 2) ? ((row_lo * Ws) & ~7) : row_lo * b.Wp;
  return b;
}

inline int ptr_mode(const void* p) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(p);
  return (a & 15) == 0 ? 2 : ((a & 3) == 0 ? 1 : 0);
}

// Copy the in-range source rows [row_lo, row_lo+RB) of channels c0 .. c0+cnt-1 of sample n into
// the band with cp.async (16- or 4-byte pieces) and zero everything else of the band (slack,
// rows outside the image).  Called by the whole block; the caller must execute
// cp_async_wait_all() and __syncthreads() before reading.  Odd row widths fall back to plain
// 2-byte copies behind an extra barrier.
// load_band_group: the same for a group of nt threads (whole warps) numbered tid = 0 .. nt-1 that synchronises on
// named barrier bar_id (bar_id 0: the whole block, __syncthreads).
__device__ __forceinline__ void group_sync(int bar_id, int nt) {
  if (bar_id == 0) __syncthreads();
  else asm volatile("bar.sync %0, %1;\n" ::"r"(bar_id), "r"(nt) : "memory");
}
__device__ __forceinline__ void load_band_group(__half* __restrict__ band, const Band& b, const __half* __restrict__ src, int n,
                                                int C, int c0, int cnt, int Hs, int Ws, int tid, int nt, int bar_id) {
  const int lane = tid & 31, warp = tid >> 5, nwarps = nt >> 5;
  const int r_s = max(b.row_lo, 0), r_e = min(b.row_lo + b.RB, Hs);
  const size_t plane = (size_t)Hs * Ws;
  const __half* s0 = src + ((size_t)n * C + c0) * plane;
  if (b.mode == 0 || r_e <= r_s) {
    const uint4 z = make_uint4(0, 0, 0, 0);
    uint4* b4 = reinterpret_cast<uint4*>(band);
    const int nv = cnt * b.pitch_c / 8;
    for (int i = tid; i < nv; i += nt) b4[i] = z;
    if (r_e <= r_s) return;
    group_sync(bar_id, nt);
    // 2-byte copies: a thread takes one (channel, row) and walks along it, eight independent loads in flight
    const int rows = r_e - r_s;
    const int tasks = cnt * rows;
    for (int t = tid; t < tasks; t += nt) {
      const int j = t / rows, r = r_s + (t - j * rows);
      const __half* sp = s0 + (size_t)j * plane + (size_t)r * Ws;
      __half* dp = band + (size_t)j * b.pitch_c + kSlack + (r * b.Wp - b.org);
      for (int c0w = 0; c0w < Ws; c0w += 8) {
        __half val[8];
#pragma unroll
        for (int k = 0; k < 8; ++k)
          if (c0w + k < Ws) val[k] = __ldg(sp + c0w + k);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          if (c0w + k < Ws) dp[c0w + k] = val[k];
      }
    }
    return;
  }
  // contiguous span [lo, hi) of each channel band that receives data (in halves, relative to the channel)
  int gs, lo, hi;
  if (b.mode == 2) {
    gs = (r_s * Ws) & ~7;
    const int ge = min((r_e * Ws + 7) & ~7, (int)plane);
    lo = kSlack + (gs - b.org);
    hi = lo + (ge - gs);
  } else {
    gs = r_s * Ws;
    lo = kSlack + (r_s * b.Wp - b.org);
    hi = lo + (r_e - r_s) * Ws;
  }
  const int head = lo >> 1, tail = (b.pitch_c - hi) >> 1;  // 4-byte words to zero in front / behind
  const int esz = b.mode == 2 ? 8 : 2;                       // halves per copy
  const int npiece = (hi - lo) / esz;
  __half* ch = band + (size_t)warp * b.pitch_c;
  const __half* sp = s0 + (size_t)warp * plane + gs;
  const size_t sstep = (size_t)nwarps * plane;
  const int dstep = nwarps * b.pitch_c;
  for (int j = warp; j < cnt; j += nwarps, ch += dstep, sp += sstep) {
    if (b.mode == 2) {
      for (int v = lane; v < npiece; v += 32) cp_async16(ch + lo + v * 8, sp + v * 8);
    } else {
      for (int v = lane; v < npiece; v += 32) cp_async4(ch + lo + v * 2, sp + v * 2);
    }
    unsigned* zw = reinterpret_cast<unsigned*>(ch);
    if (lane < head) zw[lane] = 0u;
    for (int v = lane + 32; v < head; v += 32) zw[v] = 0u;
    unsigned* zt = reinterpret_cast<unsigned*>(ch + hi);
    if (lane < tail) zt[lane] = 0u;
    for (int v = lane + 32; v < tail; v += 32) zt[v] = 0u;
  }
}
// Copies of ESZ halves each (8: cp.async 16 bytes, 2: 4 bytes) for the span [lo, hi) of cnt channel bands: thread tid of nt takes
// the (channel, piece) pairs tid, tid + nt, ... in channel-major order and steps both pointers incrementally.
template <int ESZ>
__device__ __forceinline__ void flat_copies(__half* __restrict__ band, int pitch_c, int lo, int hi, const __half* __restrict__ s0,
                                            size_t plane, int cnt, int tid, int nt) {
  const int npiece = (hi - lo) / ESZ;
  const int dc = nt / npiece, dv = nt - dc * npiece;
  int c = tid / npiece, v = tid - c * npiece;
  const __half* sp = s0 + (size_t)c * plane + v * ESZ;
  __half* dp = band + (size_t)c * pitch_c + lo + v * ESZ;
  const size_t s_step = (size_t)dc * plane + dv * ESZ, s_wrap = plane - (size_t)npiece * ESZ;
  const int d_step = dc * pitch_c + dv * ESZ, d_wrap = pitch_c - npiece * ESZ;
  while (c < cnt) {
    if (ESZ == 8) cp_async16(dp, sp);
    else cp_async4(dp, sp);
    c += dc; v += dv; sp += s_step; dp += d_step;
    if (v >= npiece) { v -= npiece; ++c; sp += s_wrap; dp += d_wrap; }
  }
}
// The same copy (16- or 4-byte pieces) with the (channel, piece) pairs spread evenly over the nt threads and advanced
// incrementally: every lane busy and every channel's copies in flight at once, where the one-warp-per-channel loops above
// leave lanes idle on the last pass over a row and walk through the channels one after the other.  Same instruction count
// (measured), 3-4 % less time in the four kernels.
// Odd row widths, and bands without a row inside the image, go through load_band_group.
__device__ __forceinline__ void load_band_flat(__half* __restrict__ band, const Band& b, const __half* __restrict__ src, int n,
                                               int C, int c0, int cnt, int Hs, int Ws, int tid, int nt, int bar_id) {
  const int r_s = max(b.row_lo, 0), r_e = min(b.row_lo + b.RB, Hs);
  if (b.mode == 0 || r_e <= r_s) {
    load_band_group(band, b, src, n, C, c0, cnt, Hs, Ws, tid, nt, bar_id);
    return;
  }
  const size_t plane = (size_t)Hs * Ws;
  // contiguous span [lo, hi) of each channel band that receives data, as in load_band_group
  int gs, lo, hi;
  if (b.mode == 2) {
    gs = (r_s * Ws) & ~7;
    const int ge = min((r_e * Ws + 7) & ~7, (int)plane);
    lo = kSlack + (gs - b.org);
    hi = lo + (ge - gs);
  } else {
    gs = r_s * Ws;
    lo = kSlack + (r_s * b.Wp - b.org);
    hi = lo + (r_e - r_s) * Ws;
  }
  if (b.mode == 2) flat_copies<8>(band, b.pitch_c, lo, hi, src + ((size_t)n * C + c0) * plane + gs, plane, cnt, tid, nt);
  else flat_copies<2>(band, b.pitch_c, lo, hi, src + ((size_t)n * C + c0) * plane + gs, plane, cnt, tid, nt);
  // zero what the copies leave out: the words in front of lo and behind hi of every channel
  const int head = lo >> 1, tail = (b.pitch_c - hi) >> 1, nz = head + tail;
  if (nz > 0) {
    const int dc = nt / nz, dv = nt - dc * nz;
    int c = tid / nz, v = tid - c * nz;
    while (c < cnt) {
      unsigned* ch = reinterpret_cast<unsigned*>(band + (size_t)c * b.pitch_c);
      ch[v < head ? v : (hi >> 1) + (v - head)] = 0u;
      c += dc; v += dv;
      if (v >= nz) { v -= nz; ++c; }
    }
  }
}
__device__ __forceinline__ void load_band(__half* __restrict__ band, const Band& b, const __half* __restrict__ src, int n, int C,
                                          int c0, int cnt, int Hs, int Ws) {
  load_band_flat(band, b, src, n, C, c0, cnt, Hs, Ws, threadIdx.x, blockDim.x, 0);
}

// Offset (in halves, even) of the window of pixel pair (ow, ow+1), row selector 0, inside a channel band.
__device__ __forceinline__ int window_offset(const Band& b, int srow0, int ow, int S) {
  return kSlack + srow0 * b.Wp + (ow * S - 2) - b.org;
}

// ---------------------------------------------------------------- hat-product (beta) fragments
// For the 8 pixels of an item and the 9 taps: beta[(pixel, tap)][cell] = hat(u - a) * hat(v - b),
// i.e. the four bilinear coefficients scattered into a row of 16 cells, zero when the tap is
// unused (outside the image / the bank).  Built cooperatively by the warp, three taps at a
// time -- one lane per (pixel, tap) -- into a swizzled table, then read back as mma B fragments:
//   bf[t][0] = cells (2q, 2q+1) of pixel gq, bf[t][1] = cells (2q+8, 2q+9) of pixel gq.
// The kernel-space offsets come from a band of the 18 offset planes in shared memory (rb, rband).
// With KEEP_UV the bank coordinates are left in uv[tap*8 + pixel] (u = 1e30 marks an unused tap).
template <int S, bool TRANSPOSED, bool KEEP_UV>
__device__ __forceinline__ void build_beta(unsigned (&bf)[9][2], unsigned* __restrict__ T, float2* __restrict__ uv,
                                           const __half* __restrict__ rband, const Band& rb, const Geom& g, int drow, int ow0,
                                           int Hs, int Ws, int Wd, int lane) {
  const float uh0 = (float)(g.scH - 3) * 0.5f, uw0 = (float)(g.scW - 3) * 0.5f;
  __half* Th = reinterpret_cast<__half*>(T);
  const int gq = lane >> 2, q = lane & 3;
  const int px = lane & 7, tt = lane >> 3;  // builder role (lanes 0..23)
  const int pc = ow0 + px;
#pragma unroll
  for (int pass = 0; pass < 3; ++pass) {
    {
      const uint4 z = make_uint4(0, 0, 0, 0);
      uint4* t4 = reinterpret_cast<uint4*>(T);
      t4[lane] = z;
      if (lane < kBetaWords / 4 - 32) t4[32 + lane] = z;
    }
    __syncwarp();
    if (lane < 24) {
      const int fh = pass, fw = tt;
      const int t = pass * 3 + tt;
      int orow, ocol;
      bool ok;
      if (!TRANSPOSED) {
        const int sr = drow * S - 1 + fh, sc = pc * S - 1 + fw;
        ok = pc < Wd && sr >= 0 && sr < Hs && sc >= 0 && sc < Ws;
        orow = drow;
        ocol = pc;
      } else {
        // the output pixel that reaches destination (drow, pc) through tap (fh, fw), if any
        const int tr = drow + 1 - fh, tc = pc + 1 - fw;
        orow = tr / S;
        ocol = tc / S;
        ok = pc < Wd && tr >= 0 && tc >= 0 && orow * S == tr && ocol * S == tc && orow < Hs && ocol < Ws;
      }
      const int off = ok ? kSlack + orow * rb.Wp + ocol - rb.org : kSlack;
      const __half* rp = rband + (size_t)(2 * t) * rb.pitch_c + off;
      const float u = ((float)fh + __half2float(rp[0])) + uh0;
      const float v = ((float)fw + __half2float(rp[rb.pitch_c])) + uw0;
      const bool valid = ok && u > -1.f && v > -1.f && u < (float)g.scH && v < (float)g.scW;
      if (KEEP_UV) uv[t * 8 + px] = make_float2(valid ? u : 1e30f, v);
      if (valid) {
        const float fu = floorf(u), fv = floorf(v);
        const int h0 = (int)fu, w0 = (int)fv;
        const float lh = u - fu, lw = v - fv;
        const int sw = (px >> 2) << 2;
        __half* row = Th + (tt * 8 + px) * 16;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int a = h0 + (k >> 1), b = w0 + (k & 1);
          if (a >= 0 && a < g.scH && b >= 0 && b < g.scW) {
            const int cell = a * g.scW + b;
            const float coef = ((k >> 1) ? lh : 1.f - lh) * ((k & 1) ? lw : 1.f - lw);
            row[(((cell >> 1) ^ sw) << 1) + (cell & 1)] = __float2half_rn(coef);
          }
        }
      }
    }
    __syncwarp();
    {
      const int sw = (gq >> 2) << 2;
#pragma unroll
      for (int k = 0; k < 3; ++k) {
        bf[pass * 3 + k][0] = T[(k * 8 + gq) * 8 + (q ^ sw)];
        bf[pass * 3 + k][1] = T[(k * 8 + gq) * 8 + ((q + 4) ^ sw)];
      }
    }
    __syncwarp();
  }
}

// ---------------------------------------------------------------- beta fragments, computed per lane
// Same fragments as build_beta, without the table: lane (gq, q) evaluates the hat products of
// pixel ow0 + gq at its own four cells (2q, 2q+1, 2q+8, 2q+9) for each tap.  ca/cb are the (row,
// column) of those cells as floats, cellok marks cells that exist (scope smaller than 16 cells);
// SC44 = 4x4 scope, where the four cells share two rows and two columns.
struct LaneCells {
  float ca[4], cb[4];
  bool ok[4];
};
__device__ __forceinline__ LaneCells lane_cells(const Geom& g, int q) {
  LaneCells lc;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int cell = 2 * q + (k & 1) + (k >> 1) * 8;
    lc.ok[k] = cell < g.cells;
    const int a = cell / g.scW;
    lc.ca[k] = (float)a;
    lc.cb[k] = (float)(cell - a * g.scW);
  }
  return lc;
}
__device__ __forceinline__ float hat(float t) { return __saturatef(1.f - fabsf(t)); }  // max(0, 1 - |t|) in one add
__device__ __forceinline__ unsigned pack2(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const unsigned*>(&h);
}

// IMAGE_MASK = false keeps the taps whose integer source position lies in the padding (the DK + DCN
// operator decides validity on the deformed position instead).
template <int S, bool TRANSPOSED, bool IMAGE_MASK = true>
__device__ __forceinline__ void beta_direct(unsigned (&bf)[9][2], const __half* __restrict__ rband, const Band& rb,
                                            const Geom& g, const LaneCells& lc, bool sc44, int drow, int ow0, int Hs, int Ws,
                                            int Wd, int gq) {
  const int pc = ow0 + gq;
  int roff[3], coff[3];
  bool rok[3], cok[3];
#pragma unroll
  for (int f = 0; f < 3; ++f) {
    if (!TRANSPOSED) {
      const int sr = drow * S - 1 + f, sc = pc * S - 1 + f;
      rok[f] = !IMAGE_MASK || (sr >= 0 && sr < Hs);
      cok[f] = pc < Wd && (!IMAGE_MASK || (sc >= 0 && sc < Ws));
      roff[f] = drow * rb.Wp;
      coff[f] = pc;
    } else {
      const int tr = drow + 1 - f, tc = pc + 1 - f;
      const int orow = S == 1 ? tr : tr >> 1, ocol = S == 1 ? tc : tc >> 1;
      rok[f] = tr >= 0 && (S == 1 || !(tr & 1)) && orow < Hs;
      cok[f] = pc < Wd && tc >= 0 && (S == 1 || !(tc & 1)) && ocol < Ws;
      roff[f] = rok[f] ? orow * rb.Wp : 0;
      coff[f] = cok[f] ? ocol : 0;
    }
  }
  const float uh0 = (float)(g.scH - 3) * 0.5f, uw0 = (float)(g.scW - 3) * 0.5f;
  const __half* base = rband + kSlack - rb.org;
  const int p2 = 2 * rb.pitch_c;
#pragma unroll
  for (int fh = 0; fh < 3; ++fh) {
#pragma unroll
    for (int fw = 0; fw < 3; ++fw) {
      const int t = fh * 3 + fw;
      const bool ok = rok[fh] && cok[fw];
      const __half* rp = base + t * p2 + roff[fh] + coff[fw];
      const float u = ((float)fh + __half2float(rp[0])) + uh0;
      const float v = ok ? ((float)fw + __half2float(rp[rb.pitch_c])) + uw0 : 1e30f;  // unused tap: every hat is 0
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

// Bank coordinates (u, v) of the 72 (pixel, tap) pairs of an item, left in uv[tap*8 + pixel]
// (u = 1e30 marks a tap that is unused: in the padding or outside the bank).  Lanes 0..23, three passes.
template <int S, bool IMAGE_MASK = true>
__device__ __forceinline__ void item_uv(float2* __restrict__ uv, const __half* __restrict__ rband, const Band& rb, const Geom& g,
                                        int drow, int ow0, int lane) {
  const float uh0 = (float)(g.scH - 3) * 0.5f, uw0 = (float)(g.scW - 3) * 0.5f;
  const int px = lane & 7, fw = lane >> 3;
  const int pc = ow0 + px;
  const int sc = pc * S - 1 + fw;
  const bool cok = pc < g.Wo && (!IMAGE_MASK || (sc >= 0 && sc < g.W));
  const __half* base = rband + kSlack - rb.org + drow * rb.Wp + pc;
  if (lane < 24) {
#pragma unroll
    for (int fh = 0; fh < 3; ++fh) {
      const int t = fh * 3 + fw;
      const int sr = drow * S - 1 + fh;
      const __half* rp = base + (size_t)(2 * t) * rb.pitch_c;
      const float u = ((float)fh + __half2float(rp[0])) + uh0;
      const float v = ((float)fw + __half2float(rp[rb.pitch_c])) + uw0;
      const bool valid = cok && (!IMAGE_MASK || (sr >= 0 && sr < g.H)) && u > -1.f && v > -1.f && u < (float)g.scH && v < (float)g.scW;
      uv[t * 8 + px] = make_float2(valid ? u : 1e30f, v);
    }
  }
}

}  // namespace mma
}  // namespace dk
