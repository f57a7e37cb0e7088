// Sparse convolution with fp32-class accuracy on the warp-level tensor path, accumulators in
// registers: the kernel for narrow layers (32 or 64 output planes) with many rows.
//
// Same mathematics and the same dense rulebook as the other convolution kernels (the reference's
// per-offset gather / GEMM / scatter-add is CPU/Convolution.cpp:137-148 and
// CUDA/Convolution.cu:57-233,618-642).  The work is laid out by OUTPUT ROW, not by rule:
//
//   warp      32 consecutive output rows as two 16-row tiles of mma.sync, their 32 x Cout
//             accumulators in registers for the whole filter.  For every filter offset the warp
//             gathers the input rows of its rows (16-byte cp.async into a private ring of stages,
//             zero fill where the rulebook has no rule) and multiplies them with the offset's
//             weights.  A 16-row tile without a rule for the offset is skipped: rows come sorted by
//             coordinate, so the rules of an offset cluster (54 % of the (offset, 16-row tile) slots
//             of an indoor scan hold a rule, at 62 % fill)
//   weights   prepared (per call, or once per layer under a weight token) as the per-lane fragment
//             image of (offset, 32-plane chunk) slabs: bf16 h / m pairs, 4 or 8 KB per slab (the
//             tf32 form: tf32 and bf16 parts, twice that); every warp reads its B fragments
//             straight from that image with 128-bit loads; they come from L2 (the slabs of the 20
//             warps of an SM do not fit L1 beside the shared memory, hit rate 9 %; an L1 prefetch a
//             step ahead made it slower), and the other warps cover the latency
//   nothing   is shared between warps: no barrier, no shared-memory accumulator, no pair lists.
//             A CTA is one warp; 12 to 21 of them are resident per SM
//   arithmetic the fp32-class mode in its default form: x = h + m with h = bf16(x), m = bf16(x - h);
//             D += A_m B_h + A_h B_m + A_h B_h as three bf16 m16n8k16 per 16 planes, fp32
//             accumulators (TC_BF16X3; 2e-6 to 6e-6 of max against the reference's CPU operator).
//             The other form (SCN_X3_FORM=tf32): x = hi + lo with hi = x truncated to tf32, the
//             large term as two tf32 m16n8k8, the two small ones as one bf16 m16n8k16 each: four
//             instructions per 16 planes and twice the weight image; 25 to 30 % slower
//   store     bias, then optionally the scale / shift / leaky ReLU of the eval-mode BatchNorm that
//             follows the layer, then each row once
//   also here k_conv_rows_thin (first layers, at most four input planes) and k_conv_rows_scatter
//             (Deconvolution with filter = stride, run from its input side)
//
// Against the compacting kernel of conv_pipe.cu this issues 1.4 to 1.6 times the tensor
// instructions (the zero rows inside a tile) but half the instructions around each of them.
#include <stdlib.h>

#include "metadata.cuh"
#include "tc_ptx.cuh"

namespace scn {

// optional per-plane scale / shift / leaky ReLU applied to a finished output value: the eval-mode
// BatchNorm (+ activation) that follows the convolution, with the same rounding as the stand-alone
// kernel (separate multiply and add)
__device__ __forceinline__ float rows_epilogue(float v, float sc, float sh, float leak) {
  const float y = __fadd_rn(__fmul_rn(v, sc), sh);
  return y * (y > 0.f ? 1.f : leak);
}

constexpr int kRChunk = 32;                    // input planes per step
constexpr int kRAStride = kRChunk + 4;         // floats; rows g and g + 1 land on different bank quads
constexpr int kRAStages = 2;                   // per-warp ring of gathered rows (three: slower, fewer warps fit)
constexpr int kRMaxK = 32;
constexpr int kRStageFloats = 32 * kRAStride;  // one stage: [row][plane]

__device__ __forceinline__ void rows_mma(float (&d)[4], const unsigned (&a)[4], const unsigned (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ void rows_split(float x, unsigned &hi, unsigned &lo) {
  hi = __float_as_uint(x) & 0xFFFFE000u;
  lo = __float_as_uint(x - __uint_as_float(hi));
}

__device__ __forceinline__ void rows_mma_bf16(float (&d)[4], const unsigned (&a)[4], const unsigned (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
// two values as a bf16 pair, `first` in the low half (the lower k index of the fragment register)
__device__ __forceinline__ unsigned rows_pack_bf16(float first, float second) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(first, second);
  return *reinterpret_cast<const unsigned *>(&v);
}

// The product of 16 input planes is four tensor instructions: the large term hi x hi as two tf32
// m16n8k8, the two small terms lo x W and x x W_lo as one bf16 m16n8k16 each (a bf16 instruction
// takes the issue slot of a tf32 one and covers twice the planes; the small terms are 2^-11 of
// the result, so bf16's 2^-9 leaves 2^-20).  Lane (g, t) feeds planes P+t, P+t+4 (the first tf32
// instruction's k = t, t+4) and P+8+t, P+12+t (the second's) into k slots 2t, 2t+1 and 2t+8, 2t+9
// of the bf16 instructions, the same assignment on the A and the B side.
//
// W [K][cin][cout] -> image [K][cin / 32][2][cout / 8][32][2] of uint4:
//   [0] = tf32 hi of W[P+t][n], W[P+t+4][n], W[P+8+t][n], W[P+12+t][n]       (n = 8 nt + g)
//   [1] = bf16 pairs (W[P+t], W[P+t+4]), (W[P+8+t], W[P+12+t]), then the same of W - hi
__global__ void k_rows_prepare(const float *__restrict__ w, uint4 *__restrict__ img, int K, int cin, int cout) {
  const int nt_n = cout / 8, nch = cin / kRChunk;
  const long long total = (long long)K * nch * 2 * nt_n * 32;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int lane = (int)(i & 31);
  long long r = i >> 5;
  const int nt = (int)(r % nt_n);
  r /= nt_n;
  const int kp = (int)(r & 1);
  r >>= 1;
  const int c = (int)(r % nch);
  const int k = (int)(r / nch);
  const int g = lane >> 2, t = lane & 3;
  const int p0 = c * kRChunk + kp * 16 + t, n = nt * 8 + g;
  const float *wk = w + ((long long)k * cin + p0) * cout + n;
  const float x0 = wk[0], x1 = wk[4 * (long long)cout], x2 = wk[8 * (long long)cout], x3 = wk[12 * (long long)cout];
  uint4 hi, lo;
  rows_split(x0, hi.x, lo.x);
  rows_split(x1, hi.y, lo.y);
  rows_split(x2, hi.z, lo.z);
  rows_split(x3, hi.w, lo.w);
  uint4 pk;
  pk.x = rows_pack_bf16(x0, x1);
  pk.y = rows_pack_bf16(x2, x3);
  pk.z = rows_pack_bf16(__uint_as_float(lo.x), __uint_as_float(lo.y));
  pk.w = rows_pack_bf16(__uint_as_float(lo.z), __uint_as_float(lo.w));
  img[2 * i] = hi;
  img[2 * i + 1] = pk;
}

// The image of the bf16 three-term form: [K][cin / 32][2][cout / 8][32] of uint4 =
//   bf16 pairs (h(W[P+t]), h(W[P+t+4])), (h(W[P+8+t]), h(W[P+12+t])), then the same of m = bf16(W - h)
__global__ void k_rows_prepare_b3(const float *__restrict__ w, uint4 *__restrict__ img, int K, int cin, int cout) {
  const int nt_n = cout / 8, nch = cin / kRChunk;
  const long long total = (long long)K * nch * 2 * nt_n * 32;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int lane = (int)(i & 31);
  long long r = i >> 5;
  const int nt = (int)(r % nt_n);
  r /= nt_n;
  const int kp = (int)(r & 1);
  r >>= 1;
  const int c = (int)(r % nch);
  const int k = (int)(r / nch);
  const int g = lane >> 2, t = lane & 3;
  const int p0 = c * kRChunk + kp * 16 + t, n = nt * 8 + g;
  const float *wk = w + ((long long)k * cin + p0) * cout + n;
  float x[4] = {wk[0], wk[4 * (long long)cout], wk[8 * (long long)cout], wk[12 * (long long)cout]};
  float m[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) m[e] = x[e] - __bfloat162float(__float2bfloat16_rn(x[e]));
  uint4 q;
  q.x = rows_pack_bf16(x[0], x[1]);
  q.y = rows_pack_bf16(x[2], x[3]);
  q.z = rows_pack_bf16(m[0], m[1]);
  q.w = rows_pack_bf16(m[2], m[3]);
  img[i] = q;
}

// a pair of floats as a bf16 pair (round to nearest) and the pair of what the rounding left over
__device__ __forceinline__ void rows_split_bf16(float a, float b, unsigned &h, unsigned &m) {
  h = rows_pack_bf16(a, b);
  const float ra = a - __uint_as_float(h << 16), rb = b - __uint_as_float(h & 0xFFFF0000u);
  m = rows_pack_bf16(ra, rb);
}

// One (offset, 32-plane chunk) step of a warp: its two 16-row tiles times the slab.
// D fragment: d[mt][nt] = rows (g, g + 8) of tile mt x planes 8 nt + 2 t, + 1.
// The A values are read with scalar loads in fragment order.  (Reading a lane's eight planes of a
// row with two 128-bit loads and picking the fragments out of them makes the compiler move every
// value into place: 2.2 register moves per tensor instruction, measured on this kernel and on a
// probe; with scalar loads there are none.)
// A 16-row tile without a rule for the offset (m0 / m1 = 0, warp-uniform) is left out.  Tried and
// not kept: always multiplying both tiles (16 % more tensor instructions; faster by 5 % for 32
// output planes, slower by 12 % for 64); accumulators of their own for the two small terms (more
// accurate, 2e-6, but the registers cost more warps than the shorter dependency chains gain);
// weight fragments held two k-blocks ahead in registers (same); the image without the split,
// hi and lo made in registers (half the L2 traffic, 6 % slower); both tiles' instructions interleaved
// in the tf32 + bf16 form (5 % slower: registers); no shared memory at all, the A values read straight
// from the feature matrix one half-step ahead (27 % slower: registers, and the loads' latency).
// MODE (a TcMode): TC_TF32X3 as described above; TC_TF32 only the two tf32 instructions, on the values as
// they are (the tensor core drops the low mantissa bits); TC_BF16 only the bf16 instruction x x W.  The
// single-pass modes read only their half of the weight image.  TC_BF16X3: the three bf16 products of the
// h / m split (bp = {h pair, h pair, m pair, m pair} of the image of k_rows_prepare_b3): three tensor
// instructions per 16 planes instead of four, and half the weight image.
template <int NT, int MODE = TC_TF32X3>
__device__ __forceinline__ void rows_tile16v(float (&d)[NT][4], const float (&x)[8], const unsigned (&bh)[NT][4],
                                             const unsigned (&bp)[NT][4]);

template <int NT, int MODE = TC_TF32X3>
__device__ __forceinline__ void rows_tile16(float (&d)[NT][4], const float *ap, const unsigned (&bh)[NT][4],
                                            const unsigned (&bp)[NT][4]) {
  const float x[8] = {ap[0], ap[4], ap[8], ap[12],
                      ap[8 * kRAStride], ap[8 * kRAStride + 4], ap[8 * kRAStride + 8], ap[8 * kRAStride + 12]};
  rows_tile16v<NT, MODE>(d, x, bh, bp);
}

// x[0..3]: planes P+t, P+t+4, P+8+t, P+12+t of row g; x[4..7]: the same of row g + 8
template <int NT, int MODE>
__device__ __forceinline__ void rows_tile16v(float (&d)[NT][4], const float (&x)[8], const unsigned (&bh)[NT][4],
                                             const unsigned (&bp)[NT][4]) {
  const float x00 = x[0], x01 = x[1], x02 = x[2], x03 = x[3], x10 = x[4], x11 = x[5], x12 = x[6], x13 = x[7];
  if (MODE == TC_BF16) {
    unsigned ax[4];
    ax[0] = rows_pack_bf16(x00, x01);
    ax[1] = rows_pack_bf16(x10, x11);
    ax[2] = rows_pack_bf16(x02, x03);
    ax[3] = rows_pack_bf16(x12, x13);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const unsigned b[2] = {bp[nt][0], bp[nt][1]};
      rows_mma_bf16(d[nt], ax, b);
    }
    return;
  }
  if (MODE == TC_BF16X3) {
    unsigned ah[4], am[4];
    rows_split_bf16(x00, x01, ah[0], am[0]);
    rows_split_bf16(x10, x11, ah[1], am[1]);
    rows_split_bf16(x02, x03, ah[2], am[2]);
    rows_split_bf16(x12, x13, ah[3], am[3]);
    // the small terms first; consecutive instructions write different accumulators
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const unsigned b[2] = {bp[nt][0], bp[nt][1]};
      rows_mma_bf16(d[nt], am, b);
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const unsigned b[2] = {bp[nt][2], bp[nt][3]};
      rows_mma_bf16(d[nt], ah, b);
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const unsigned b[2] = {bp[nt][0], bp[nt][1]};
      rows_mma_bf16(d[nt], ah, b);
    }
    return;
  }
  if (MODE == TC_TF32) {
    const unsigned h0[4] = {__float_as_uint(x00), __float_as_uint(x10), __float_as_uint(x01), __float_as_uint(x11)};
    const unsigned h1[4] = {__float_as_uint(x02), __float_as_uint(x12), __float_as_uint(x03), __float_as_uint(x13)};
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const unsigned b[2] = {bh[nt][0], bh[nt][1]};
      rows_mma(d[nt], h0, b);
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const unsigned b[2] = {bh[nt][2], bh[nt][3]};
      rows_mma(d[nt], h1, b);
    }
    return;
  }
  unsigned h0[4], h1[4], l[8];
  rows_split(x00, h0[0], l[0]);
  rows_split(x10, h0[1], l[1]);
  rows_split(x01, h0[2], l[2]);
  rows_split(x11, h0[3], l[3]);
  rows_split(x02, h1[0], l[4]);
  rows_split(x12, h1[1], l[5]);
  rows_split(x03, h1[2], l[6]);
  rows_split(x13, h1[3], l[7]);
  unsigned alo[4], ax[4];
  alo[0] = rows_pack_bf16(__uint_as_float(l[0]), __uint_as_float(l[2]));  // row g:     planes P+t, P+t+4
  alo[1] = rows_pack_bf16(__uint_as_float(l[1]), __uint_as_float(l[3]));  // row g + 8
  alo[2] = rows_pack_bf16(__uint_as_float(l[4]), __uint_as_float(l[6]));  // row g:     planes P+8+t, P+12+t
  alo[3] = rows_pack_bf16(__uint_as_float(l[5]), __uint_as_float(l[7]));
  ax[0] = rows_pack_bf16(x00, x01);
  ax[1] = rows_pack_bf16(x10, x11);
  ax[2] = rows_pack_bf16(x02, x03);
  ax[3] = rows_pack_bf16(x12, x13);
  // the small terms first; consecutive instructions write different accumulators
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const unsigned b[2] = {bp[nt][0], bp[nt][1]};
    rows_mma_bf16(d[nt], alo, b);
  }
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const unsigned b[2] = {bp[nt][2], bp[nt][3]};
    rows_mma_bf16(d[nt], ax, b);
  }
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const unsigned b[2] = {bh[nt][0], bh[nt][1]};
    rows_mma(d[nt], h0, b);
  }
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const unsigned b[2] = {bh[nt][2], bh[nt][3]};
    rows_mma(d[nt], h1, b);
  }
}

// The three bf16 products of one 16 x 16 A tile whose fragments are split already (ah = h pairs, am = m pairs, in
// the plane order of rows_tile16v) against the slab's weights.
template <int NT>
__device__ __forceinline__ void rows_mma3(float (&d)[NT][4], const unsigned (&ah)[4], const unsigned (&am)[4],
                                          const unsigned (&bp)[NT][4]) {
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const unsigned b[2] = {bp[nt][0], bp[nt][1]};
    rows_mma_bf16(d[nt], am, b);
  }
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const unsigned b[2] = {bp[nt][2], bp[nt][3]};
    rows_mma_bf16(d[nt], ah, b);
  }
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const unsigned b[2] = {bp[nt][0], bp[nt][1]};
    rows_mma_bf16(d[nt], ah, b);
  }
}

template <int NT, int MODE>
__device__ __forceinline__ void rows_chunk(float (&d)[2][NT][4], const float *a_stage, const uint4 *w_slab,
                                           int lane, unsigned m0, unsigned m1) {
  const int g = lane >> 2, t = lane & 3;
  const float *a_lane = a_stage + g * kRAStride + t;
#pragma unroll
  for (int kp = 0; kp < 2; ++kp) {
    unsigned bh[NT][4], bp[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      if (MODE == TC_BF16X3) {
        const uint4 q = __ldg(w_slab + (kp * NT + nt) * 32 + lane);
        bp[nt][0] = q.x, bp[nt][1] = q.y, bp[nt][2] = q.z, bp[nt][3] = q.w;
        continue;
      }
      if (MODE != TC_BF16) {
        const uint4 q0 = __ldg(w_slab + ((kp * NT + nt) * 32 + lane) * 2);
        bh[nt][0] = q0.x, bh[nt][1] = q0.y, bh[nt][2] = q0.z, bh[nt][3] = q0.w;
      }
      if (MODE == TC_BF16) {  // only the pair of bf16 W
        const uint2 q1 = __ldg(reinterpret_cast<const uint2 *>(w_slab + ((kp * NT + nt) * 32 + lane) * 2 + 1));
        bp[nt][0] = q1.x, bp[nt][1] = q1.y;
      } else if (MODE == TC_TF32X3) {
        const uint4 q1 = __ldg(w_slab + ((kp * NT + nt) * 32 + lane) * 2 + 1);
        bp[nt][0] = q1.x, bp[nt][1] = q1.y, bp[nt][2] = q1.z, bp[nt][3] = q1.w;
      }
    }
    if (m0 != 0) rows_tile16<NT, MODE>(d[0], a_lane + kp * 16, bh, bp);
    if (m1 != 0) rows_tile16<NT, MODE>(d[1], a_lane + 16 * kRAStride + kp * 16, bh, bp);
  }
}

// NCH: the number of 32-plane input chunks as a constant (0: the run-time argument)
template <int NT, int MODE, int NCH>
__global__ void __launch_bounds__(32)
k_conv_rows(const float *__restrict__ in, int ld_in, long long n_in, float *__restrict__ out, int ld_out,
            long long n_out, const uint4 *__restrict__ img, const float *__restrict__ bias,
            const float *__restrict__ bn_scale, const float *__restrict__ bn_shift, float leak,
            const int *__restrict__ nbr, int K, int nch_arg, int *flags) {
  const int nch = NCH ? NCH : nch_arg;
  // the specialised kernels are launched on dense matrices only: the row strides are constants as well
  if (NCH) {
    ld_in = NCH * kRChunk;
    ld_out = NT * 8;
  }
  constexpr unsigned kFull = 0xffffffffu;
  constexpr int kSlab = (MODE == TC_BF16X3 ? 2 : 4) * NT * 32;  // uint4 per (offset, chunk) slab
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int lane = threadIdx.x;
  float *a_ring = reinterpret_cast<float *>(smem_raw);
  const long long row0 = (long long)blockIdx.x * 32;
  if (row0 >= n_out) return;
  const long long my_row = row0 + lane;

  // ---- which offsets have a rule for any of the warp's rows ---------------------------------------
  unsigned wmask = 0;
  for (int k0 = 0; k0 < K; k0 += 8) {
    int v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int k = k0 + u;
      v[u] = (k < K && my_row < n_out) ? __ldg(nbr + (long long)k * n_out + my_row) : -1;
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      if (v[u] >= n_in) atomicOr(flags, FLAG_BAD_ROW);
      if (__any_sync(kFull, v[u] >= 0 && v[u] < n_in)) wmask |= 1u << (k0 + u);
    }
  }

  float d[2][NT][4];
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) d[mt][nt][0] = d[mt][nt][1] = d[mt][nt][2] = d[mt][nt][3] = 0.f;

  // Gathers run kRAStages - 1 steps ahead of the arithmetic; the rulebook entries of the rows (one
  // per lane) are read one offset ahead of the gather that needs them and handed to the copying
  // lanes by shuffles.
  unsigned irem = wmask;  // offsets whose gathers are still to be issued
  auto load_entry = [&](unsigned rem) -> int {
    if (!rem || my_row >= n_out) return -1;
    const int v = __ldg(nbr + (long long)(__ffs(rem) - 1) * n_out + my_row);
    return v < n_in ? v : -1;
  };
  int vcur = load_entry(irem), vnext = load_entry(irem & (irem - 1));
  int ic = 0, istage = 0;
  const int piece = (lane & 7) * 4, prow = lane >> 3;
  unsigned mk_q[kRAStages];  // which rows of the steps in flight have a rule
#pragma unroll
  for (int s = 0; s < kRAStages; ++s) mk_q[s] = 0;
  auto issue = [&] {
#pragma unroll
    for (int s = 0; s < kRAStages - 1; ++s) mk_q[s] = mk_q[s + 1];
    mk_q[kRAStages - 1] = 0;
    if (irem) {
      const unsigned mk = __ballot_sync(kFull, vcur >= 0);
      mk_q[kRAStages - 1] = mk;
      float *dst = a_ring + istage * kRStageFloats + piece;
      const float *col = in + ic * kRChunk + piece;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if ((i < 4 ? (mk & 0xFFFFu) : (mk >> 16)) == 0) continue;  // such a tile is not read
        const int rr = prow + 4 * i;
        const int v = __shfl_sync(kFull, vcur, rr);
        cp_async16(smem_u32(dst + rr * kRAStride), v >= 0 ? col + (long long)v * ld_in : in, v >= 0 ? 16u : 0u);
      }
      if (++ic == nch) {
        ic = 0;
        irem &= irem - 1;
        vcur = vnext;
        vnext = load_entry(irem & (irem - 1));
      }
    }
    cp_async_commit();  // one group per call, empty or not: wait_group's count stays fixed
    istage = istage + 1 == kRAStages ? 0 : istage + 1;
  };
#pragma unroll
  for (int s = 0; s < kRAStages - 1; ++s) issue();

  int cstage = 0;
  for (unsigned rem = wmask; rem; rem &= rem - 1) {
    const int k = __ffs(rem) - 1;
#pragma unroll
    for (int c = 0; c < (NCH ? NCH : nch); ++c) {
      cp_async_wait<kRAStages - 2>();  // the rows of this step have landed (this lane's copies)
      __syncwarp();                    // ... every lane's; and the previous step's reads are done
      issue();
      rows_chunk<NT, MODE>(d, a_ring + cstage * kRStageFloats, img + ((long long)k * nch + c) * kSlab, lane,
                           mk_q[0] & 0xFFFFu, mk_q[0] >> 16);
      cstage = cstage + 1 == kRAStages ? 0 : cstage + 1;
    }
  }
  cp_async_wait<0>();

  // ---- the warp's rows, written once ---------------------------------------------------------------
  const int g = lane >> 2, t2 = (lane & 3) * 2;
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const long long r = row0 + mt * 16 + h * 8 + g;
      if (r >= n_out) continue;
      float *dst = out + r * ld_out + t2;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        float2 v = make_float2(d[mt][nt][h * 2], d[mt][nt][h * 2 + 1]);
        if (bias) {
          const float2 b = __ldg(reinterpret_cast<const float2 *>(bias + nt * 8 + t2));
          v.x += b.x;
          v.y += b.y;
        }
        if (bn_scale) {
          const float2 sc = __ldg(reinterpret_cast<const float2 *>(bn_scale + nt * 8 + t2));
          const float2 sh = __ldg(reinterpret_cast<const float2 *>(bn_shift + nt * 8 + t2));
          v.x = rows_epilogue(v.x, sc.x, sh.x, leak);
          v.y = rows_epilogue(v.y, sc.y, sh.y, leak);
        }
        __stcs(reinterpret_cast<float2 *>(dst + nt * 8), v);
      }
    }
}

template <int NT, int MODE, int NCH = 0>
static int launch_rows(const float *in, int ld_in, long long n_in, float *out, int ld_out, long long n_out,
                       const uint4 *img, const float *bias, const float *bn_scale, const float *bn_shift, float leak,
                       const int *table, int K, int nch, int *flags, cudaStream_t stream) {
  static bool configured[64] = {false};
  int dev = 0;
  SCN_CUDA_CHECK(cudaGetDevice(&dev));
  const size_t smem = (size_t)kRAStages * kRStageFloats * sizeof(float);
  auto kernel = k_conv_rows<NT, MODE, NCH>;
  if (dev >= 64 || !configured[dev]) {
    SCN_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    // 9 KB of shared memory per warp: a carve-out of 80 % holds 20 warps per SM (the registers allow
    // more with 32 output planes), the rest of the 256 KB stays L1 for the weight image
    // with 64 output planes the registers of the three-term mode hold the SM to 12 warps (110 KB of rings): half
    // the SM's memory is enough and the other half serves the weight fragments as L1 (3 % faster)
    // (measured with the bf16 form: carve-outs of 70, 80, 90 and 100 % give the same times within 2 %)
    SCN_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                        NT > 4 ? (MODE == TC_TF32X3 ? 50 : MODE == TC_BF16X3 ? 70 : 80) : 80));
    if (dev < 64) configured[dev] = true;
  }
  SCN_LAUNCH(kernel, (unsigned)ceil_div(n_out, 32LL), 32, smem, stream, in, ld_in, n_in, out, ld_out, n_out, img, bias,
             bn_scale, bn_shift, leak, table, K, nch, flags);
  SCN_CUDA_CHECK(cudaGetLastError());
  return SCN_OK;
}

// ---- first layers: at most four input planes --------------------------------------------------------
// The same row-stationary scheme without shared memory: a lane's A fragment of m16n8k4 is one
// input value of two rows, read straight from the feature matrix (the rows are 4 to 16 bytes long,
// too short and too misaligned for 16-byte copies), the B fragments come from a 2 KB-per-offset
// image that stays in L1.  Four offsets are in flight at a time.
__device__ __forceinline__ void rows_mma_k4(float (&d)[4], const unsigned (&a)[2], unsigned b) {
  asm volatile(
      "mma.sync.aligned.m16n8k4.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(b));
}

// W [K][cin][cout] -> image [K][cout / 8][32] of (hi, lo) of W[k][t][8 nt + g], zero for t >= cin
__global__ void k_rows_thin_prepare(const float *__restrict__ w, uint2 *__restrict__ img, int K, int cin, int cout) {
  const int nt_n = cout / 8;
  const long long total = (long long)K * nt_n * 32;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int lane = (int)(i & 31), nt = (int)((i >> 5) % nt_n), k = (int)((i >> 5) / nt_n);
  const int g = lane >> 2, t = lane & 3;
  uint2 o = make_uint2(0u, 0u);
  if (t < cin) rows_split(w[((long long)k * cin + t) * cout + nt * 8 + g], o.x, o.y);
  img[i] = o;
}

template <int NT>
__global__ void __launch_bounds__(128)
k_conv_rows_thin(const float *__restrict__ in, long long n_in, float *__restrict__ out, long long n_out,
                 const uint2 *__restrict__ img, const float *__restrict__ bias, const float *__restrict__ bn_scale,
                 const float *__restrict__ bn_shift, float leak, const int *__restrict__ nbr, int K, int cin,
                 int *flags) {
  constexpr unsigned kFull = 0xffffffffu;
  constexpr int kGroup = 4;  // offsets in flight
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const long long row0 = ((long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * 32;
  if (row0 >= n_out) return;
  const long long my_row = row0 + lane;
  const bool t_ok = t < cin;
  float d[2][NT][4];
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) d[mt][nt][0] = d[mt][nt][1] = d[mt][nt][2] = d[mt][nt][3] = 0.f;

  for (int k0 = 0; k0 < K; k0 += kGroup) {
    int v[kGroup];
#pragma unroll
    for (int u = 0; u < kGroup; ++u) {
      const int k = k0 + u;
      v[u] = (k < K && my_row < n_out) ? __ldg(nbr + (long long)k * n_out + my_row) : -1;
    }
    float x[kGroup][2][2];  // [offset][tile][row g / g + 8]: plane t of the input row
#pragma unroll
    for (int u = 0; u < kGroup; ++u) {
      if (v[u] >= n_in) {
        atomicOr(flags, FLAG_BAD_ROW);
        v[u] = -1;
      }
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int idx = __shfl_sync(kFull, v[u], mt * 16 + h * 8 + g);
          x[u][mt][h] = (idx >= 0 && t_ok) ? __ldg(in + (long long)idx * cin + t) : 0.f;
        }
    }
#pragma unroll
    for (int u = 0; u < kGroup; ++u) {
      const unsigned mk = __ballot_sync(kFull, v[u] >= 0);
      if (mk == 0) continue;
      unsigned bh[NT], bl[NT];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const uint2 b = __ldg(img + ((long long)(k0 + u) * NT + nt) * 32 + lane);
        bh[nt] = b.x, bl[nt] = b.y;
      }
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        if (((mt == 0) ? (mk & 0xFFFFu) : (mk >> 16)) == 0) continue;
        unsigned ah[2], al[2];
        rows_split(x[u][mt][0], ah[0], al[0]);
        rows_split(x[u][mt][1], ah[1], al[1]);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) rows_mma_k4(d[mt][nt], al, bh[nt]);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) rows_mma_k4(d[mt][nt], ah, bl[nt]);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) rows_mma_k4(d[mt][nt], ah, bh[nt]);
      }
    }
  }

  const int t2 = t * 2;
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const long long r = row0 + mt * 16 + h * 8 + g;
      if (r >= n_out) continue;
      float *dst = out + r * (NT * 8) + t2;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        float2 y = make_float2(d[mt][nt][h * 2], d[mt][nt][h * 2 + 1]);
        if (bias) {
          const float2 b = __ldg(reinterpret_cast<const float2 *>(bias + nt * 8 + t2));
          y.x += b.x;
          y.y += b.y;
        }
        if (bn_scale) {
          const float2 sc = __ldg(reinterpret_cast<const float2 *>(bn_scale + nt * 8 + t2));
          const float2 sh = __ldg(reinterpret_cast<const float2 *>(bn_shift + nt * 8 + t2));
          y.x = rows_epilogue(y.x, sc.x, sh.x, leak);
          y.y = rows_epilogue(y.y, sc.y, sh.y, leak);
        }
        __stcs(reinterpret_cast<float2 *>(dst + nt * 8), y);
      }
    }
}

// ---- the same in the bf16 three-term form: four offsets per tensor instruction ------------------------------
// With at most four input planes an m16n8k16 instruction has room for four filter offsets: k = 4 o + p for
// offset o of a group of four and plane p.  A lane's A fragment is then two planes (2 (t & 1), + 1) of offsets
// t >> 1 and 2 + (t >> 1) of rows g and g + 8, read straight from the feature matrix and split into the bf16
// parts h and m; the B fragments come from an image of [group][n-tile][lane] (h pairs, m pairs).  Per 16-row
// tile and group of four offsets: 3 instructions per 8 output planes, against 12 of m16n8k4 in the tf32 form
// (which is bound by the issue rate of those: 0.27 ms for 1.59 M rows, 27 offsets, 3 -> 32 planes; this form
// 0.21 ms, bound by its scalar loads of the input values).
__global__ void k_rows_thin_prepare_b3(const float *__restrict__ w, uint4 *__restrict__ img, int K, int cin, int cout) {
  const int nt_n = cout / 8, n_groups = (K + 3) / 4;
  const long long total = (long long)n_groups * nt_n * 32;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int lane = (int)(i & 31), nt = (int)((i >> 5) % nt_n), grp = (int)((i >> 5) / nt_n);
  const int g = lane >> 2, t = lane & 3, p0 = 2 * (t & 1);
  float x[2][2];  // [k half: offsets t >> 1 and 2 + (t >> 1)][plane p0, p0 + 1]
#pragma unroll
  for (int e = 0; e < 2; ++e)
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const int k = grp * 4 + 2 * e + (t >> 1), p = p0 + q;
      x[e][q] = (k < K && p < cin) ? w[((long long)k * cin + p) * cout + nt * 8 + g] : 0.f;
    }
  uint4 o;
  rows_split_bf16(x[0][0], x[0][1], o.x, o.z);
  rows_split_bf16(x[1][0], x[1][1], o.y, o.w);
  img[i] = o;  // (b0 h, b1 h, b0 m, b1 m)
}

template <int NT>
__global__ void __launch_bounds__(128)
k_conv_rows_thin_b3(const float *__restrict__ in, long long n_in, float *__restrict__ out, long long n_out,
                    const uint4 *__restrict__ img, const float *__restrict__ bias, const float *__restrict__ bn_scale,
                    const float *__restrict__ bn_shift, float leak, const int *__restrict__ nbr, int K, int cin,
                    int *flags) {
  constexpr unsigned kFull = 0xffffffffu;
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const long long row0 = ((long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * 32;
  if (row0 >= n_out) return;
  const long long my_row = row0 + lane;
  const int p0 = 2 * (t & 1), o_lo = t >> 1;
  const bool p0_ok = p0 < cin, p1_ok = p0 + 1 < cin;
  float d[2][NT][4];
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) d[mt][nt][0] = d[mt][nt][1] = d[mt][nt][2] = d[mt][nt][3] = 0.f;

  const int n_groups = (K + 3) / 4;
  int v[4];
#pragma unroll
  for (int u = 0; u < 4; ++u) v[u] = (u < K && my_row < n_out) ? __ldg(nbr + (long long)u * n_out + my_row) : -1;
  for (int grp = 0; grp < n_groups; ++grp) {
    int vn[4];  // the next group's rulebook entries, in flight while this group is computed
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int k = (grp + 1) * 4 + u;
      vn[u] = (k < K && my_row < n_out) ? __ldg(nbr + (long long)k * n_out + my_row) : -1;
    }
    unsigned any = 0;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (v[u] >= n_in) {
        atomicOr(flags, FLAG_BAD_ROW);
        v[u] = -1;
      }
      any |= __ballot_sync(kFull, v[u] >= 0);
    }
    if (any != 0) {
      // this lane's values: [tile][row g / g + 8][k half][plane p0 / p0 + 1]
      float x[2][2][2][2];
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int src = mt * 16 + h * 8 + g;
          const int i0 = __shfl_sync(kFull, v[0], src), i1 = __shfl_sync(kFull, v[1], src);
          const int i2 = __shfl_sync(kFull, v[2], src), i3 = __shfl_sync(kFull, v[3], src);
          const int idx[2] = {o_lo ? i1 : i0, o_lo ? i3 : i2};
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const float *row = in + (long long)idx[e] * cin + p0;
            x[mt][h][e][0] = (idx[e] >= 0 && p0_ok) ? __ldg(row) : 0.f;
            x[mt][h][e][1] = (idx[e] >= 0 && p1_ok) ? __ldg(row + 1) : 0.f;
          }
        }
      unsigned bp[NT][4];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const uint4 q = __ldg(img + ((long long)grp * NT + nt) * 32 + lane);
        bp[nt][0] = q.x, bp[nt][1] = q.y, bp[nt][2] = q.z, bp[nt][3] = q.w;
      }
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        if (((mt == 0) ? (any & 0xFFFFu) : (any >> 16)) == 0) continue;
        unsigned ah[4], am[4];  // a0: row g, k half 0; a1: row g + 8, half 0; a2: row g, half 1; a3: row g + 8, half 1
        rows_split_bf16(x[mt][0][0][0], x[mt][0][0][1], ah[0], am[0]);
        rows_split_bf16(x[mt][1][0][0], x[mt][1][0][1], ah[1], am[1]);
        rows_split_bf16(x[mt][0][1][0], x[mt][0][1][1], ah[2], am[2]);
        rows_split_bf16(x[mt][1][1][0], x[mt][1][1][1], ah[3], am[3]);
        rows_mma3<NT>(d[mt], ah, am, bp);
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) v[u] = vn[u];
  }

  const int t2 = t * 2;
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const long long r = row0 + mt * 16 + h * 8 + g;
      if (r >= n_out) continue;
      float *dst = out + r * (NT * 8) + t2;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        float2 y = make_float2(d[mt][nt][h * 2], d[mt][nt][h * 2 + 1]);
        if (bias) {
          const float2 b = __ldg(reinterpret_cast<const float2 *>(bias + nt * 8 + t2));
          y.x += b.x;
          y.y += b.y;
        }
        if (bn_scale) {
          const float2 sc = __ldg(reinterpret_cast<const float2 *>(bn_scale + nt * 8 + t2));
          const float2 sh = __ldg(reinterpret_cast<const float2 *>(bn_shift + nt * 8 + t2));
          y.x = rows_epilogue(y.x, sc.x, sh.x, leak);
          y.y = rows_epilogue(y.y, sc.y, sh.y, leak);
        }
        __stcs(reinterpret_cast<float2 *>(dst + nt * 8), y);
      }
    }
}

bool conv_rows_thin_supported(const float *out, const float *bias, int cin, int cout, int groups) {
  return groups == 1 && cin >= 1 && cin <= 4 && (cout == 16 || cout == 32 || cout == 64) &&
         (uintptr_t)out % 8 == 0 && (uintptr_t)bias % 8 == 0;
}

int conv_forward_rows_thin(const float *in, long long n_in, float *out, long long n_out, const float *weight,
                           const float *bias, const float *bn_scale, const float *bn_shift, float leak,
                           const int *table, int K, int cin, int cout, int *flags, cudaStream_t stream) {
  if (n_out == 0) return SCN_OK;
  if (split_mode_of_env() == TC_BF16X3) {  // the default form of the fp32-class mode
    const long long total = (long long)((K + 3) / 4) * (cout / 8) * 32;
    WeightImage wi;
    bool build = true;
    SCN_TRY(weight_image_get(WIMG_ROWS_THIN, K, cin, cout, 1, (size_t)total * sizeof(uint4), stream, &wi, &build));
    uint4 *img = (uint4 *)wi.ptr;
    if (build)
      SCN_LAUNCH(k_rows_thin_prepare_b3, (unsigned)ceil_div(total, 256LL), 256, 0, stream, weight, img, K, cin, cout);
    const unsigned grid = (unsigned)ceil_div(n_out, 128LL);
    if (cout == 16)
      SCN_LAUNCH(k_conv_rows_thin_b3<2>, grid, 128, 0, stream, in, n_in, out, n_out, img, bias, bn_scale, bn_shift, leak, table, K, cin, flags);
    else if (cout == 32)
      SCN_LAUNCH(k_conv_rows_thin_b3<4>, grid, 128, 0, stream, in, n_in, out, n_out, img, bias, bn_scale, bn_shift, leak, table, K, cin, flags);
    else
      SCN_LAUNCH(k_conv_rows_thin_b3<8>, grid, 128, 0, stream, in, n_in, out, n_out, img, bias, bn_scale, bn_shift, leak, table, K, cin, flags);
    const cudaError_t e = cudaGetLastError();
    const int rf = weight_image_put(wi, stream);
    SCN_CUDA_CHECK(e);
    return rf;
  }
  const long long total = (long long)K * (cout / 8) * 32;
  WeightImage wi;
  bool build = true;
  SCN_TRY(weight_image_get(WIMG_ROWS_THIN, K, cin, cout, 0, (size_t)total * sizeof(uint2), stream, &wi, &build));
  uint2 *img = (uint2 *)wi.ptr;
  if (build)
    SCN_LAUNCH(k_rows_thin_prepare, (unsigned)ceil_div(total, 256LL), 256, 0, stream, weight, img, K, cin, cout);
  const unsigned grid = (unsigned)ceil_div(n_out, 128LL);
  if (cout == 16)
    SCN_LAUNCH(k_conv_rows_thin<2>, grid, 128, 0, stream, in, n_in, out, n_out, img, bias, bn_scale, bn_shift, leak, table, K, cin, flags);
  else if (cout == 32)
    SCN_LAUNCH(k_conv_rows_thin<4>, grid, 128, 0, stream, in, n_in, out, n_out, img, bias, bn_scale, bn_shift, leak, table, K, cin, flags);
  else
    SCN_LAUNCH(k_conv_rows_thin<8>, grid, 128, 0, stream, in, n_in, out, n_out, img, bias, bn_scale, bn_shift, leak, table, K, cin, flags);
  const cudaError_t e = cudaGetLastError();
  const int rf = weight_image_put(wi, stream);
  SCN_CUDA_CHECK(e);
  return rf;
}

// ---- transposed rulebooks whose output rows have one rule each (Deconvolution with filter = stride) --------
// Run from the output side, the children of a coarse site sit at different filter offsets, so a 16-row tile of
// fine rows meets several offsets with a few rows each.  Run from the input side a warp takes 32 consecutive
// COARSE rows (dense, no gather, no transposed table), multiplies them with W[k] for every offset k at which
// any of them has a child, and stores each product row at the child's row: every fine row is written exactly
// once (filter = stride makes the children of different sites and offsets disjoint and covers every fine
// site), so nothing is accumulated in memory.  Measured 10 % faster than the gather form (64 -> 32 planes,
// 1.59 M fine rows: 0.33 against 0.37 ms; rows sorted by coordinate keep the gather form's tiles to two offsets);
// with the bf16 three-term form 0.26 ms, and 0.17 ms once the warp's input rows are read and split once and
// held in registers for all offsets (32 output planes, at most 64 input planes).
// NCH: the number of 32-plane input chunks as a constant (0: the run-time argument), as in k_conv_rows.
template <int NT, int MODE, int NCH>
__global__ void __launch_bounds__(32)
k_conv_rows_scatter(const float *__restrict__ in, int ld_in, long long n_in, float *__restrict__ out, int ld_out,
                    long long n_out, const uint4 *__restrict__ img, const float *__restrict__ bias,
                    const float *__restrict__ bn_scale, const float *__restrict__ bn_shift, float leak,
                    const int *__restrict__ child_of /* [K][n_in] -> output row */, int K, int nch_arg, int *flags) {
  const int nch = NCH ? NCH : nch_arg;
  if (NCH) {  // dense matrices: constant row strides
    ld_in = NCH * kRChunk;
    ld_out = NT * 8;
  }
  constexpr unsigned kFull = 0xffffffffu;
  constexpr int kSlab = (MODE == TC_BF16X3 ? 2 : 4) * NT * 32;
  const int lane = threadIdx.x, g = lane >> 2, t = lane & 3;
  const long long row0 = (long long)blockIdx.x * 32;
  if (row0 >= n_in) return;
  const long long my_row = row0 + lane;
  const float *ap[2][2];  // rows g / g + 8 of the two tiles; rows past the end are read as zeros
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const long long r = row0 + mt * 16 + h * 8 + g;
      ap[mt][h] = r < n_in ? in + r * ld_in + t : nullptr;
    }
  // With 32 output planes and at most 64 input planes the warp's 32 input rows fit the registers as split
  // fragments (64 registers): they are read and split once and serve every filter offset, instead of being read
  // from the feature matrix and split again for each of the K offsets.
  constexpr int kHeldChunks = NT == 4 ? 2 : 3;
  const bool held = MODE == TC_BF16X3 && nch <= kHeldChunks;
  unsigned ah[2][kHeldChunks][2][4], am[2][kHeldChunks][2][4];  // [tile][chunk][k16 half][fragment register]
  if (MODE == TC_BF16X3 && held) {
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int c = 0; c < kHeldChunks; ++c)
#pragma unroll
        for (int kp = 0; kp < 2; ++kp) {
          float x[8];
#pragma unroll
          for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int e = 0; e < 4; ++e)
              x[h * 4 + e] = (c < nch && ap[mt][h]) ? __ldg(ap[mt][h] + c * kRChunk + kp * 16 + 4 * e) : 0.f;
          rows_split_bf16(x[0], x[1], ah[mt][c][kp][0], am[mt][c][kp][0]);
          rows_split_bf16(x[4], x[5], ah[mt][c][kp][1], am[mt][c][kp][1]);
          rows_split_bf16(x[2], x[3], ah[mt][c][kp][2], am[mt][c][kp][2]);
          rows_split_bf16(x[6], x[7], ah[mt][c][kp][3], am[mt][c][kp][3]);
        }
  }
  for (int k = 0; k < K; ++k) {
    int child = my_row < n_in ? __ldg(child_of + (long long)k * n_in + my_row) : -1;
    if (child >= n_out) {
      atomicOr(flags, FLAG_BAD_ROW);
      child = -1;
    }
    const unsigned mk = __ballot_sync(kFull, child >= 0);
    if (mk == 0) continue;
    float d[2][NT][4];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) d[mt][nt][0] = d[mt][nt][1] = d[mt][nt][2] = d[mt][nt][3] = 0.f;
#pragma unroll
    for (int c = 0; c < (NCH ? NCH : nch); ++c) {
      const uint4 *w_slab = img + ((long long)k * nch + c) * kSlab;
#pragma unroll
      for (int kp = 0; kp < 2; ++kp) {
        unsigned bh[NT][4], bp[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          if (MODE == TC_BF16X3) {
            const uint4 q = __ldg(w_slab + (kp * NT + nt) * 32 + lane);
            bp[nt][0] = q.x, bp[nt][1] = q.y, bp[nt][2] = q.z, bp[nt][3] = q.w;
          } else {
            const uint4 q0 = __ldg(w_slab + ((kp * NT + nt) * 32 + lane) * 2);
            const uint4 q1 = __ldg(w_slab + ((kp * NT + nt) * 32 + lane) * 2 + 1);
            bh[nt][0] = q0.x, bh[nt][1] = q0.y, bh[nt][2] = q0.z, bh[nt][3] = q0.w;
            bp[nt][0] = q1.x, bp[nt][1] = q1.y, bp[nt][2] = q1.z, bp[nt][3] = q1.w;
          }
        }
        const int off = c * kRChunk + kp * 16;
        if constexpr (MODE == TC_BF16X3) {
          if (held) {
#pragma unroll
            for (int mt = 0; mt < 2; ++mt) {
              if ((mt == 0 ? (mk & 0xFFFFu) : (mk >> 16)) == 0) continue;
              // (c is a loop variable: the chunk is picked with selects, which keeps the arrays in registers)
              unsigned fh[4], fm[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                fh[e] = c == 0 ? ah[mt][0][kp][e] : (c == 1 ? ah[mt][1][kp][e] : ah[mt][kHeldChunks - 1][kp][e]);
                fm[e] = c == 0 ? am[mt][0][kp][e] : (c == 1 ? am[mt][1][kp][e] : am[mt][kHeldChunks - 1][kp][e]);
              }
              rows_mma3<NT>(d[mt], fh, fm, bp);
            }
            continue;
          }
        }
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
          if ((mt == 0 ? (mk & 0xFFFFu) : (mk >> 16)) == 0) continue;
          float x[8];
#pragma unroll
          for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int e = 0; e < 4; ++e) x[h * 4 + e] = ap[mt][h] ? __ldg(ap[mt][h] + off + 4 * e) : 0.f;
          rows_tile16v<NT, MODE>(d[mt], x, bh, bp);
        }
      }
    }
    // each product row to its child's row
    const int t2 = t * 2;
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int dst_row = __shfl_sync(kFull, child, mt * 16 + h * 8 + g);
        if (dst_row < 0) continue;
        float *dst = out + (long long)dst_row * ld_out + t2;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          float2 v = make_float2(d[mt][nt][h * 2], d[mt][nt][h * 2 + 1]);
          if (bias) {
            const float2 bb = __ldg(reinterpret_cast<const float2 *>(bias + nt * 8 + t2));
            v.x += bb.x;
            v.y += bb.y;
          }
          if (bn_scale) {
            const float2 sc = __ldg(reinterpret_cast<const float2 *>(bn_scale + nt * 8 + t2));
            const float2 sh = __ldg(reinterpret_cast<const float2 *>(bn_shift + nt * 8 + t2));
            v.x = rows_epilogue(v.x, sc.x, sh.x, leak);
            v.y = rows_epilogue(v.y, sc.y, sh.y, leak);
          }
          __stcs(reinterpret_cast<float2 *>(dst + nt * 8), v);
        }
      }
  }
}

// out [n_out, cout]: row child_of[k][i] = bias + in[i] @ W[k] for every rule; every output row must have exactly
// one rule (the caller's promise).  Same shapes as conv_forward_rows.
int conv_forward_rows_scatter(const float *in, long long n_in, float *out, long long n_out, const float *weight,
                              const float *bias, const float *bn_scale, const float *bn_shift, float leak,
                              const int *child_of, int K, int cin, int cout, int *flags, cudaStream_t stream) {
  if (n_out == 0 || n_in == 0) return SCN_OK;
  const int nch = cin / kRChunk;
  const long long total = (long long)K * nch * 2 * (cout / 8) * 32;
  const bool b3 = split_mode_of_env() == TC_BF16X3;
  WeightImage wi;
  bool build = true;
  SCN_TRY(weight_image_get(b3 ? WIMG_ROWS_B3 : WIMG_ROWS, K, cin, cout, 0, (size_t)total * (b3 ? 1 : 2) * sizeof(uint4),
                           stream, &wi, &build));
  uint4 *img = (uint4 *)wi.ptr;
  if (build && b3)
    SCN_LAUNCH(k_rows_prepare_b3, (unsigned)ceil_div(total, 256LL), 256, 0, stream, weight, img, K, cin, cout);
  else if (build)
    SCN_LAUNCH(k_rows_prepare, (unsigned)ceil_div(total, 256LL), 256, 0, stream, weight, img, K, cin, cout);
  const unsigned grid = (unsigned)ceil_div(n_in, 32LL);
#define SCN_SCATTER_CALL(NT, MODE, NCH) \
  SCN_LAUNCH((k_conv_rows_scatter<NT, MODE, NCH>), grid, 32, 0, stream, in, cin, n_in, out, cout, n_out, img, bias, bn_scale, bn_shift, leak, child_of, K, nch, flags)
  const bool fixed = !(getenv("SCN_ROWS_NCH") && atoi(getenv("SCN_ROWS_NCH")) == 0);
  if (cout == 32) {
    if (b3 && fixed && nch == 2) SCN_SCATTER_CALL(4, TC_BF16X3, 2);
    else if (b3) SCN_SCATTER_CALL(4, TC_BF16X3, 0);
    else SCN_SCATTER_CALL(4, TC_TF32X3, 0);
  } else {
    if (b3 && fixed && nch == 3) SCN_SCATTER_CALL(8, TC_BF16X3, 3);
    else if (b3) SCN_SCATTER_CALL(8, TC_BF16X3, 0);
    else SCN_SCATTER_CALL(8, TC_TF32X3, 0);
  }
#undef SCN_SCATTER_CALL
  const cudaError_t e = cudaGetLastError();
  const int rf = weight_image_put(wi, stream);
  SCN_CUDA_CHECK(e);
  return rf;
}

bool conv_rows_supported(const float *in, const float *out, const float *weight, const float *bias, int K, int cin,
                         int cout, int groups) {
  return groups == 1 && K <= kRMaxK && cin % kRChunk == 0 && (cout == 32 || cout == 64) &&
         (uintptr_t)in % 16 == 0 && (uintptr_t)out % 8 == 0 && (uintptr_t)bias % 8 == 0 && (uintptr_t)weight % 4 == 0;
  // (the optional scale / shift vectors of the fused BatchNorm are this library's own allocations: aligned)
}

// out [n_out, cout] = bias + sum_k in[table[k][.]] @ W[k]; precision: SCN_PRECISION_TF32X3 (fp32-class accuracy),
// SCN_PRECISION_TF32 or SCN_PRECISION_BF16 (single pass)
int conv_forward_rows(const float *in, long long n_in, float *out, long long n_out, const float *weight,
                      const float *bias, const float *bn_scale, const float *bn_shift, float leak, const int *table,
                      int K, int cin, int cout, int precision, int *flags, cudaStream_t stream) {
  if (n_out == 0) return SCN_OK;
  const int nch = cin / kRChunk;
  const long long total = (long long)K * nch * 4 * (cout / 8) * 32;
  const bool b3 = precision == SCN_PRECISION_TF32X3 && split_mode_of_env() == TC_BF16X3;
  WeightImage wi;
  bool build = true;
  SCN_TRY(weight_image_get(b3 ? WIMG_ROWS_B3 : WIMG_ROWS, K, cin, cout, 0, (size_t)total / (b3 ? 2 : 1) * sizeof(uint4),
                           stream, &wi, &build));
  uint4 *img = (uint4 *)wi.ptr;
  if (build && b3)
    SCN_LAUNCH(k_rows_prepare_b3, (unsigned)ceil_div(total / 2, 256LL), 256, 0, stream, weight, img, K, cin, cout);
  else if (build)
    SCN_LAUNCH(k_rows_prepare, (unsigned)ceil_div(total / 2, 256LL), 256, 0, stream, weight, img, K, cin, cout);
  int rc;
  // With 32, 64 or 128 input planes the chunk count (and with it the row strides) is a constant of the kernel:
  // 4-6 % faster (6.94 -> 6.53 ms per U-Net pass over 8 rooms).  SCN_ROWS_NCH=0 keeps the run-time form.
  const bool fixed = (nch <= 2 || nch == 4) && !(getenv("SCN_ROWS_NCH") && atoi(getenv("SCN_ROWS_NCH")) == 0);
#define SCN_ROWS_CALL_N(NT, MODE, N) \
  launch_rows<NT, MODE, N>(in, cin, n_in, out, cout, n_out, img, bias, bn_scale, bn_shift, leak, table, K, nch, flags, stream)
#define SCN_ROWS_CALL(NT, MODE)                           \
  (!fixed ? SCN_ROWS_CALL_N(NT, MODE, 0)                  \
          : nch == 1 ? SCN_ROWS_CALL_N(NT, MODE, 1)       \
                     : nch == 2 ? SCN_ROWS_CALL_N(NT, MODE, 2) : SCN_ROWS_CALL_N(NT, MODE, 4))
  if (precision == SCN_PRECISION_BF16)
    rc = cout == 32 ? SCN_ROWS_CALL(4, TC_BF16) : SCN_ROWS_CALL(8, TC_BF16);
  else if (precision == SCN_PRECISION_TF32)
    rc = cout == 32 ? SCN_ROWS_CALL(4, TC_TF32) : SCN_ROWS_CALL(8, TC_TF32);
  else if (b3)
    rc = cout == 32 ? SCN_ROWS_CALL(4, TC_BF16X3) : SCN_ROWS_CALL(8, TC_BF16X3);
  else
    rc = cout == 32 ? SCN_ROWS_CALL(4, TC_TF32X3) : SCN_ROWS_CALL(8, TC_TF32X3);
#undef SCN_ROWS_CALL
#undef SCN_ROWS_CALL_N
  const int rf = weight_image_put(wi, stream);
  return rc != SCN_OK ? rc : rf;
}

}  // namespace scn
