// fp32 sparse convolution, output stationary.
//
// The reference walks the filter offsets on the host and, for each, gathers the input rows of
// that offset's rules, multiplies by W[k] and adds the product into the output rows with a
// read-modify-write (CPU/Convolution.cpp:137-148, CUDA/Convolution.cu:57-233,618-642): every
// output row crosses memory once per offset.  Here a CTA owns 128 output rows for the whole
// filter: for each offset it compacts the rows of its tile that have a rule (warp ballots over
// one coalesced read of the dense rulebook), gathers those input rows into shared memory,
// multiplies by W[k] with register micro-tiles and folds the partial products into a tile
// accumulator in shared memory.  Output rows are written exactly once, and nothing is spent
// on offsets for which a tile has no neighbour.  Arithmetic is fp32 FMA throughout.
//
// The same kernel serves SubmanifoldConvolution, Convolution (table nbr) and Deconvolution
// (table tnbr): the table maps (offset, output row) to an input row or -1.
#include <stdlib.h>

#include <algorithm>

#include "metadata.cuh"

namespace scn {

// conv_pipe.cu: the software-pipelined variant for 16-byte aligned rows and <= 32 filter offsets.
bool conv_pipe_supported(const float *in, const float *out, const float *weight, const float *bias, int K, int cin,
                         int cout);
int conv_forward_pipe(const float *in, long long n_in, float *out, long long n_out, const float *weight,
                      const float *bias, const int *table, int K, int cin, int cout, int groups, int three_pass_mma,
                      int *flags, cudaStream_t stream);

constexpr int kTileRows = 128;  // output rows per CTA
constexpr int kChunk = 32;      // input planes staged per step
constexpr int kThreads = 256;
constexpr int kAStride = kTileRows + 4;  // transposed A tile row stride (floats), keeps float4 alignment

template <int BN>
struct SimtSmem {
  float acc[kTileRows][BN];     // tile accumulator
  float a_t[kChunk][kAStride];  // gathered input rows, transposed: [plane][pair]
  float w[kChunk][BN];          // W[k][c0 .. c0+32][n0 .. n0+BN]
  int pair_in[kTileRows];       // compacted rules of the current offset: input row
  int pair_out[kTileRows];      //                                       local output row
  int warp_count[kThreads / 32];
  int n_pairs;
};

template <int BN>
__global__ void __launch_bounds__(kThreads)
k_conv_simt(const float *__restrict__ in, int ld_in, long long n_in, float *__restrict__ out,
            int ld_out, long long n_out, const float *__restrict__ weight, long long w_offset_stride,
            long long w_group_stride, const float *__restrict__ bias, const int *__restrict__ nbr,
            int K, int cin, int cout, int vec_in, int vec_w, int *flags) {
  constexpr int PM = BN / 8;                // pairs per thread
  constexpr int TXN = BN / 4;               // threads across the output planes
  extern __shared__ __align__(16) unsigned char smem_raw[];
  SimtSmem<BN> &S = *reinterpret_cast<SimtSmem<BN> *>(smem_raw);

  const int tid = threadIdx.x;
  const int tx = tid % TXN, ty = tid / TXN;
  const long long row0 = (long long)blockIdx.x * kTileRows;
  const int n0 = blockIdx.y * BN;
  const int g = blockIdx.z;
  in += (long long)g * cin;
  out += (long long)g * cout;
  weight += (long long)g * w_group_stride;
  if (bias) bias += (long long)g * cout;

  for (int i = tid; i < kTileRows * BN; i += kThreads) (&S.acc[0][0])[i] = 0.f;
  __syncthreads();

  for (int k = 0; k < K; ++k) {
    // ---- compact the rules of offset k that end in this tile -----------------------------
    int idx = -1;
    if (tid < kTileRows) {
      long long r = row0 + tid;
      if (r < n_out) idx = nbr[(long long)k * n_out + r];
      if (idx >= n_in) {
        atomicOr(flags, FLAG_BAD_ROW);
        idx = -1;
      }
    }
    unsigned hit = __ballot_sync(0xffffffffu, idx >= 0);
    if ((tid & 31) == 0) S.warp_count[tid >> 5] = __popc(hit);
    __syncthreads();
    if (idx >= 0) {
      int base = 0;
      for (int w = 0; w < (tid >> 5); ++w) base += S.warp_count[w];
      int p = base + __popc(hit & ((1u << (tid & 31)) - 1));
      S.pair_in[p] = idx;
      S.pair_out[p] = tid;
    }
    if (tid == 0) S.n_pairs = S.warp_count[0] + S.warp_count[1] + S.warp_count[2] + S.warp_count[3];
    __syncthreads();
    const int P = S.n_pairs;
    if (P == 0) continue;
    const int P_pad = (P + PM - 1) / PM * PM;
    const float *wk = weight + (long long)k * w_offset_stride;

    float acc[PM][4];
#pragma unroll
    for (int j = 0; j < PM; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;

    for (int c0 = 0; c0 < cin; c0 += kChunk) {
      // ---- gather: 8 threads x float4 per row, 32 rows per pass ---------------------------
      {
        const int q = tid & 7;
        const int c = c0 + q * 4;
        for (int p = tid >> 3; p < P_pad; p += kThreads / 8) {
          float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
          if (p < P) {
            const float *src = in + (long long)S.pair_in[p] * ld_in + c;
            if (vec_in && c + 3 < cin) {
              v = __ldg(reinterpret_cast<const float4 *>(src));
            } else {
              if (c + 0 < cin) v.x = __ldg(src + 0);
              if (c + 1 < cin) v.y = __ldg(src + 1);
              if (c + 2 < cin) v.z = __ldg(src + 2);
              if (c + 3 < cin) v.w = __ldg(src + 3);
            }
          }
          S.a_t[q * 4 + 0][p] = v.x;
          S.a_t[q * 4 + 1][p] = v.y;
          S.a_t[q * 4 + 2][p] = v.z;
          S.a_t[q * 4 + 3][p] = v.w;
        }
      }
      // ---- W[k] slab ------------------------------------------------------------------------
      for (int i = tid; i < kChunk * TXN; i += kThreads) {
        int r = i / TXN, cc = (i % TXN) * 4;
        int c = c0 + r, n = n0 + cc;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c < cin) {
          const float *src = wk + (long long)c * cout + n;
          if (vec_w && n + 3 < cout) {
            v = __ldg(reinterpret_cast<const float4 *>(src));
          } else {
            if (n + 0 < cout) v.x = __ldg(src + 0);
            if (n + 1 < cout) v.y = __ldg(src + 1);
            if (n + 2 < cout) v.z = __ldg(src + 2);
            if (n + 3 < cout) v.w = __ldg(src + 3);
          }
        }
        *reinterpret_cast<float4 *>(&S.w[r][cc]) = v;
      }
      __syncthreads();
      // ---- micro-tile product ---------------------------------------------------------------
      if (ty * PM < P) {
        const int kmax = min(kChunk, cin - c0);
#pragma unroll 4
        for (int kk = 0; kk < kmax; ++kk) {
          float a[PM];
          if (PM == 2) {
            float2 t = *reinterpret_cast<const float2 *>(&S.a_t[kk][ty * PM]);
            a[0] = t.x;
            a[1] = t.y;
          } else {
#pragma unroll
            for (int j = 0; j < PM; j += 4) {
              float4 t = *reinterpret_cast<const float4 *>(&S.a_t[kk][ty * PM + j]);
              a[j] = t.x;
              a[j + 1] = t.y;
              a[j + 2] = t.z;
              a[j + 3] = t.w;
            }
          }
          float4 w4 = *reinterpret_cast<const float4 *>(&S.w[kk][tx * 4]);
#pragma unroll
          for (int j = 0; j < PM; ++j) {
            acc[j][0] = fmaf(a[j], w4.x, acc[j][0]);
            acc[j][1] = fmaf(a[j], w4.y, acc[j][1]);
            acc[j][2] = fmaf(a[j], w4.z, acc[j][2]);
            acc[j][3] = fmaf(a[j], w4.w, acc[j][3]);
          }
        }
      }
      __syncthreads();
    }
    // ---- fold into the tile accumulator: one rule per (offset, output row), so no two
    // threads touch the same accumulator row within an offset -------------------------------
#pragma unroll
    for (int j = 0; j < PM; ++j) {
      int p = ty * PM + j;
      if (p < P) {
        float4 *dst = reinterpret_cast<float4 *>(&S.acc[S.pair_out[p]][tx * 4]);
        float4 t = *dst;
        t.x += acc[j][0];
        t.y += acc[j][1];
        t.z += acc[j][2];
        t.w += acc[j][3];
        *dst = t;
      }
    }
    __syncthreads();
  }

  // ---- write the tile once -------------------------------------------------------------------
  for (int i = tid; i < kTileRows * TXN; i += kThreads) {
    int r = i / TXN, cc = (i % TXN) * 4;
    long long row = row0 + r;
    if (row >= n_out) continue;
    float4 v = *reinterpret_cast<const float4 *>(&S.acc[r][cc]);
    float vv[4] = {v.x, v.y, v.z, v.w};
    float *dst = out + row * ld_out + n0 + cc;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      int n = n0 + cc + e;
      if (n < cout) dst[e] = vv[e] + (bias ? bias[n] : 0.f);
    }
  }
}

template <int BN>
static int launch_simt(const float *in, int ld_in, long long n_in, float *out, int ld_out, long long n_out,
                       const float *weight, const float *bias, const int *table, int K, int cin, int cout,
                       int groups, int *flags, cudaStream_t stream) {
  static bool configured[64] = {false};
  int dev = 0;
  SCN_CUDA_CHECK(cudaGetDevice(&dev));
  size_t smem = sizeof(SimtSmem<BN>);
  if (dev < 64 && !configured[dev]) {
    SCN_CUDA_CHECK(cudaFuncSetAttribute(k_conv_simt<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured[dev] = true;
  }
  int vec_in = (ld_in % 4 == 0) && (cin % 4 == 0) && ((uintptr_t)in % 16 == 0);
  int vec_w = (cout % 4 == 0) && ((uintptr_t)weight % 16 == 0) && (((long long)cin * cout) % 4 == 0);
  dim3 grid((unsigned)ceil_div(n_out, kTileRows), (unsigned)ceil_div(cout, BN), (unsigned)groups);
  SCN_LAUNCH(k_conv_simt<BN>, grid, kThreads, smem, stream, in, ld_in, n_in, out, ld_out, n_out, weight, (long long)groups * cin * cout, (long long)cin * cout, bias, table, K, cin, cout, vec_in, vec_w, flags);
  SCN_CUDA_CHECK(cudaGetLastError());
  return SCN_OK;
}

// ---------------------------------------------------------------------------------------------
// Thin layers (Cin <= 3, e.g. the first layer of a network: 1 or 3 input planes).  A tile of
// gathered rows would be almost empty, so there is no tile: one thread owns one output row and
// 32 output planes in registers.  A warp reads its 32 rows' rulebook entries coalesced (one
// 128-byte load per filter offset), then walks the offsets in lockstep: a thread whose row has a
// rule loads the Cin input values and adds x_c * W[k][c][:] with W read from shared memory at a
// warp-uniform address (broadcast).
// ---------------------------------------------------------------------------------------------
constexpr int kThinMaxK = 32;
constexpr int kThinPlanes = 32;

__global__ void __launch_bounds__(128)
k_conv_thin(const float *__restrict__ in, int ld_in, long long n_in, float *__restrict__ out, int ld_out,
            long long n_out, const float *__restrict__ weight, const float *__restrict__ bias,
            const int *__restrict__ nbr, int K, int cin, int cout, int *flags) {
  extern __shared__ __align__(16) float w_s[];  // [K][cin][32]: planes n0 .. n0+31 of this CTA, zero padded
  const int n0 = blockIdx.y * kThinPlanes;
  for (int i = threadIdx.x; i < K * cin * kThinPlanes; i += blockDim.x) {
    const int n = n0 + i % kThinPlanes, kc = i / kThinPlanes;
    w_s[i] = n < cout ? __ldg(weight + (long long)kc * cout + n) : 0.f;
  }
  __syncthreads();
  const long long row = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const bool row_ok = row < n_out;
  int v[kThinMaxK];
#pragma unroll
  for (int k = 0; k < kThinMaxK; ++k) v[k] = (k < K && row_ok) ? __ldg(nbr + (long long)k * n_out + row) : -1;
  float acc[kThinPlanes];
#pragma unroll
  for (int n = 0; n < kThinPlanes; ++n) acc[n] = (bias && n0 + n < cout) ? __ldg(bias + n0 + n) : 0.f;
#pragma unroll
  for (int k = 0; k < kThinMaxK; ++k) {
    if (k >= K) break;
    int idx = v[k];
    if (idx >= n_in) {
      atomicOr(flags, FLAG_BAD_ROW);
      idx = -1;
    }
    if (idx < 0) continue;
    const float *src = in + (long long)idx * ld_in;
    for (int c = 0; c < cin; ++c) {
      const float x = __ldg(src + c);
      const float4 *w4 = reinterpret_cast<const float4 *>(w_s + (k * cin + c) * kThinPlanes);
#pragma unroll
      for (int q = 0; q < kThinPlanes / 4; ++q) {
        const float4 w = w4[q];
        acc[4 * q + 0] = fmaf(x, w.x, acc[4 * q + 0]);
        acc[4 * q + 1] = fmaf(x, w.y, acc[4 * q + 1]);
        acc[4 * q + 2] = fmaf(x, w.z, acc[4 * q + 2]);
        acc[4 * q + 3] = fmaf(x, w.w, acc[4 * q + 3]);
      }
    }
  }
  if (!row_ok) return;
  float *dst = out + row * ld_out + n0;
#pragma unroll
  for (int n = 0; n < kThinPlanes; ++n)
    if (n0 + n < cout) dst[n] = acc[n];
}

static bool conv_thin_supported(int K, int cin, int groups) { return cin <= 3 && K <= kThinMaxK && groups == 1; }

static int conv_forward_thin(const float *in, long long n_in, float *out, long long n_out, const float *weight,
                             const float *bias, const int *table, int K, int cin, int cout, int *flags,
                             cudaStream_t stream) {
  const size_t smem = (size_t)K * cin * kThinPlanes * sizeof(float);  // <= 16 KB
  dim3 grid((unsigned)ceil_div(n_out, 128), (unsigned)ceil_div(cout, kThinPlanes));
  SCN_LAUNCH(k_conv_thin, grid, 128, smem, stream, in, cin, n_in, out, cout, n_out, weight, bias, table, K, cin, cout, flags);
  SCN_CUDA_CHECK(cudaGetLastError());
  return SCN_OK;
}

// out [n_out, groups*cout] = bias + sum_k in[table[k][.]] @ W[k]; cin / cout are per group.
int conv_forward_simt(const float *in, long long n_in, float *out, long long n_out, const float *weight,
                      const float *bias, const int *table, int K, int cin, int cout, int groups,
                      int *flags, cudaStream_t stream) {
  if (n_out == 0) return SCN_OK;
  const bool block_kernel_only = getenv("SCN_SIMT_BLOCK") && atoi(getenv("SCN_SIMT_BLOCK")) != 0;
  if (!block_kernel_only && conv_thin_supported(K, cin, groups))
    return conv_forward_thin(in, n_in, out, n_out, weight, bias, table, K, cin, cout, flags, stream);
  if (!block_kernel_only && conv_pipe_supported(in, out, weight, bias, K, cin, cout))
    return conv_forward_pipe(in, n_in, out, n_out, weight, bias, table, K, cin, cout, groups, 0, flags, stream);
  int ld_in = cin * groups, ld_out = cout * groups;
  if (cout <= 16)
    return launch_simt<16>(in, ld_in, n_in, out, ld_out, n_out, weight, bias, table, K, cin, cout, groups, flags, stream);
  if (cout <= 32)
    return launch_simt<32>(in, ld_in, n_in, out, ld_out, n_out, weight, bias, table, K, cin, cout, groups, flags, stream);
  return launch_simt<64>(in, ld_in, n_in, out, ld_out, n_out, weight, bias, table, K, cin, cout, groups, flags, stream);
}

}  // namespace scn
