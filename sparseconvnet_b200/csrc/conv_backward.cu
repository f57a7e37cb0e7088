// Backward pass of the three convolution operators (the reference: CPU/Convolution.cpp:80-115,
// 152-190, CPU/Deconvolution.cpp, CUDA/Convolution.cu dConvolution_KMxKN_backward_dW*), fp32.
//
//   d_input   the same output-stationary kernels as the forward pass, run on the opposite table
//             of the dense rulebook with the weights transposed per offset:
//                 d_in[i] = sum_k d_out[t[k][i]] * W[k]^T
//             (t = tnbr for SubmanifoldConvolution / Convolution, nbr for Deconvolution);
//   d_weight  d_W[k] = sum over the rules (i, o) of offset k of in[i]^T d_out[o]: the rules are cut
//             into chunks of rulebook entries, every CTA reduces one chunk of one offset into a
//             32 x 32 tile, and the chunks' partial tiles are added in a fixed order, so the
//             result is bit-reproducible (no floating-point atomics);
//   d_bias    column sums of d_out, the same two steps.
#include <algorithm>

#include <stdlib.h>

#include <atomic>

#include "metadata.cuh"

namespace scn {

extern std::atomic<int> g_backward_precision;
int conv_forward_dispatch(const float *in, long long rows_in, float *out, long long rows_out, const float *weight,
                          const float *bias, const int *table, int K, int cin, int cout, int groups, int precision,
                          int *flags, cudaStream_t stream, const float *bn_scale = nullptr,
                          const float *bn_shift = nullptr, float leak = 1.f, const float *pre_scale = nullptr,
                          const float *pre_shift = nullptr, float pre_leak = 1.f, const float *in_b = nullptr,
                          int planes_a = 0);
int conv_forward_simt(const float *in, long long n_in, float *out, long long n_out, const float *weight,
                      const float *bias, const int *table, int K, int cin, int cout, int groups, int *flags,
                      cudaStream_t stream);

// W [K][groups][cin][cout] -> [K][groups][cout][cin]
__global__ void k_transpose_weight(const float *__restrict__ w, float *__restrict__ wt, long long n_mats, int cin,
                                   int cout) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long per = (long long)cin * cout;
  if (idx >= n_mats * per) return;
  const long long m = idx / per;
  const int c = (int)((idx % per) / cout), n = (int)(idx % cout);
  wt[m * per + (long long)n * cin + c] = w[idx];
}

// partial[chunk][k][g][c][n] = sum over the chunk's rulebook entries j of offset k of
//   in[in_row(j)][g*cin + c] * d_out[out_row(j)][g*cout + n]
// where (in_row, out_row) = (nbr[k][j], j), or (j, nbr[k][j]) when the operator runs the rulebook
// backwards (Deconvolution).  grid = (chunks, K, groups * c-tiles * n-tiles), 256 threads,
// 32 x 32 tile, 2 x 2 outputs per thread.
__global__ void __launch_bounds__(256)
k_conv_dweight(const float *__restrict__ in, int ld_in, long long n_in_rows, const float *__restrict__ dout,
               int ld_out, long long n_out_rows, const int *__restrict__ nbr, long long n_entries, int swap,
               int cin, int cout, int groups, long long chunk_rows, float *__restrict__ partial, int *flags) {
  __shared__ float A[32][33], B[32][33];
  const int tid = threadIdx.x;
  const int k = blockIdx.y;
  const int tiles_c = (cin + 31) / 32, tiles_n = (cout + 31) / 32;
  int z = blockIdx.z;
  const int tn = z % tiles_n;
  z /= tiles_n;
  const int tc = z % tiles_c;
  const int g = z / tiles_c;
  const int c0 = tc * 32, n0 = tn * 32;
  const long long j0 = (long long)blockIdx.x * chunk_rows;
  const long long j1 = min(n_entries, j0 + chunk_rows);
  const int lr = tid >> 3, lq = (tid & 7) * 4;  // loader: row of the 32-entry slab, first of 4 columns
  const int ty = tid >> 4, tx = tid & 15;       // 2 x 2 outputs at (2 ty, 2 tx)
  float acc[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
  for (long long jb = j0; jb < j1; jb += 32) {
    const long long j = jb + lr;
    long long ri = -1, ro = -1;
    if (j < j1) {
      const int a = nbr[(long long)k * n_entries + j];
      if (a >= 0) {
        ri = swap ? j : a;
        ro = swap ? a : j;
        if (ri >= n_in_rows || ro >= n_out_rows) {
          atomicOr(flags, FLAG_BAD_ROW);
          ri = ro = -1;
        }
      }
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int c = c0 + lq + e, n = n0 + lq + e;
      A[lr][lq + e] = (ri >= 0 && c < cin) ? in[ri * ld_in + g * cin + c] : 0.f;
      B[lr][lq + e] = (ro >= 0 && n < cout) ? dout[ro * ld_out + g * cout + n] : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int r = 0; r < 32; ++r) {
      const float a0 = A[r][2 * ty], a1 = A[r][2 * ty + 1], b0 = B[r][2 * tx], b1 = B[r][2 * tx + 1];
      acc[0][0] = fmaf(a0, b0, acc[0][0]);
      acc[0][1] = fmaf(a0, b1, acc[0][1]);
      acc[1][0] = fmaf(a1, b0, acc[1][0]);
      acc[1][1] = fmaf(a1, b1, acc[1][1]);
    }
    __syncthreads();
  }
  float *dst = partial + (((long long)blockIdx.x * gridDim.y + k) * groups + g) * cin * cout;
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int jn = 0; jn < 2; ++jn) {
      const int c = c0 + 2 * ty + i, n = n0 + 2 * tx + jn;
      if (c < cin && n < cout) dst[(long long)c * cout + n] = acc[i][jn];
    }
}

// The same partial sums on the warp-level tensor path, for groups = 1 and plane counts that are
// multiples of 32: grid = (chunks, K, c-tiles * n-tiles), four warps.  Each warp takes a contiguous
// quarter of the chunk's rulebook entries, keeps only the entries that hold a rule (a third of them
// on surface data: the FMA kernel above multiplies the empty ones as zeros), and accumulates the
// 32 x 32 tile  in^T [32 x 8 rules] x d_out [8 rules x 32]  per block of eight rules with
// mma.sync.m16n8k8 on the hi/lo split of both operands (hi x hi + hi x lo + lo x hi, fp32
// accumulate: fp32-class accuracy).  The four warps' tiles are added in warp order, so the result
// does not depend on timing.
__device__ __forceinline__ void dw_mma(float (&d)[4], const unsigned (&a)[4], const unsigned (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ void dw_split(float x, unsigned &hi, unsigned &lo) {
  hi = __float_as_uint(x) & 0xFFFFE000u;
  lo = __float_as_uint(x - __uint_as_float(hi));
}

__global__ void __launch_bounds__(128)
k_conv_dweight_mma(const float *__restrict__ in, int ld_in, long long n_in_rows, const float *__restrict__ dout,
                   int ld_out, long long n_out_rows, const int *__restrict__ nbr, long long n_entries, int swap,
                   int cin, int cout, long long chunk_rows, float *__restrict__ partial, int *flags) {
  constexpr unsigned kFull = 0xffffffffu;
  __shared__ int q_in[4][64], q_out[4][64];  // per warp: rules waiting for a block of eight
  __shared__ float tile[4][32][33];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int k = blockIdx.y;
  const int tiles_n = cout / 32;
  const int c0 = (blockIdx.z / tiles_n) * 32, n0 = (blockIdx.z % tiles_n) * 32;
  const long long j0 = (long long)blockIdx.x * chunk_rows;
  const long long j1 = min(n_entries, j0 + chunk_rows);
  const long long per_warp = ((j1 - j0 + 3) / 4 + 31) / 32 * 32;
  const long long w0 = min(j1, j0 + warp * per_warp), w1 = min(j1, w0 + per_warp);
  const int *col = nbr + (long long)k * n_entries;

  float d[2][4][4];
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) d[mt][nt][0] = d[mt][nt][1] = d[mt][nt][2] = d[mt][nt][3] = 0.f;

  // one block of eight rules starting at queue position `head`; `count` (< 8 only at the end) are real
  auto block = [&](int head, int count) {
    const int p0 = (head + t) & 63, p1 = (head + t + 4) & 63;
    const bool ok0 = t < count, ok1 = t + 4 < count;
    const long long ri0 = ok0 ? q_in[warp][p0] : 0, ri1 = ok1 ? q_in[warp][p1] : 0;
    const long long ro0 = ok0 ? q_out[warp][p0] : 0, ro1 = ok1 ? q_out[warp][p1] : 0;
    const float *a0p = in + ri0 * ld_in + c0 + g, *a1p = in + ri1 * ld_in + c0 + g;
    const float *b0p = dout + ro0 * ld_out + n0 + g, *b1p = dout + ro1 * ld_out + n0 + g;
    float av[2][4], bv[4][2];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt) {  // A[m = plane][k = rule]: a0 (g, t), a1 (g + 8, t), a2 (g, t + 4), a3 (g + 8, t + 4)
      av[mt][0] = ok0 ? __ldg(a0p + mt * 16) : 0.f;
      av[mt][1] = ok0 ? __ldg(a0p + mt * 16 + 8) : 0.f;
      av[mt][2] = ok1 ? __ldg(a1p + mt * 16) : 0.f;
      av[mt][3] = ok1 ? __ldg(a1p + mt * 16 + 8) : 0.f;
    }
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {  // B[k = rule][n = plane]: b0 (t, g), b1 (t + 4, g)
      bv[nt][0] = ok0 ? __ldg(b0p + nt * 8) : 0.f;
      bv[nt][1] = ok1 ? __ldg(b1p + nt * 8) : 0.f;
    }
    unsigned ah[2][4], al[2][4], bh[4][2], bl[4][2];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int e = 0; e < 4; ++e) dw_split(av[mt][e], ah[mt][e], al[mt][e]);
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      dw_split(bv[nt][0], bh[nt][0], bl[nt][0]);
      dw_split(bv[nt][1], bh[nt][1], bl[nt][1]);
    }
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) dw_mma(d[mt][nt], al[mt], bh[nt]);
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) dw_mma(d[mt][nt], ah[mt], bl[nt]);
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) dw_mma(d[mt][nt], ah[mt], bh[nt]);
  };

  int head = 0, tail = 0;  // queue positions (not wrapped)
  for (long long jb = w0; jb < w1; jb += 32) {
    const long long j = jb + lane;
    int ri = -1, ro = -1;
    if (j < w1) {
      const int a = __ldg(col + j);
      if (a >= 0) {
        ri = swap ? (int)j : a;
        ro = swap ? a : (int)j;
        if (ri >= n_in_rows || ro >= n_out_rows) {
          atomicOr(flags, FLAG_BAD_ROW);
          ri = ro = -1;
        }
      }
    }
    const unsigned m = __ballot_sync(kFull, ri >= 0);
    if (ri >= 0) {
      const int p = (tail + __popc(m & ((1u << lane) - 1u))) & 63;
      q_in[warp][p] = ri;
      q_out[warp][p] = ro;
    }
    tail += __popc(m);
    __syncwarp();
    while (tail - head >= 8) {
      block(head, 8);
      head += 8;
    }
    __syncwarp();  // the blocks' reads of the queue come before the next group's writes
  }
  if (tail > head) block(head, tail - head);

  // ---- the four warps' tiles, added in warp order ------------------------------------------------
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {  // d0 (g, 2t), d1 (g, 2t + 1), d2 (g + 8, 2t), d3 (g + 8, 2t + 1)
      tile[warp][mt * 16 + g][nt * 8 + 2 * t] = d[mt][nt][0];
      tile[warp][mt * 16 + g][nt * 8 + 2 * t + 1] = d[mt][nt][1];
      tile[warp][mt * 16 + g + 8][nt * 8 + 2 * t] = d[mt][nt][2];
      tile[warp][mt * 16 + g + 8][nt * 8 + 2 * t + 1] = d[mt][nt][3];
    }
  __syncthreads();
  float *dst = partial + ((long long)blockIdx.x * gridDim.y + k) * cin * cout;
  for (int i = threadIdx.x; i < 32 * 32; i += 128) {
    const int c = i >> 5, n = i & 31;
    dst[(long long)(c0 + c) * cout + n0 + n] = ((tile[0][c][n] + tile[1][c][n]) + tile[2][c][n]) + tile[3][c][n];
  }
}

// partial[chunk][p] = sum over the chunk's rows of x[row][p]; grid = (plane tiles of 32, chunks)
__global__ void __launch_bounds__(256)
k_column_sums(const float *__restrict__ x, long long n_rows, int planes, long long chunk_rows,
              float *__restrict__ partial) {
  __shared__ float sh[8][33];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int p = blockIdx.x * 32 + lane;
  const long long r0 = (long long)blockIdx.y * chunk_rows, r1 = min(n_rows, r0 + chunk_rows);
  float s = 0.f;
  if (p < planes)
    for (long long r = r0 + w; r < r1; r += 8) s += x[r * planes + p];
  sh[w][lane] = s;
  __syncthreads();
  if (w == 0 && p < planes) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += sh[i][lane];
    partial[(long long)blockIdx.y * planes + p] = t;
  }
}

// out[i] = sum over chunks, in order, of partial[chunk][i]
__global__ void k_sum_chunks(const float *__restrict__ partial, int chunks, long long n, float *__restrict__ out) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float acc = 0.f;
  for (int c = 0; c < chunks; ++c) acc += partial[(long long)c * n + i];
  out[i] = acc;
}

static int n_chunks(long long rows) { return (int)std::max<long long>(1, std::min<long long>(64, rows / 4096)); }

// Runs the backward pass for one operator call.  `transposed` as in the forward pass (Deconvolution).
static int run_conv_backward(scn_metadata *md, Rulebook &rb, bool transposed, const float *in, float *d_in,
                             const float *d_out, const float *weight, float *d_weight, float *d_bias,
                             int n_in_planes, int n_out_planes, int groups, cudaStream_t stream) {
  SCN_REQUIRE(groups >= 1 && n_in_planes >= 1 && n_out_planes >= 1 && n_in_planes % groups == 0 &&
                  n_out_planes % groups == 0,
              SCN_ERR_BAD_ARG, "planes %d -> %d not divisible into %d groups", n_in_planes, n_out_planes, groups);
  SCN_REQUIRE(weight && d_weight, SCN_ERR_BAD_ARG, "null weight or weight gradient");
  const int cin = n_in_planes / groups, cout = n_out_planes / groups, K = rb.n_offsets;
  const long long rows_in = transposed ? rb.n_out : rb.n_in;
  const long long rows_out = transposed ? rb.n_in : rb.n_out;
  const long long w_elems = (long long)K * groups * cin * cout;
  if (!md->flags_dev) {
    SCN_TRY(device_alloc((void **)&md->flags_dev, sizeof(int), stream));
    SCN_CUDA_CHECK(cudaMemsetAsync(md->flags_dev, 0, sizeof(int), stream));
  }
  if (rows_out == 0 || rows_in == 0) {  // no rule: gradients are zero
    SCN_CUDA_CHECK(cudaMemsetAsync(d_weight, 0, sizeof(float) * (size_t)w_elems, stream));
    if (d_bias) SCN_CUDA_CHECK(cudaMemsetAsync(d_bias, 0, sizeof(float) * (size_t)n_out_planes, stream));
    if (rows_in > 0 && d_in)
      SCN_CUDA_CHECK(cudaMemsetAsync(d_in, 0, sizeof(float) * (size_t)rows_in * n_in_planes, stream));
    return SCN_OK;
  }
  SCN_REQUIRE(in && d_out, SCN_ERR_BAD_ARG, "null features");

  // ---- d_bias -------------------------------------------------------------------------------------
  if (d_bias) {
    const int chunks = n_chunks(rows_out);
    const long long chunk_rows = ceil_div(rows_out, chunks);
    float *partial = nullptr;
    SCN_TRY(device_alloc((void **)&partial, sizeof(float) * (size_t)chunks * n_out_planes, stream));
    SCN_LAUNCH(k_column_sums, dim3((unsigned)ceil_div(n_out_planes, 32), (unsigned)chunks), 256, 0, stream, d_out, rows_out, n_out_planes, chunk_rows, partial);
    SCN_LAUNCH(k_sum_chunks, (unsigned)ceil_div(n_out_planes, 256), 256, 0, stream, partial, chunks, (long long)n_out_planes, d_bias);
    SCN_CUDA_CHECK(cudaGetLastError());
    SCN_TRY(device_free(partial, stream));
  }

  // ---- d_weight -----------------------------------------------------------------------------------
  {
    const long long n_entries = rb.n_out;  // nbr is [K][rb.n_out]
    const int chunks = n_chunks(n_entries);
    const long long chunk_rows = ceil_div(ceil_div(n_entries, chunks), 32) * 32;
    float *partial = nullptr;
    SCN_TRY(device_alloc((void **)&partial, sizeof(float) * (size_t)chunks * w_elems, stream));
    const int tiles = groups * (int)ceil_div(cin, 32) * (int)ceil_div(cout, 32);
    const bool fma_only = getenv("SCN_DWEIGHT_FMA") && atoi(getenv("SCN_DWEIGHT_FMA")) != 0;
    if (groups == 1 && cin % 32 == 0 && cout % 32 == 0 && !fma_only)
      SCN_LAUNCH(k_conv_dweight_mma, dim3((unsigned)chunks, (unsigned)K, (unsigned)tiles), 128, 0, stream, in, n_in_planes, rows_in, d_out, n_out_planes, rows_out, rb.nbr, n_entries, transposed ? 1 : 0, cin, cout, chunk_rows, partial, md->flags_dev);
    else
      SCN_LAUNCH(k_conv_dweight, dim3((unsigned)chunks, (unsigned)K, (unsigned)tiles), 256, 0, stream, in, n_in_planes, rows_in, d_out, n_out_planes, rows_out, rb.nbr, n_entries, transposed ? 1 : 0, cin, cout, groups, chunk_rows, partial, md->flags_dev);
    SCN_LAUNCH(k_sum_chunks, (unsigned)ceil_div(w_elems, 256), 256, 0, stream, partial, chunks, w_elems, d_weight);
    SCN_CUDA_CHECK(cudaGetLastError());
    SCN_TRY(device_free(partial, stream));
  }

  // ---- d_input ------------------------------------------------------------------------------------
  if (d_in) {
    float *wt = nullptr;
    SCN_TRY(device_alloc((void **)&wt, sizeof(float) * (size_t)w_elems, stream));
    SCN_LAUNCH(k_transpose_weight, (unsigned)ceil_div(w_elems, 256), 256, 0, stream, weight, wt, (long long)K * groups, cin, cout);
    const int *table = rb.nbr;  // Deconvolution: coarse row <- fine rows
    if (!transposed) {
      SCN_TRY(rulebook_transposed(rb, stream));
      table = rb.tnbr;
    }
    SCN_TRY(conv_forward_dispatch(d_out, rows_out, d_in, rows_in, wt, nullptr, table, K, cout, cin, groups,
                                  g_backward_precision.load(), md->flags_dev, stream));
    SCN_TRY(device_free(wt, stream));
  }
  return SCN_OK;
}

}  // namespace scn

using namespace scn;

extern "C" {

int scn_submanifold_convolution_backward(scn_metadata *md, const int64_t *spatial_size, const int64_t *filter_size,
                                         const float *in_features, float *d_in_features,
                                         const float *d_out_features, const float *weight, float *d_weight,
                                         float *d_bias, int n_in_planes, int n_out_planes, int groups,
                                         void *stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  SCN_REQUIRE(md && spatial_size && filter_size, SCN_ERR_BAD_ARG, "null argument");
  Rulebook *rb = nullptr;
  SCN_TRY(get_submanifold_rulebook(md, spatial_size, filter_size, stream, &rb));
  return run_conv_backward(md, *rb, false, in_features, d_in_features, d_out_features, weight, d_weight, d_bias,
                           n_in_planes, n_out_planes, groups, stream);
}

int scn_convolution_backward(scn_metadata *md, const int64_t *input_size, const int64_t *output_size,
                             const int64_t *filter_size, const int64_t *filter_stride, const float *in_features,
                             float *d_in_features, const float *d_out_features, const float *weight,
                             float *d_weight, float *d_bias, int n_in_planes, int n_out_planes, int groups,
                             void *stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  SCN_REQUIRE(md && input_size && output_size && filter_size && filter_stride, SCN_ERR_BAD_ARG, "null argument");
  Rulebook *rb = nullptr;
  SCN_TRY(get_strided_rulebook(md, input_size, output_size, filter_size, filter_stride, stream, &rb));
  return run_conv_backward(md, *rb, false, in_features, d_in_features, d_out_features, weight, d_weight, d_bias,
                           n_in_planes, n_out_planes, groups, stream);
}

int scn_deconvolution_backward(scn_metadata *md, const int64_t *input_size, const int64_t *output_size,
                               const int64_t *filter_size, const int64_t *filter_stride, const float *in_features,
                               float *d_in_features, const float *d_out_features, const float *weight,
                               float *d_weight, float *d_bias, int n_in_planes, int n_out_planes, int groups,
                               void *stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  SCN_REQUIRE(md && input_size && output_size && filter_size && filter_stride, SCN_ERR_BAD_ARG, "null argument");
  Rulebook *rb = nullptr;
  SCN_TRY(get_strided_rulebook(md, output_size, input_size, filter_size, filter_stride, stream, &rb));
  return run_conv_backward(md, *rb, true, in_features, d_in_features, d_out_features, weight, d_weight, d_bias,
                           n_in_planes, n_out_planes, groups, stream);
}
}
