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

#include <atomic>

#include "metadata.cuh"

namespace scn {

extern std::atomic<int> g_backward_precision;
int conv_forward_dispatch(const float *in, long long rows_in, float *out, long long rows_out, const float *weight,
                          const float *bias, const int *table, int K, int cin, int cout, int groups, int precision,
                          int *flags, cudaStream_t stream);
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
