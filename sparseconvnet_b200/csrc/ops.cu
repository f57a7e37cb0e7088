// Bandwidth-bound feature operators: input-layer duplicate handling, BatchNorm + leaky ReLU,
// rulebook-driven max pooling and sparse-to-dense.  Each is one pass over its rows.
#include <algorithm>

#include "metadata.cuh"

namespace scn {

// ------------------------------------------------------------------------------------------
// InputLayer feature pass (CPU/IOLayers.cpp:11-29): out[row] = sum_i mult * in[r_i], summed in
// ascending input-row order with separate multiply and add, as the reference's scalar loop
// does, so modes 1-3 are bit-exact and mode 4 differs only where 1/count is inexact.
// ------------------------------------------------------------------------------------------
__global__ void k_input_features(const float *__restrict__ in, float *__restrict__ out,
                                 const int *__restrict__ start, const int *__restrict__ rows,
                                 long long n_out, int C, int mode) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n_out * C) return;
  long long r = idx / C;
  int c = (int)(idx % C);
  int s = start[r], e = start[r + 1];
  float acc = 0.f;
  if (mode == 1) {
    acc = in[(long long)rows[s] * C + c];
  } else if (mode == 2) {
    acc = in[(long long)rows[e - 1] * C + c];
  } else {
    float mult = (mode == 4 && e > s) ? 1.0f / (float)(e - s) : 1.0f;
    for (int j = s; j < e; ++j) acc = __fadd_rn(acc, __fmul_rn(mult, in[(long long)rows[j] * C + c]));
  }
  out[idx] = acc;
}

// OutputLayer / BLOutputLayer (CPU/IOLayers.cpp:31-47,95-114,197-215): the feature row of a
// site goes back, unscaled, to the input points its rule names -- the first point of the site
// (mode 1), the last (mode 2) or all of them (modes 3, 4).  Points that no rule names (dropped
// duplicates, empty slots of a batch x length array) keep the zeros the output was cleared to.
__global__ void k_output_features(const float *__restrict__ in, float *__restrict__ out,
                                  const int *__restrict__ start, const int *__restrict__ rows,
                                  long long n_sites, int C, int mode, int scale_mean) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n_sites * C) return;
  long long r = idx / C;
  int c = (int)(idx % C);
  int s = start[r], e = start[r + 1];
  if (e <= s) return;
  // scale_mean: the backward pass of a mode-4 InputLayer hands every point 1/count of the site's row
  const float v = scale_mean ? __fmul_rn(1.0f / (float)(e - s), in[idx]) : in[idx];
  if (mode == 1) {
    out[(long long)rows[s] * C + c] = v;
  } else if (mode == 2) {
    out[(long long)rows[e - 1] * C + c] = v;
  } else {
    for (int j = s; j < e; ++j) out[(long long)rows[j] * C + c] = v;
  }
}

// ------------------------------------------------------------------------------------------
// BatchNorm + leaky ReLU (CPU/BatchNormalization.cpp:12-62)
// ------------------------------------------------------------------------------------------

// per-plane sum and sum of squares; grid.x tiles planes by 32, grid.y splits the rows
__global__ void __launch_bounds__(256)
k_bn_stats(const float *__restrict__ in, long long n_rows, int C, long long in_stride,
           double *__restrict__ sums /* [2][C] */) {
  __shared__ float sh_s[8][33], sh_q[8][33];
  int lane = threadIdx.x & 31, wy = threadIdx.x >> 5;
  int c = blockIdx.x * 32 + lane;
  float s = 0.f, q = 0.f;
  if (c < C)
    for (long long r = (long long)blockIdx.y * 8 + wy; r < n_rows; r += (long long)gridDim.y * 8) {
      float v = in[r * in_stride + c];
      s += v;
      q += v * v;
    }
  sh_s[wy][lane] = s;
  sh_q[wy][lane] = q;
  __syncthreads();
  if (wy == 0 && c < C) {
    double ds = 0, dq = 0;
    for (int j = 0; j < 8; ++j) {
      ds += sh_s[j][lane];
      dq += sh_q[j][lane];
    }
    atomicAdd(&sums[c], ds);
    atomicAdd(&sums[C + c], dq);
  }
}

// Turns either running statistics (eval) or batch sums (train) into saveMean / saveInvStd and
// updates the running statistics in training mode: momentum weighs the OLD value, the
// normalising variance is biased, the running variance unbiased (CPU/BatchNormalization.cpp:32-46).
__global__ void k_bn_finalize(int C, long long n_rows, const double *__restrict__ sums,
                              float *save_mean, float *save_invstd, float *running_mean,
                              float *running_var, float eps, float momentum, int train,
                              int count_follows_sums = 0) {
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  if (count_follows_sums) {  // the row count of all devices, summed along with the array
    n_rows = (long long)sums[2 * C];
    if (n_rows == 0) return;
  }
  if (train) {
    double mean = sums[c] / (double)n_rows;
    double ss = sums[C + c] - mean * mean * (double)n_rows;
    save_mean[c] = (float)mean;
    running_mean[c] = momentum * running_mean[c] + (1 - momentum) * (float)mean;
    running_var[c] = momentum * running_var[c] + (1 - momentum) * (float)(ss / (double)(n_rows - 1));
    save_invstd[c] = powf((float)(ss / (double)n_rows) + eps, -0.5f);
  } else {
    save_mean[c] = running_mean[c];
    save_invstd[c] = powf(running_var[c] + eps, -0.5f);
  }
}

// y = x * w + b, y *= (y > 0 ? 1 : leak); four planes per thread when the layout allows.
// With `running_var` (eval mode) the statistics are the running ones: every CTA derives mean and
// inverse deviation from them (the same expressions as k_bn_finalize), and the first one also
// stores them in save_mean / save_invstd as the reference does; no separate launch.
template <int VEC>
__global__ void __launch_bounds__(256)
k_bn_apply(const float *__restrict__ in, float *__restrict__ out, long long n_rows, int C,
           long long in_stride, long long out_stride, float *save_mean, float *save_invstd,
           const float *__restrict__ running_mean, const float *__restrict__ running_var, float eps,
           const float *__restrict__ weight, const float *__restrict__ bias, float leak) {
  extern __shared__ float sh_wb[];  // [2][C]
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float mean, invstd;
    if (running_var) {
      mean = running_mean[c];
      invstd = powf(running_var[c] + eps, -0.5f);
      if (blockIdx.x == 0) {
        save_mean[c] = mean;
        save_invstd[c] = invstd;
      }
    } else {
      mean = save_mean[c];
      invstd = save_invstd[c];
    }
    float w = invstd * (weight ? weight[c] : 1.f);
    sh_wb[c] = w;
    sh_wb[C + c] = __fadd_rn(__fmul_rn(-mean, w), bias ? bias[c] : 0.f);
  }
  __syncthreads();
  int cv = C / VEC;
  long long total = n_rows * cv;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    long long r = idx / cv;
    int c = (int)(idx % cv) * VEC;
    if (VEC == 4) {
      float4 x = *reinterpret_cast<const float4 *>(in + r * in_stride + c);
      float4 y;
      y.x = __fadd_rn(__fmul_rn(x.x, sh_wb[c + 0]), sh_wb[C + c + 0]);
      y.y = __fadd_rn(__fmul_rn(x.y, sh_wb[c + 1]), sh_wb[C + c + 1]);
      y.z = __fadd_rn(__fmul_rn(x.z, sh_wb[c + 2]), sh_wb[C + c + 2]);
      y.w = __fadd_rn(__fmul_rn(x.w, sh_wb[c + 3]), sh_wb[C + c + 3]);
      y.x *= (y.x > 0.f) ? 1.f : leak;
      y.y *= (y.y > 0.f) ? 1.f : leak;
      y.z *= (y.z > 0.f) ? 1.f : leak;
      y.w *= (y.w > 0.f) ? 1.f : leak;
      *reinterpret_cast<float4 *>(out + r * out_stride + c) = y;
    } else {
      float y = __fadd_rn(__fmul_rn(in[r * in_stride + c], sh_wb[c]), sh_wb[C + c]);
      out[r * out_stride + c] = y * ((y > 0.f) ? 1.f : leak);
    }
  }
}

// ------------------------------------------------------------------------------------------
// BatchNorm + leaky ReLU, backward (CPU/BatchNormalization.cpp:64-107).  With d = d_out * (out > 0
// ? 1 : leakiness):  d_bias = sum d,  dotp = sum (x - mean) d,  d_weight = dotp * invstd,
//   d_in = (d - d_bias / n - (x - mean) * dotp * invstd^2 / n) * invstd * weight.
// The reference applies this formula in eval mode too (with the running statistics in mean /
// invstd); so does this.  The two sums are accumulated in double, chunk by chunk, and the chunks
// are added in a fixed order.
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
k_bn_back_sums(const float *__restrict__ in, const float *__restrict__ out, const float *__restrict__ d_out,
               long long n_rows, int C, long long in_stride, long long out_stride,
               const float *__restrict__ mean, float leak, long long chunk_rows,
               double *__restrict__ partial /* [chunks][2][C] */) {
  __shared__ double sh_s[8][33], sh_q[8][33];
  const int lane = threadIdx.x & 31, wy = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;
  const long long r0 = (long long)blockIdx.y * chunk_rows, r1 = min(n_rows, r0 + chunk_rows);
  double s = 0.0, q = 0.0;
  if (c < C) {
    const float m = mean[c];
    long long r = r0 + wy;
    for (; r + 24 < r1; r += 32) {  // four rows in flight per thread
      float d[4], o[4], x[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        d[u] = d_out[(r + 8 * u) * out_stride + c];
        o[u] = out[(r + 8 * u) * out_stride + c];
        x[u] = in[(r + 8 * u) * in_stride + c];
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (!(o[u] > 0.f)) d[u] *= leak;
        s += d[u];
        q += (double)(x[u] - m) * d[u];
      }
    }
    for (; r < r1; r += 8) {
      float d = d_out[r * out_stride + c];
      if (!(out[r * out_stride + c] > 0.f)) d *= leak;
      s += d;
      q += (double)(in[r * in_stride + c] - m) * d;
    }
  }
  sh_s[wy][lane] = s;
  sh_q[wy][lane] = q;
  __syncthreads();
  if (wy == 0 && c < C) {
    double ts = 0.0, tq = 0.0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      ts += sh_s[i][lane];
      tq += sh_q[i][lane];
    }
    partial[((long long)blockIdx.y * 2 + 0) * C + c] = ts;
    partial[((long long)blockIdx.y * 2 + 1) * C + c] = tq;
  }
}

__global__ void k_bn_back_finalize(const double *__restrict__ partial, int chunks, int C, long long n_rows,
                                   const float *__restrict__ invstd, float *__restrict__ d_weight,
                                   float *__restrict__ d_bias, float *__restrict__ coef /* [2][C] */) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  double s = 0.0, q = 0.0;
  for (int i = 0; i < chunks; ++i) {
    s += partial[((long long)i * 2 + 0) * C + c];
    q += partial[((long long)i * 2 + 1) * C + c];
  }
  const float is = invstd[c];
  if (d_bias) d_bias[c] = (float)s;
  if (d_weight) d_weight[c] = (float)q * is;
  coef[c] = (float)(s / (double)n_rows);                      // gradMean
  coef[C + c] = (float)(q * (double)is * (double)is / (double)n_rows);  // k
}

// The two-phase form of the backward pass (rows spread over several devices): the chunk sums of one device
// added in their fixed order ...
__global__ void k_bn_back_reduce(const double *__restrict__ partial, int chunks, int C, double *__restrict__ sums) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  double s = 0.0, q = 0.0;
  for (int i = 0; i < chunks; ++i) {
    s += partial[((long long)i * 2 + 0) * C + c];
    q += partial[((long long)i * 2 + 1) * C + c];
  }
  sums[c] = s;
  sums[C + c] = q;
}

// ... and, once the caller has added the devices' sums, the coefficients of k_bn_back_apply from the totals and
// the parameter gradients from this device's own sums (the same expressions as k_bn_back_finalize).
__global__ void k_bn_back_coef(const double *__restrict__ local, const double *__restrict__ total, int C,
                               long long n_rows_total, const float *__restrict__ invstd,
                               float *__restrict__ d_weight, float *__restrict__ d_bias,
                               float *__restrict__ coef /* [2][C] */) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  if (n_rows_total < 0) n_rows_total = (long long)total[2 * C];  // summed along with the array
  if (n_rows_total == 0) n_rows_total = 1;                        // no rows anywhere: all sums are zero
  const float is = invstd[c];
  if (d_bias) d_bias[c] = (float)local[c];
  if (d_weight) d_weight[c] = (float)local[C + c] * is;
  coef[c] = (float)(total[c] / (double)n_rows_total);
  coef[C + c] = (float)(total[C + c] * (double)is * (double)is / (double)n_rows_total);
}

__global__ void __launch_bounds__(256)
k_bn_back_apply(const float *__restrict__ in, float *__restrict__ d_in, const float *__restrict__ out,
                const float *__restrict__ d_out, long long n_rows, int C, long long in_stride,
                long long out_stride, const float *__restrict__ mean, const float *__restrict__ invstd,
                const float *__restrict__ weight, const float *__restrict__ coef, float leak) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n_rows * C) return;
  const long long r = idx / C;
  const int c = (int)(idx % C);
  float d = d_out[r * out_stride + c];
  if (!(out[r * out_stride + c] > 0.f)) d *= leak;
  const float x = in[r * in_stride + c] - mean[c];
  d_in[r * in_stride + c] = (d - coef[c] - x * coef[C + c]) * invstd[c] * (weight ? weight[c] : 1.f);
}

// ------------------------------------------------------------------------------------------
// MaxPooling (CPU/MaxPooling.cpp:7-20,37-60): the reference zero-fills the output and then
// takes elementwise maxima over the rules, so the result is max(0, max of inputs).  Output
// stationary here: each output element is written once.
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
k_max_pool(const float *__restrict__ in, float *__restrict__ out, const int *__restrict__ nbr,
           long long n_out, long long n_in, int K, int C_out, int in_stride, int drop, int *flags) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n_out * C_out) return;
  long long o = idx / C_out;
  int c = (int)(idx % C_out);
  float m = 0.f;
  for (int k = 0; k < K; ++k) {
    int i = nbr[(long long)k * n_out + o];
    if (i < 0) continue;
    if (i >= n_in) {
      atomicOr(flags, FLAG_BAD_ROW);
      continue;
    }
    float v = in[(long long)i * in_stride + drop + c];
    if (m < v) m = v;
  }
  out[idx] = m;
}

// ------------------------------------------------------------------------------------------
// AveragePooling (CPU/AveragePooling.cpp:7-20,38-61): out[o] = sum over the rules of o, in
// ascending filter-offset order, of in[i] / filterVolume -- the divisor is the filter volume, not
// the number of rules, and every term is divided before it is added, as the reference does.
// UnPooling (CPU/UnPooling.cpp:7-19,35-59): the rulebook of (fine -> coarse) read backwards:
// out[fine] = sum over offsets of in[coarse]; `nbr` is then the transposed table [K][n fine].
// ------------------------------------------------------------------------------------------
template <bool AVERAGE>
__global__ void __launch_bounds__(256)
k_sum_pool(const float *__restrict__ in, float *__restrict__ out, const int *__restrict__ nbr,
           long long n_out, long long n_in, int K, int C_out, int in_stride, int drop, int *flags) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n_out * C_out) return;
  long long o = idx / C_out;
  int c = (int)(idx % C_out);
  const float fv = (float)K;
  float acc = 0.f;
  for (int k = 0; k < K; ++k) {
    int i = nbr[(long long)k * n_out + o];
    if (i < 0) continue;
    if (i >= n_in) {
      atomicOr(flags, FLAG_BAD_ROW);
      continue;
    }
    float v = in[(long long)i * in_stride + drop + c];
    acc = __fadd_rn(acc, AVERAGE ? __fdiv_rn(v, fv) : v);
  }
  out[idx] = acc;
}

// ------------------------------------------------------------------------------------------
// SparseToDense (CPU/SparseToDense.cpp:7-19,35-64): dense[b][c][offset(x)] = feat[row][c]
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
k_sparse_to_dense(KeyLayout L, const unsigned long long *__restrict__ row_keys,
                  const float *__restrict__ in, float *__restrict__ out, long long n_rows, int C,
                  long long volume) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n_rows * C) return;
  long long r = idx / C;
  int c = (int)(idx % C);
  unsigned long long key = row_keys[r];
  if (key == kEmptyKey) return;
  int x[kMaxDim], b;
  unpack_key(L, key, x, b);
  long long lin = 0;
  for (int d = 0; d < L.dim; ++d) lin = lin * L.size[d] + x[d];
  out[((long long)b * C + c) * volume + lin] = in[idx];
}

// ------------------------------------------------------------------------------------------
// Backward passes of the pooling operators, input stationary (each d_in element is written once,
// sums in ascending filter-offset order).  `table` maps (offset, d_in row) to the d_out row.
//   OP 0  MaxPooling (CPU/MaxPooling.cpp:22-35): d_out flows to every input equal to the pooled
//         maximum
//   OP 1  AveragePooling (CPU/AveragePooling.cpp:21-35): d_out / pool volume
//   OP 2  UnPooling (CPU/UnPooling.cpp:20-32): plain sum
// The first `drop` planes of d_in (features the forward pass ignored) are zero.
// ------------------------------------------------------------------------------------------
template <int OP>
__global__ void __launch_bounds__(256)
k_pool_backward(const float *__restrict__ in, float *__restrict__ d_in, const float *__restrict__ out,
                const float *__restrict__ d_out, const int *__restrict__ table, long long n_rows,
                long long n_other, int K, int C_in, int drop, int *flags) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n_rows * C_in) return;
  const long long i = idx / C_in;
  const int c = (int)(idx % C_in) - drop;
  if (c < 0) {
    d_in[idx] = 0.f;
    return;
  }
  const int C_out = C_in - drop;
  const float fv = (float)K;
  const float x = OP == 0 ? in[idx] : 0.f;
  float acc = 0.f;
  for (int k = 0; k < K; ++k) {
    const int o = table[(long long)k * n_rows + i];
    if (o < 0) continue;
    if (o >= n_other) {
      atomicOr(flags, FLAG_BAD_ROW);
      continue;
    }
    const float g = d_out[(long long)o * C_out + c];
    if (OP == 0) {
      if (out[(long long)o * C_out + c] == x) acc = __fadd_rn(acc, g);
    } else if (OP == 1) {
      acc = __fadd_rn(acc, __fdiv_rn(g, fv));
    } else {
      acc = __fadd_rn(acc, g);
    }
  }
  d_in[idx] = acc;
}

// SparseToDense backward (CPU/SparseToDense.cpp:20-33): d_in[row][c] = d_dense[b][c][offset(x)]
__global__ void __launch_bounds__(256)
k_dense_to_sparse_grad(KeyLayout L, const unsigned long long *__restrict__ row_keys,
                       const float *__restrict__ d_dense, float *__restrict__ d_in, long long n_rows, int C,
                       long long volume) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n_rows * C) return;
  long long r = idx / C;
  int c = (int)(idx % C);
  unsigned long long key = row_keys[r];
  if (key == kEmptyKey) {
    d_in[idx] = 0.f;
    return;
  }
  int x[kMaxDim], b;
  unpack_key(L, key, x, b);
  long long lin = 0;
  for (int d = 0; d < L.dim; ++d) lin = lin * L.size[d] + x[d];
  d_in[idx] = d_dense[((long long)b * C + c) * volume + lin];
}

// ------------------------------------------------------------------------------------------------
// Rows times a small matrix: out[r, :] = bias + in[r, :] * W, W [n_in][n_out] with n_out <= 32.
// NetworkInNetwork_updateOutput (CPU/NetworkInNetwork.cpp:7-23) and the per-voxel class head of the
// segmentation networks are this shape: millions of rows, a few dozen columns.  The operation is bound
// by reading the rows once and writing the scores once; a dense-library GEMM picks a tile shape made for
// wide outputs and takes several times that.  A warp takes 32 rows at a time: 32 planes of them are read
// with coalesced 16-byte loads (four rows per instruction) into a padded tile of shared memory, then every
// lane reads its own row from the tile and adds its products to the n_out sums it keeps in registers
// (fp32 FMA, plane order -- the order a scalar loop over n_in has); the weights (zero-padded to a multiple
// of four columns) sit in shared memory and are read as broadcasts.
constexpr int kAffineChunk = 32;                  // planes per pass through shared memory
constexpr int kAffineStride = kAffineChunk + 4;   // floats: the 32 lanes' 16-byte reads of their rows do not collide

template <int COUT4>
__global__ void __launch_bounds__(256)
k_rows_affine(const float *__restrict__ in, float *__restrict__ out, long long n_rows, int cin, int cout,
              const float *__restrict__ weight, const float *__restrict__ bias) {
  extern __shared__ float4 sh_w4[];  // [cin][COUT4], then one [32][kAffineStride] tile per warp
  float *sh_w = reinterpret_cast<float *>(sh_w4);
  constexpr int CP = COUT4 * 4;
  for (int i = threadIdx.x; i < cin * CP; i += blockDim.x) {
    const int k = i / CP, c = i % CP;
    sh_w[i] = c < cout ? weight[(size_t)k * cout + c] : 0.f;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float *tile = sh_w + (size_t)cin * CP + (size_t)warp * 32 * kAffineStride;
  const long long warps = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long row0 = ((long long)blockIdx.x * (blockDim.x >> 5) + warp) * 32; row0 < n_rows; row0 += warps * 32) {
    float acc[CP];
#pragma unroll
    for (int c = 0; c < CP; ++c) acc[c] = (bias && c < cout) ? bias[c] : 0.f;
    for (int p0 = 0; p0 < cin; p0 += kAffineChunk) {
      const int width = min(kAffineChunk, cin - p0);  // a multiple of four
      // coalesced: lane -> (row lane / 8 + 4 i, 16-byte piece lane % 8)
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int r = (lane >> 3) + 4 * i, piece = lane & 7;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (row0 + r < n_rows && piece * 4 < width)
          v = __ldcs(reinterpret_cast<const float4 *>(in + (row0 + r) * cin + p0 + piece * 4));
        *reinterpret_cast<float4 *>(tile + r * kAffineStride + piece * 4) = v;
      }
      __syncwarp();
      const float4 *mine = reinterpret_cast<const float4 *>(tile + lane * kAffineStride);
      for (int q = 0; q < width / 4; ++q) {
        const float4 x = mine[q];
        const float xs[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
          for (int c4 = 0; c4 < COUT4; ++c4) {
            const float4 w = sh_w4[(p0 + q * 4 + j) * COUT4 + c4];
            acc[c4 * 4 + 0] = fmaf(xs[j], w.x, acc[c4 * 4 + 0]);
            acc[c4 * 4 + 1] = fmaf(xs[j], w.y, acc[c4 * 4 + 1]);
            acc[c4 * 4 + 2] = fmaf(xs[j], w.z, acc[c4 * 4 + 2]);
            acc[c4 * 4 + 3] = fmaf(xs[j], w.w, acc[c4 * 4 + 3]);
          }
        }
      }
      __syncwarp();
    }
    const long long r = row0 + lane;
    if (r < n_rows) {
      float *o = out + r * cout;
      if (cout % 4 == 0) {
#pragma unroll
        for (int c4 = 0; c4 < COUT4; ++c4)
          if (c4 * 4 < cout)
            __stcs(reinterpret_cast<float4 *>(o + c4 * 4),
                   make_float4(acc[c4 * 4], acc[c4 * 4 + 1], acc[c4 * 4 + 2], acc[c4 * 4 + 3]));
      } else {
#pragma unroll
        for (int c = 0; c < CP; ++c)
          if (c < cout) o[c] = acc[c];
      }
    }
  }
}

}  // namespace scn

using namespace scn;

extern "C" {

int scn_input_layer_forward(scn_metadata *md, const float *in_features, int64_t n_in,
                            float *out_features, int64_t n_out, int n_planes, void *stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  SCN_REQUIRE(md && md->input_mode >= 0, SCN_ERR_BAD_ARG, "scn_md_input_layer has not been called");
  SCN_REQUIRE(n_in == md->input_n_rows && n_out == md->input_n_active, SCN_ERR_SIZE_MISMATCH,
              "input layer: got %lld -> %lld rows, metadata has %lld -> %lld", (long long)n_in,
              (long long)n_out, md->input_n_rows, md->input_n_active);
  SCN_REQUIRE(n_planes >= 1, SCN_ERR_BAD_ARG, "n_planes must be positive");
  if (n_out == 0) return SCN_OK;
  SCN_REQUIRE(in_features && out_features, SCN_ERR_BAD_ARG, "null features");
  SCN_TRY(md_touch(md, stream));
  if (md->input_mode == 0) {  // row i <-> input i (CPU/IOLayers.cpp:61-63)
    if (in_features != out_features)
      SCN_CUDA_CHECK(cudaMemcpyAsync(out_features, in_features, sizeof(float) * (size_t)n_in * n_planes,
                                     cudaMemcpyDeviceToDevice, stream));
    return SCN_OK;
  }
  long long total = (long long)n_out * n_planes;
  SCN_LAUNCH(k_input_features, (unsigned)ceil_div(total, 256), 256, 0, stream, in_features, out_features, md->input_csr_start, md->input_csr_rows, n_out, n_planes, md->input_mode);
  SCN_CUDA_CHECK(cudaGetLastError());
  return SCN_OK;
}

int scn_output_layer_forward(scn_metadata *md, const float *in_features, int64_t n_in, float *out_features,
                             int64_t n_out, int n_planes, void *stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  SCN_REQUIRE(md, SCN_ERR_BAD_ARG, "null metadata");
  SCN_REQUIRE(md->input_mode >= 0, SCN_ERR_NO_GRID, "no input layer has been run on this metadata");
  SCN_REQUIRE(n_planes >= 1, SCN_ERR_BAD_ARG, "n_planes %d", n_planes);
  SCN_REQUIRE(n_in == md->input_n_active, SCN_ERR_SIZE_MISMATCH, "input has %lld rows, the input layer made %lld",
              (long long)n_in, (long long)md->input_n_active);
  SCN_REQUIRE(n_out == md->input_n_rows, SCN_ERR_SIZE_MISMATCH, "output has %lld rows, the input layer read %lld",
              (long long)n_out, (long long)md->input_n_rows);
  if (n_out == 0) return SCN_OK;
  SCN_REQUIRE(out_features && (in_features || n_in == 0), SCN_ERR_BAD_ARG, "null features");
  SCN_TRY(md_touch(md, stream));
  const size_t bytes = sizeof(float) * (size_t)n_out * n_planes;
  if (md->input_mode == 0) {  // rows are the input points themselves
    SCN_CUDA_CHECK(cudaMemcpyAsync(out_features, in_features, bytes, cudaMemcpyDeviceToDevice, stream));
    return SCN_OK;
  }
  SCN_CUDA_CHECK(cudaMemsetAsync(out_features, 0, bytes, stream));
  if (n_in == 0) return SCN_OK;
  long long total = (long long)n_in * n_planes;
  SCN_LAUNCH(k_output_features, (unsigned)ceil_div(total, 256), 256, 0, stream, in_features, out_features, md->input_csr_start, md->input_csr_rows, n_in, n_planes, md->input_mode, 0);
  SCN_CUDA_CHECK(cudaGetLastError());
  return SCN_OK;
}

int scn_batchnorm_forward(const float *in_features, float *out_features, int64_t n_rows, int n_planes,
                          int64_t in_stride, int64_t out_stride, float *save_mean, float *save_invstd,
                          float *running_mean, float *running_var, const float *weight,
                          const float *bias, double eps, double momentum, int train, double leakiness,
                          void *stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  SCN_REQUIRE(n_planes >= 1 && n_planes <= 4096, SCN_ERR_UNSUPPORTED, "n_planes %d unsupported", n_planes);
  SCN_REQUIRE(save_mean && save_invstd && running_mean && running_var, SCN_ERR_BAD_ARG, "null statistics");
  SCN_REQUIRE(in_stride >= n_planes && out_stride >= n_planes, SCN_ERR_BAD_ARG, "row stride below n_planes");
  if (n_rows == 0) return SCN_OK;
  SCN_REQUIRE(in_features && out_features, SCN_ERR_BAD_ARG, "null features");
  double *sums = nullptr;
  if (train) {
    SCN_TRY(device_alloc((void **)&sums, sizeof(double) * 2 * n_planes, stream));
    SCN_CUDA_CHECK(cudaMemsetAsync(sums, 0, sizeof(double) * 2 * n_planes, stream));
    unsigned gy = (unsigned)std::min<long long>(ceil_div(n_rows, 64), 1024);
    SCN_LAUNCH(k_bn_stats, dim3((unsigned)ceil_div(n_planes, 32), gy), 256, 0, stream, in_features, n_rows, n_planes, in_stride, sums);
  }
  if (train)
    SCN_LAUNCH(k_bn_finalize, (unsigned)ceil_div(n_planes, 128), 128, 0, stream, n_planes, n_rows, sums, save_mean, save_invstd, running_mean, running_var, (float)eps, (float)momentum, train);
  const float *rm = train ? nullptr : running_mean, *rv = train ? nullptr : running_var;
  bool vec4 = (n_planes % 4 == 0) && (in_stride % 4 == 0) && (out_stride % 4 == 0) &&
              ((uintptr_t)in_features % 16 == 0) && ((uintptr_t)out_features % 16 == 0);
  long long work = n_rows * (vec4 ? n_planes / 4 : n_planes);
  unsigned blocks = (unsigned)std::min<long long>(ceil_div(work, 256), 148 * 16);
  size_t smem = sizeof(float) * 2 * n_planes;
  if (vec4)
    SCN_LAUNCH(k_bn_apply<4>, blocks, 256, smem, stream, in_features, out_features, n_rows, n_planes, in_stride, out_stride, save_mean, save_invstd, rm, rv, (float)eps, weight, bias, (float)leakiness);
  else
    SCN_LAUNCH(k_bn_apply<1>, blocks, 256, smem, stream, in_features, out_features, n_rows, n_planes, in_stride, out_stride, save_mean, save_invstd, rm, rv, (float)eps, weight, bias, (float)leakiness);
  SCN_CUDA_CHECK(cudaGetLastError());
  if (sums) SCN_TRY(device_free(sums, stream));
  return SCN_OK;
}

// Eval-mode BatchNorm (+ leaky ReLU) of the column-wise concatenation [a | b] without the concatenation being
// written first: a JoinTable followed by a BatchNormalization as one pass (read a and b once, write the
// result once; torch.cat + the stand-alone operator read and write the joined matrix twice).
__global__ void __launch_bounds__(256)
k_bn_apply_join(const float *__restrict__ a, int ca, const float *__restrict__ b, int cb, float *__restrict__ out,
                long long n_rows, const float *__restrict__ running_mean, const float *__restrict__ running_var,
                float eps, const float *__restrict__ weight, const float *__restrict__ bias, float leak) {
  extern __shared__ float sh_wb[];  // [2][ca + cb]
  const int C = ca + cb;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const float w = powf(running_var[c] + eps, -0.5f) * (weight ? weight[c] : 1.f);
    sh_wb[c] = w;
    sh_wb[C + c] = __fadd_rn(__fmul_rn(-running_mean[c], w), bias ? bias[c] : 0.f);
  }
  __syncthreads();
  const int cv = C / 4, cav = ca / 4;
  const long long total = n_rows * cv;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long r = idx / cv;
    const int q = (int)(idx % cv), c = q * 4;
    const float4 x = q < cav ? *reinterpret_cast<const float4 *>(a + r * ca + c)
                             : *reinterpret_cast<const float4 *>(b + r * cb + (c - ca));
    float4 y;
    y.x = __fadd_rn(__fmul_rn(x.x, sh_wb[c + 0]), sh_wb[C + c + 0]);
    y.y = __fadd_rn(__fmul_rn(x.y, sh_wb[c + 1]), sh_wb[C + c + 1]);
    y.z = __fadd_rn(__fmul_rn(x.z, sh_wb[c + 2]), sh_wb[C + c + 2]);
    y.w = __fadd_rn(__fmul_rn(x.w, sh_wb[c + 3]), sh_wb[C + c + 3]);
    y.x *= (y.x > 0.f) ? 1.f : leak;
    y.y *= (y.y > 0.f) ? 1.f : leak;
    y.z *= (y.z > 0.f) ? 1.f : leak;
    y.w *= (y.w > 0.f) ? 1.f : leak;
    *reinterpret_cast<float4 *>(out + r * C + c) = y;
  }
}

int scn_batchnorm_join_forward(const float *in_a, int planes_a, const float *in_b, int planes_b, float *out_features,
                               int64_t n_rows, const float *running_mean, const float *running_var,
                               const float *weight, const float *bias, double eps, double leakiness, void *stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  SCN_REQUIRE(planes_a >= 4 && planes_b >= 4 && planes_a % 4 == 0 && planes_b % 4 == 0 && planes_a + planes_b <= 4096,
              SCN_ERR_UNSUPPORTED, "plane counts %d + %d unsupported (multiples of four)", planes_a, planes_b);
  SCN_REQUIRE(running_mean && running_var, SCN_ERR_BAD_ARG, "null statistics");
  if (n_rows == 0) return SCN_OK;
  SCN_REQUIRE(in_a && in_b && out_features, SCN_ERR_BAD_ARG, "null features");
  SCN_REQUIRE((uintptr_t)in_a % 16 == 0 && (uintptr_t)in_b % 16 == 0 && (uintptr_t)out_features % 16 == 0,
              SCN_ERR_BAD_ARG, "feature matrices must be 16-byte aligned");
  const int C = planes_a + planes_b;
  const long long work = n_rows * (C / 4);
  const unsigned blocks = (unsigned)std::min<long long>(ceil_div(work, 256), 148 * 16);
  SCN_LAUNCH(k_bn_apply_join, blocks, 256, sizeof(float) * 2 * C, stream, in_a, planes_a, in_b, planes_b, out_features,
             n_rows, running_mean, running_var, (float)eps, weight, bias, (float)leakiness);
  SCN_CUDA_CHECK(cudaGetLastError());
  return SCN_OK;
}

int scn_rows_affine_forward(const float *in_features, float *out_features, int64_t n_rows, int n_in_planes,
                            int n_out_planes, const float *weight, const float *bias, void *stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  SCN_REQUIRE(n_in_planes >= 4 && n_in_planes % 4 == 0 && n_in_planes <= 256, SCN_ERR_UNSUPPORTED,
              "n_in_planes %d unsupported (a multiple of four, at most 256)", n_in_planes);
  SCN_REQUIRE(n_out_planes >= 1 && n_out_planes <= 32, SCN_ERR_UNSUPPORTED,
              "n_out_planes %d unsupported (1..32; wider products belong to the dense matrix library)",
              n_out_planes);
  SCN_REQUIRE(n_rows >= 0 && n_rows < (1ll << 31) * 256, SCN_ERR_BAD_ARG, "bad row count");
  if (n_rows == 0) return SCN_OK;
  SCN_REQUIRE(in_features && out_features && weight, SCN_ERR_BAD_ARG, "null argument");
  SCN_REQUIRE((uintptr_t)in_features % 16 == 0 && (uintptr_t)out_features % 16 == 0, SCN_ERR_BAD_ARG,
              "feature matrices must be 16-byte aligned");
  const int c4 = (n_out_planes + 3) / 4;
  const unsigned blocks = (unsigned)std::min<long long>(ceil_div(n_rows, 256), 148 * 8);
  const size_t smem = sizeof(float) * (4 * (size_t)c4 * n_in_planes + 8 * 32 * kAffineStride);
  // up to 32 KB of weights + 37 KB of tiles: above the 48 KB a kernel gets without asking
  static bool configured[64] = {false};
  int dev = 0;
  SCN_CUDA_CHECK(cudaGetDevice(&dev));
  const bool configure = dev < 0 || dev >= 64 || !configured[dev];
#define SCN_AFFINE(N)                                                                                       \
  case N:                                                                                                   \
    if (configure)                                                                                          \
      SCN_CUDA_CHECK(cudaFuncSetAttribute(k_rows_affine<N>, cudaFuncAttributeMaxDynamicSharedMemorySize,    \
                                          72 * 1024));                                                      \
    SCN_LAUNCH(k_rows_affine<N>, blocks, 256, smem, stream, in_features, out_features, (long long)n_rows,   \
               n_in_planes, n_out_planes, weight, bias);                                                    \
    break;
  switch (c4) {
    SCN_AFFINE(1) SCN_AFFINE(2) SCN_AFFINE(3) SCN_AFFINE(4) SCN_AFFINE(5) SCN_AFFINE(6) SCN_AFFINE(7) SCN_AFFINE(8)
  }
#undef SCN_AFFINE
  SCN_CUDA_CHECK(cudaGetLastError());
  return SCN_OK;
}

int scn_batchnorm_backward(const float *in_features, float *d_in_features, const float *out_features,
                           const float *d_out_features, int64_t n_rows, int n_planes, int64_t in_stride,
                           int64_t out_stride, const float *save_mean, const float *save_invstd,
                           const float *weight, float *d_weight, float *d_bias, double leakiness, void *stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  SCN_REQUIRE(n_planes >= 1 && n_planes <= 4096, SCN_ERR_UNSUPPORTED, "n_planes %d unsupported", n_planes);
  SCN_REQUIRE(save_mean && save_invstd, SCN_ERR_BAD_ARG, "null statistics");
  SCN_REQUIRE(in_stride >= n_planes && out_stride >= n_planes, SCN_ERR_BAD_ARG, "row stride below n_planes");
  if (n_rows == 0) {
    if (d_weight) SCN_CUDA_CHECK(cudaMemsetAsync(d_weight, 0, sizeof(float) * n_planes, stream));
    if (d_bias) SCN_CUDA_CHECK(cudaMemsetAsync(d_bias, 0, sizeof(float) * n_planes, stream));
    return SCN_OK;
  }
  SCN_REQUIRE(in_features && d_in_features && out_features && d_out_features, SCN_ERR_BAD_ARG, "null features");
  const int chunks = (int)std::max<long long>(1, std::min<long long>(1024, n_rows / 256));
  const long long chunk_rows = ceil_div(n_rows, chunks);
  double *partial = nullptr;
  float *coef = nullptr;
  SCN_TRY(device_alloc((void **)&partial, sizeof(double) * 2 * (size_t)chunks * n_planes, stream));
  SCN_TRY(device_alloc((void **)&coef, sizeof(float) * 2 * (size_t)n_planes, stream));
  SCN_LAUNCH(k_bn_back_sums, dim3((unsigned)ceil_div(n_planes, 32), (unsigned)chunks), 256, 0, stream, in_features, out_features, d_out_features, n_rows, n_planes, in_stride, out_stride, save_mean, (float)leakiness, chunk_rows, partial);
  SCN_LAUNCH(k_bn_back_finalize, (unsigned)ceil_div(n_planes, 128), 128, 0, stream, partial, chunks, n_planes, n_rows, save_invstd, d_weight, d_bias, coef);
  SCN_LAUNCH(k_bn_back_apply, (unsigned)ceil_div(n_rows * n_planes, 256), 256, 0, stream, in_features, d_in_features, out_features, d_out_features, n_rows, n_planes, in_stride, out_stride, save_mean, save_invstd, weight, coef, (float)leakiness);
  SCN_CUDA_CHECK(cudaGetLastError());
  SCN_TRY(device_free(partial, stream));
  SCN_TRY(device_free(coef, stream));
  return SCN_OK;
}

static void launch_bn_apply(const float *in, float *out, long long n_rows, int n_planes, long long in_stride,
                            long long out_stride, float *save_mean, float *save_invstd, const float *weight,
                            const float *bias, float leakiness, cudaStream_t stream) {
  const bool vec4 = (n_planes % 4 == 0) && (in_stride % 4 == 0) && (out_stride % 4 == 0) &&
                    ((uintptr_t)in % 16 == 0) && ((uintptr_t)out % 16 == 0);
  const long long work = n_rows * (vec4 ? n_planes / 4 : n_planes);
  const unsigned blocks = (unsigned)std::min<long long>(ceil_div(work, 256), 148 * 16);
  const size_t smem = sizeof(float) * 2 * n_planes;
  if (vec4)
    SCN_LAUNCH(k_bn_apply<4>, blocks, 256, smem, stream, in, out, n_rows, n_planes, in_stride, out_stride, save_mean, save_invstd, nullptr, nullptr, 0.f, weight, bias, leakiness);
  else
    SCN_LAUNCH(k_bn_apply<1>, blocks, 256, smem, stream, in, out, n_rows, n_planes, in_stride, out_stride, save_mean, save_invstd, nullptr, nullptr, 0.f, weight, bias, leakiness);
}

int scn_batchnorm_moments(const float *in_features, int64_t n_rows, int n_planes, int64_t in_stride, double *sums,
                          void *stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  SCN_REQUIRE(n_planes >= 1 && n_planes <= 4096, SCN_ERR_UNSUPPORTED, "n_planes %d unsupported", n_planes);
  SCN_REQUIRE(sums && n_rows >= 0, SCN_ERR_BAD_ARG, "null sums or negative row count");
  SCN_REQUIRE(in_stride >= n_planes, SCN_ERR_BAD_ARG, "row stride below n_planes");
  SCN_CUDA_CHECK(cudaMemsetAsync(sums, 0, sizeof(double) * 2 * n_planes, stream));
  if (n_rows == 0) return SCN_OK;
  SCN_REQUIRE(in_features, SCN_ERR_BAD_ARG, "null features");
  const unsigned gy = (unsigned)std::min<long long>(ceil_div(n_rows, 64), 1024);
  SCN_LAUNCH(k_bn_stats, dim3((unsigned)ceil_div(n_planes, 32), gy), 256, 0, stream, in_features, n_rows, n_planes, in_stride, sums);
  SCN_CUDA_CHECK(cudaGetLastError());
  return SCN_OK;
}

int scn_batchnorm_forward_moments(const float *in_features, float *out_features, int64_t n_rows,
                                  int64_t n_rows_total, int n_planes, int64_t in_stride, int64_t out_stride,
                                  const double *sums, float *save_mean, float *save_invstd, float *running_mean,
                                  float *running_var, const float *weight, const float *bias, double eps,
                                  double momentum, double leakiness, void *stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  SCN_REQUIRE(n_planes >= 1 && n_planes <= 4096, SCN_ERR_UNSUPPORTED, "n_planes %d unsupported", n_planes);
  SCN_REQUIRE(sums && save_mean && save_invstd && running_mean && running_var, SCN_ERR_BAD_ARG, "null statistics");
  SCN_REQUIRE(in_stride >= n_planes && out_stride >= n_planes, SCN_ERR_BAD_ARG, "row stride below n_planes");
  SCN_REQUIRE(n_rows >= 0 && (n_rows_total < 0 || n_rows_total >= n_rows), SCN_ERR_BAD_ARG,
              "total row count below this device's");
  if (n_rows_total == 0) return SCN_OK;
  SCN_LAUNCH(k_bn_finalize, (unsigned)ceil_div(n_planes, 128), 128, 0, stream, n_planes, (long long)n_rows_total, sums, save_mean, save_invstd, running_mean, running_var, (float)eps, (float)momentum, 1, n_rows_total < 0 ? 1 : 0);
  if (n_rows > 0) {
    SCN_REQUIRE(in_features && out_features, SCN_ERR_BAD_ARG, "null features");
    launch_bn_apply(in_features, out_features, n_rows, n_planes, in_stride, out_stride, save_mean, save_invstd, weight, bias, (float)leakiness, stream);
  }
  SCN_CUDA_CHECK(cudaGetLastError());
  return SCN_OK;
}

int scn_batchnorm_backward_sums(const float *in_features, const float *out_features, const float *d_out_features,
                                int64_t n_rows, int n_planes, int64_t in_stride, int64_t out_stride,
                                const float *save_mean, double leakiness, double *sums, void *stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  SCN_REQUIRE(n_planes >= 1 && n_planes <= 4096, SCN_ERR_UNSUPPORTED, "n_planes %d unsupported", n_planes);
  SCN_REQUIRE(sums && save_mean && n_rows >= 0, SCN_ERR_BAD_ARG, "null sums or statistics");
  SCN_REQUIRE(in_stride >= n_planes && out_stride >= n_planes, SCN_ERR_BAD_ARG, "row stride below n_planes");
  if (n_rows == 0) {
    SCN_CUDA_CHECK(cudaMemsetAsync(sums, 0, sizeof(double) * 2 * n_planes, stream));
    return SCN_OK;
  }
  SCN_REQUIRE(in_features && out_features && d_out_features, SCN_ERR_BAD_ARG, "null features");
  const int chunks = (int)std::max<long long>(1, std::min<long long>(1024, n_rows / 256));
  const long long chunk_rows = ceil_div(n_rows, chunks);
  double *partial = nullptr;
  SCN_TRY(device_alloc((void **)&partial, sizeof(double) * 2 * (size_t)chunks * n_planes, stream));
  SCN_LAUNCH(k_bn_back_sums, dim3((unsigned)ceil_div(n_planes, 32), (unsigned)chunks), 256, 0, stream, in_features, out_features, d_out_features, (long long)n_rows, n_planes, (long long)in_stride, (long long)out_stride, save_mean, (float)leakiness, chunk_rows, partial);
  SCN_LAUNCH(k_bn_back_reduce, (unsigned)ceil_div(n_planes, 128), 128, 0, stream, partial, chunks, n_planes, sums);
  const cudaError_t err = cudaGetLastError();
  SCN_TRY(device_free(partial, stream));
  SCN_CUDA_CHECK(err);
  return SCN_OK;
}

int scn_batchnorm_backward_sums_apply(const float *in_features, float *d_in_features, const float *out_features,
                                      const float *d_out_features, int64_t n_rows, int64_t n_rows_total,
                                      int n_planes, int64_t in_stride, int64_t out_stride, const float *save_mean,
                                      const float *save_invstd, const float *weight, const double *local_sums,
                                      const double *total_sums, float *d_weight, float *d_bias, double leakiness,
                                      void *stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  SCN_REQUIRE(n_planes >= 1 && n_planes <= 4096, SCN_ERR_UNSUPPORTED, "n_planes %d unsupported", n_planes);
  SCN_REQUIRE(save_mean && save_invstd && local_sums && total_sums, SCN_ERR_BAD_ARG, "null statistics or sums");
  SCN_REQUIRE(in_stride >= n_planes && out_stride >= n_planes, SCN_ERR_BAD_ARG, "row stride below n_planes");
  SCN_REQUIRE(n_rows >= 0 && (n_rows_total < 0 || (n_rows_total >= n_rows && n_rows_total >= 1)), SCN_ERR_BAD_ARG,
              "total row count below this device's, or no rows at all");
  float *coef = nullptr;
  SCN_TRY(device_alloc((void **)&coef, sizeof(float) * 2 * (size_t)n_planes, stream));
  SCN_LAUNCH(k_bn_back_coef, (unsigned)ceil_div(n_planes, 128), 128, 0, stream, local_sums, total_sums, n_planes, (long long)n_rows_total, save_invstd, d_weight, d_bias, coef);
  if (n_rows > 0) {
    if (!(in_features && d_in_features && out_features && d_out_features)) {
      device_free(coef, stream);
      SCN_REQUIRE(false, SCN_ERR_BAD_ARG, "null features");
    }
    SCN_LAUNCH(k_bn_back_apply, (unsigned)ceil_div(n_rows * n_planes, 256), 256, 0, stream, in_features, d_in_features, out_features, d_out_features, (long long)n_rows, n_planes, (long long)in_stride, (long long)out_stride, save_mean, save_invstd, weight, coef, (float)leakiness);
  }
  const cudaError_t err = cudaGetLastError();
  SCN_TRY(device_free(coef, stream));
  SCN_CUDA_CHECK(err);
  return SCN_OK;
}

int scn_max_pooling_forward(scn_metadata *md, const int64_t *input_size, const int64_t *output_size,
                            const int64_t *pool_size, const int64_t *pool_stride,
                            const float *in_features, float *out_features, int n_planes_in,
                            int n_features_to_drop, void *stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  SCN_REQUIRE(md && input_size && output_size && pool_size && pool_stride, SCN_ERR_BAD_ARG, "null argument");
  SCN_REQUIRE(n_features_to_drop >= 0 && n_features_to_drop < n_planes_in, SCN_ERR_BAD_ARG,
              "n_features_to_drop %d not in [0, %d)", n_features_to_drop, n_planes_in);
  Rulebook *rb = nullptr;
  SCN_TRY(get_strided_rulebook(md, input_size, output_size, pool_size, pool_stride, stream, &rb));
  if (rb->n_out == 0) return SCN_OK;
  SCN_REQUIRE(in_features && out_features, SCN_ERR_BAD_ARG, "null features");
  int c_out = n_planes_in - n_features_to_drop;
  long long total = rb->n_out * c_out;
  SCN_LAUNCH(k_max_pool, (unsigned)ceil_div(total, 256), 256, 0, stream, in_features, out_features, rb->nbr, rb->n_out, rb->n_in, rb->n_offsets, c_out, n_planes_in, n_features_to_drop, md->flags_dev);
  SCN_CUDA_CHECK(cudaGetLastError());
  return SCN_OK;
}

int scn_average_pooling_forward(scn_metadata *md, const int64_t *input_size, const int64_t *output_size,
                                const int64_t *pool_size, const int64_t *pool_stride,
                                const float *in_features, float *out_features, int n_planes_in,
                                int n_features_to_drop, void *stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  SCN_REQUIRE(md && input_size && output_size && pool_size && pool_stride, SCN_ERR_BAD_ARG, "null argument");
  SCN_REQUIRE(n_features_to_drop >= 0 && n_features_to_drop < n_planes_in, SCN_ERR_BAD_ARG,
              "n_features_to_drop %d not in [0, %d)", n_features_to_drop, n_planes_in);
  Rulebook *rb = nullptr;
  SCN_TRY(get_strided_rulebook(md, input_size, output_size, pool_size, pool_stride, stream, &rb));
  if (rb->n_out == 0) return SCN_OK;
  SCN_REQUIRE(in_features && out_features, SCN_ERR_BAD_ARG, "null features");
  int c_out = n_planes_in - n_features_to_drop;
  long long total = rb->n_out * c_out;
  SCN_LAUNCH(k_sum_pool<true>, (unsigned)ceil_div(total, 256), 256, 0, stream, in_features, out_features, rb->nbr, rb->n_out, rb->n_in, rb->n_offsets, c_out, n_planes_in, n_features_to_drop, md->flags_dev);
  SCN_CUDA_CHECK(cudaGetLastError());
  return SCN_OK;
}

int scn_unpooling_forward(scn_metadata *md, const int64_t *input_size, const int64_t *output_size,
                          const int64_t *pool_size, const int64_t *pool_stride, const float *in_features,
                          float *out_features, int n_planes_in, int n_features_to_drop, void *stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  SCN_REQUIRE(md && input_size && output_size && pool_size && pool_stride, SCN_ERR_BAD_ARG, "null argument");
  SCN_REQUIRE(n_features_to_drop >= 0 && n_features_to_drop < n_planes_in, SCN_ERR_BAD_ARG,
              "n_features_to_drop %d not in [0, %d)", n_features_to_drop, n_planes_in);
  // the fine grid (output_size) must exist: its sites are what gets un-pooled onto
  SCN_REQUIRE(find_grid(md, output_size), SCN_ERR_NO_GRID, "UnPooling: no grid for the output spatial size");
  Rulebook *rb = nullptr;  // rulebook of fine (output_size) -> coarse (input_size)
  SCN_TRY(get_strided_rulebook(md, output_size, input_size, pool_size, pool_stride, stream, &rb));
  if (rb->n_in == 0) return SCN_OK;
  SCN_REQUIRE(out_features && (in_features || rb->n_out == 0), SCN_ERR_BAD_ARG, "null features");
  SCN_TRY(rulebook_transposed(*rb, stream));
  int c_out = n_planes_in - n_features_to_drop;
  long long total = rb->n_in * c_out;
  SCN_LAUNCH(k_sum_pool<false>, (unsigned)ceil_div(total, 256), 256, 0, stream, in_features, out_features, rb->tnbr, rb->n_in, rb->n_out, rb->n_offsets, c_out, n_planes_in, n_features_to_drop, md->flags_dev);
  SCN_CUDA_CHECK(cudaGetLastError());
  return SCN_OK;
}

int scn_sparse_to_dense_forward(scn_metadata *md, const int64_t *spatial_size, const float *in_features,
                                float *out_dense, int n_planes, void *stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  SCN_REQUIRE(md && spatial_size, SCN_ERR_BAD_ARG, "null argument");
  Grid *g = find_grid(md, spatial_size);
  SCN_REQUIRE(g, SCN_ERR_NO_GRID, "no grid for that spatial size");
  long long volume = 1;
  for (int d = 0; d < md->dim; ++d) volume *= spatial_size[d];
  size_t bytes = sizeof(float) * (size_t)g->batch_size * n_planes * volume;
  if (bytes == 0) return SCN_OK;
  SCN_REQUIRE(out_dense, SCN_ERR_BAD_ARG, "null output");
  SCN_TRY(md_touch(md, stream));
  SCN_CUDA_CHECK(cudaMemsetAsync(out_dense, 0, bytes, stream));
  if (g->n_active == 0) return SCN_OK;
  SCN_REQUIRE(in_features, SCN_ERR_BAD_ARG, "null features");
  long long total = g->n_active * n_planes;
  SCN_LAUNCH(k_sparse_to_dense, (unsigned)ceil_div(total, 256), 256, 0, stream, g->layout, g->row_keys, in_features, out_dense, g->n_active, n_planes, volume);
  SCN_CUDA_CHECK(cudaGetLastError());
  return SCN_OK;
}

/* ---- backward passes of the feature operators ------------------------------------------------ */

int scn_input_layer_backward(scn_metadata *md, float *d_in_features, int64_t n_points,
                             const float *d_out_features, int64_t n_sites, int n_planes, void *stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  SCN_REQUIRE(md && md->input_mode >= 0, SCN_ERR_NO_GRID, "no input layer has been run on this metadata");
  SCN_REQUIRE(n_points == md->input_n_rows && n_sites == md->input_n_active, SCN_ERR_SIZE_MISMATCH,
              "input layer backward: got %lld points, %lld sites; metadata has %lld, %lld", (long long)n_points,
              (long long)n_sites, md->input_n_rows, md->input_n_active);
  SCN_REQUIRE(n_planes >= 1, SCN_ERR_BAD_ARG, "n_planes must be positive");
  if (n_points == 0) return SCN_OK;
  SCN_REQUIRE(d_in_features && (d_out_features || n_sites == 0), SCN_ERR_BAD_ARG, "null features");
  const size_t bytes = sizeof(float) * (size_t)n_points * n_planes;
  if (md->input_mode == 0) {
    SCN_CUDA_CHECK(cudaMemcpyAsync(d_in_features, d_out_features, bytes, cudaMemcpyDeviceToDevice, stream));
    return SCN_OK;
  }
  SCN_CUDA_CHECK(cudaMemsetAsync(d_in_features, 0, bytes, stream));
  if (n_sites == 0) return SCN_OK;
  long long total = (long long)n_sites * n_planes;
  SCN_LAUNCH(k_output_features, (unsigned)ceil_div(total, 256), 256, 0, stream, d_out_features, d_in_features, md->input_csr_start, md->input_csr_rows, n_sites, n_planes, md->input_mode, md->input_mode == 4 ? 1 : 0);
  SCN_CUDA_CHECK(cudaGetLastError());
  return SCN_OK;
}

int scn_output_layer_backward(scn_metadata *md, float *d_in_features, int64_t n_sites,
                              const float *d_out_features, int64_t n_points, int n_planes, void *stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  SCN_REQUIRE(md && md->input_mode >= 0, SCN_ERR_NO_GRID, "no input layer has been run on this metadata");
  SCN_REQUIRE(n_points == md->input_n_rows && n_sites == md->input_n_active, SCN_ERR_SIZE_MISMATCH,
              "output layer backward: got %lld points, %lld sites; metadata has %lld, %lld", (long long)n_points,
              (long long)n_sites, md->input_n_rows, md->input_n_active);
  SCN_REQUIRE(n_planes >= 1, SCN_ERR_BAD_ARG, "n_planes must be positive");
  if (n_sites == 0) return SCN_OK;
  SCN_REQUIRE(d_in_features && d_out_features, SCN_ERR_BAD_ARG, "null features");
  if (md->input_mode == 0) {
    SCN_CUDA_CHECK(cudaMemcpyAsync(d_in_features, d_out_features, sizeof(float) * (size_t)n_sites * n_planes,
                                   cudaMemcpyDeviceToDevice, stream));
    return SCN_OK;
  }
  // every site collects, unscaled, the gradients of the points its rule names (CPU/IOLayers.cpp:116-136)
  const int mode = md->input_mode == 4 ? 3 : md->input_mode;
  long long total = (long long)n_sites * n_planes;
  SCN_LAUNCH(k_input_features, (unsigned)ceil_div(total, 256), 256, 0, stream, d_out_features, d_in_features, md->input_csr_start, md->input_csr_rows, n_sites, n_planes, mode);
  SCN_CUDA_CHECK(cudaGetLastError());
  return SCN_OK;
}

static int pool_backward(scn_metadata *md, int op, const int64_t *input_size, const int64_t *output_size,
                         const int64_t *pool_size, const int64_t *pool_stride, const float *in_features,
                         float *d_in_features, const float *out_features, const float *d_out_features,
                         int n_planes_in, int n_features_to_drop, cudaStream_t stream) {
  SCN_REQUIRE(md && input_size && output_size && pool_size && pool_stride, SCN_ERR_BAD_ARG, "null argument");
  SCN_REQUIRE(n_features_to_drop >= 0 && n_features_to_drop < n_planes_in, SCN_ERR_BAD_ARG,
              "n_features_to_drop %d not in [0, %d)", n_features_to_drop, n_planes_in);
  Rulebook *rb = nullptr;
  const int *table = nullptr;
  long long n_rows = 0, n_other = 0;
  if (op == 2) {  // UnPooling: input = coarse; rulebook of (fine = output_size) -> (coarse = input_size)
    SCN_TRY(get_strided_rulebook(md, output_size, input_size, pool_size, pool_stride, stream, &rb));
    table = rb->nbr;
    n_rows = rb->n_out;
    n_other = rb->n_in;
  } else {
    SCN_TRY(get_strided_rulebook(md, input_size, output_size, pool_size, pool_stride, stream, &rb));
    SCN_TRY(rulebook_transposed(*rb, stream));
    table = rb->tnbr;
    n_rows = rb->n_in;
    n_other = rb->n_out;
  }
  if (n_rows == 0) return SCN_OK;
  SCN_REQUIRE(d_in_features && (d_out_features || n_other == 0), SCN_ERR_BAD_ARG, "null gradient");
  SCN_REQUIRE(op != 0 || (in_features && (out_features || n_other == 0)), SCN_ERR_BAD_ARG, "null features");
  long long total = n_rows * n_planes_in;
  unsigned blocks = (unsigned)ceil_div(total, 256);
  if (op == 0)
    SCN_LAUNCH(k_pool_backward<0>, blocks, 256, 0, stream, in_features, d_in_features, out_features, d_out_features, table, n_rows, n_other, rb->n_offsets, n_planes_in, n_features_to_drop, md->flags_dev);
  else if (op == 1)
    SCN_LAUNCH(k_pool_backward<1>, blocks, 256, 0, stream, in_features, d_in_features, out_features, d_out_features, table, n_rows, n_other, rb->n_offsets, n_planes_in, n_features_to_drop, md->flags_dev);
  else
    SCN_LAUNCH(k_pool_backward<2>, blocks, 256, 0, stream, in_features, d_in_features, out_features, d_out_features, table, n_rows, n_other, rb->n_offsets, n_planes_in, n_features_to_drop, md->flags_dev);
  SCN_CUDA_CHECK(cudaGetLastError());
  return SCN_OK;
}

int scn_max_pooling_backward(scn_metadata *md, const int64_t *input_size, const int64_t *output_size,
                             const int64_t *pool_size, const int64_t *pool_stride, const float *in_features,
                             float *d_in_features, const float *out_features, const float *d_out_features,
                             int n_planes_in, int n_features_to_drop, void *stream) {
  return pool_backward(md, 0, input_size, output_size, pool_size, pool_stride, in_features, d_in_features,
                       out_features, d_out_features, n_planes_in, n_features_to_drop, (cudaStream_t)stream);
}

int scn_average_pooling_backward(scn_metadata *md, const int64_t *input_size, const int64_t *output_size,
                                 const int64_t *pool_size, const int64_t *pool_stride, float *d_in_features,
                                 const float *d_out_features, int n_planes_in, int n_features_to_drop,
                                 void *stream) {
  return pool_backward(md, 1, input_size, output_size, pool_size, pool_stride, nullptr, d_in_features, nullptr,
                       d_out_features, n_planes_in, n_features_to_drop, (cudaStream_t)stream);
}

int scn_unpooling_backward(scn_metadata *md, const int64_t *input_size, const int64_t *output_size,
                           const int64_t *pool_size, const int64_t *pool_stride, float *d_in_features,
                           const float *d_out_features, int n_planes_in, int n_features_to_drop, void *stream) {
  return pool_backward(md, 2, input_size, output_size, pool_size, pool_stride, nullptr, d_in_features, nullptr,
                       d_out_features, n_planes_in, n_features_to_drop, (cudaStream_t)stream);
}

int scn_sparse_to_dense_backward(scn_metadata *md, const int64_t *spatial_size, float *d_in_features,
                                 const float *d_out_dense, int n_planes, void *stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  SCN_REQUIRE(md && spatial_size, SCN_ERR_BAD_ARG, "null argument");
  Grid *g = find_grid(md, spatial_size);
  SCN_REQUIRE(g, SCN_ERR_NO_GRID, "no grid for that spatial size");
  if (g->n_active == 0) return SCN_OK;
  SCN_REQUIRE(d_in_features && d_out_dense, SCN_ERR_BAD_ARG, "null gradient");
  long long volume = 1;
  for (int d = 0; d < md->dim; ++d) volume *= spatial_size[d];
  long long total = g->n_active * n_planes;
  SCN_LAUNCH(k_dense_to_sparse_grad, (unsigned)ceil_div(total, 256), 256, 0, stream, g->layout, g->row_keys, d_out_dense, d_in_features, g->n_active, n_planes, volume);
  SCN_CUDA_CHECK(cudaGetLastError());
  return SCN_OK;
}
}
