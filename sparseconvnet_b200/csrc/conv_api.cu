// C-ABI entry points of the three convolution operators: rulebook lookup (built on first use
// and cached, like the reference's Metadata), shape checks, kernel choice.
#include <stdlib.h>

#include <algorithm>
#include <atomic>
#include <map>
#include <mutex>
#include <tuple>

#include "metadata.cuh"
#include "tc_ptx.cuh"

namespace scn {
int conv_forward_simt(const float *in, long long n_in, float *out, long long n_out, const float *weight,
                      const float *bias, const int *table, int K, int cin, int cout, int groups,
                      int *flags, cudaStream_t stream);
int conv_forward_tc(const float *in, long long n_in, float *out, long long n_out, const float *weight,
                    const float *bias, const float *bn_scale, const float *bn_shift, float leak, const int *table,
                    int K, int cin, int cout, int precision, int *flags, cudaStream_t stream,
                    const float *pre_scale = nullptr, const float *pre_shift = nullptr, float pre_leak = 1.f,
                    const float *in_b = nullptr, int planes_a = 0);
bool conv_tc_supported(int cin, int cout, int groups, int precision);
bool conv_tc_splits_rows(int precision, int cin, long long n_in, long long n_out);
int conv_forward_tma(const float *in, long long n_in, float *out, long long n_out, const float *weight,
                     const float *bias, const int *table, int K, int cin, int cout, int precision, int *flags,
                     cudaStream_t stream);
bool conv_tma_supported(int K, int cin, int cout, int groups, int precision, long long n_in);
bool conv_wide_supported(int K, int cin, int cout, int groups, int precision, long long n_in);
int conv_forward_wide(const float *in, long long n_in, float *out, long long n_out, const float *weight,
                      const float *bias, const float *bn_scale, const float *bn_shift, float leak, const int *table,
                      int K, int cin, int cout, int precision, int *flags, cudaStream_t stream,
                      const float *pre_scale = nullptr, const float *pre_shift = nullptr, float pre_leak = 1.f,
                      const float *in_b = nullptr, int planes_a = 0);
bool conv_pipe_supported(const float *in, const float *out, const float *weight, const float *bias, int K, int cin,
                         int cout);
int conv_forward_pipe(const float *in, long long n_in, float *out, long long n_out, const float *weight,
                      const float *bias, const int *table, int K, int cin, int cout, int groups, int three_pass_mma,
                      int *flags, cudaStream_t stream);

bool conv_rows_supported(const float *in, const float *out, const float *weight, const float *bias, int K, int cin,
                         int cout, int groups);
int conv_forward_rows(const float *in, long long n_in, float *out, long long n_out, const float *weight,
                      const float *bias, const float *bn_scale, const float *bn_shift, float leak, const int *table,
                      int K, int cin, int cout, int precision, int *flags, cudaStream_t stream);

bool conv_rows_thin_supported(const float *out, const float *bias, int cin, int cout, int groups);
int conv_forward_rows_thin(const float *in, long long n_in, float *out, long long n_out, const float *weight,
                           const float *bias, const float *bn_scale, const float *bn_shift, float leak,
                           const int *table, int K, int cin, int cout, int *flags, cudaStream_t stream);

int conv_forward_rows_scatter(const float *in, long long n_in, float *out, long long n_out, const float *weight,
                              const float *bias, const float *bn_scale, const float *bn_shift, float leak,
                              const int *child_of, int K, int cin, int cout, int *flags, cudaStream_t stream);

int split_mode_of_env(int dflt) {
  const char *e = getenv("SCN_X3_FORM");
  if (e && e[0] == 't') return TC_TF32X3;
  if (e && e[0] == 'b') return TC_BF16X3;
  return dflt;
}

// ---- prepared weight images kept under a caller-chosen token ------------------------------------------
namespace {
struct WeightKey {
  int device;
  unsigned long long token;
  int kind, K, cin, cout, extra;
  bool operator<(const WeightKey &o) const {
    return std::tie(device, token, kind, K, cin, cout, extra) <
           std::tie(o.device, o.token, o.kind, o.K, o.cin, o.cout, o.extra);
  }
};
std::mutex g_weight_mu;
std::map<WeightKey, void *> g_weight_images;
thread_local unsigned long long g_weight_token = 0;
}  // namespace

int weight_image_get(int kind, int K, int cin, int cout, int extra, size_t bytes, cudaStream_t stream,
                     WeightImage *img, bool *needs_build) {
  *needs_build = true;
  img->cached = false;
  if (g_weight_token != 0) {
    int dev = 0;
    SCN_CUDA_CHECK(cudaGetDevice(&dev));
    const WeightKey key{dev, g_weight_token, kind, K, cin, cout, extra};
    std::lock_guard<std::mutex> lock(g_weight_mu);
    auto it = g_weight_images.find(key);
    if (it != g_weight_images.end()) {
      img->ptr = it->second;
      *needs_build = false;
    } else {
      SCN_TRY(device_alloc(&img->ptr, bytes, stream));
      g_weight_images[key] = img->ptr;
    }
    img->cached = true;
    return SCN_OK;
  }
  return device_alloc(&img->ptr, bytes, stream);
}

int weight_image_put(WeightImage &img, cudaStream_t stream) {
  if (img.cached || !img.ptr) return SCN_OK;
  void *p = img.ptr;
  img.ptr = nullptr;
  return device_free(p, stream);
}

static thread_local int g_last_kernel = -1;
static std::atomic<int> g_deferred_counts{0};
std::atomic<int> g_backward_precision{SCN_PRECISION_FP32};  // arithmetic of the input-gradient pass

// Kernel choice for out [rows_out, groups * cout] = bias + sum_k in[table[k][.]] @ W[k]; shared by the
// forward operators and by the input-gradient pass of the backward ones (same kernels, opposite table).
// y = y * scale[plane] + shift[plane], then leaky ReLU, in place: the eval-mode BatchNorm behind a
// convolution whose kernel has no fused epilogue
__global__ void k_scale_shift_act(float *__restrict__ y, long long n_rows, int planes, const float *__restrict__ scale,
                                  const float *__restrict__ shift, float leak) {
  const long long total = n_rows * planes;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % planes);
    float v = __fadd_rn(__fmul_rn(y[i], scale[c]), shift[c]);
    v *= (v > 0.f) ? 1.f : leak;
    y[i] = v;
  }
}

// the same out of place: the eval-mode BatchNorm in FRONT of a convolution whose kernel has no split pass to take it
// (planes a multiple of four and 16-byte aligned matrices: four planes per thread; otherwise one)
__global__ void k_scale_shift_act_to(const float *__restrict__ x, float *__restrict__ y, long long n_rows, int planes,
                                     const float *__restrict__ scale, const float *__restrict__ shift, float leak, int vec) {
  if (vec) {
    const long long total = n_rows * planes / 4;
    const int pv = planes / 4;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
      const int c = (int)(i % pv) * 4;
      const float4 v = __ldg(reinterpret_cast<const float4 *>(x) + i);
      const float4 sc = __ldg(reinterpret_cast<const float4 *>(scale + c)), sh = __ldg(reinterpret_cast<const float4 *>(shift + c));
      float4 o;
      o.x = __fadd_rn(__fmul_rn(v.x, sc.x), sh.x), o.y = __fadd_rn(__fmul_rn(v.y, sc.y), sh.y);
      o.z = __fadd_rn(__fmul_rn(v.z, sc.z), sh.z), o.w = __fadd_rn(__fmul_rn(v.w, sc.w), sh.w);
      o.x *= (o.x > 0.f) ? 1.f : leak, o.y *= (o.y > 0.f) ? 1.f : leak;
      o.z *= (o.z > 0.f) ? 1.f : leak, o.w *= (o.w > 0.f) ? 1.f : leak;
      reinterpret_cast<float4 *>(y)[i] = o;
    }
    return;
  }
  const long long total = n_rows * planes;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % planes);
    float v = __fadd_rn(__fmul_rn(x[i], scale[c]), shift[c]);
    v *= (v > 0.f) ? 1.f : leak;
    y[i] = v;
  }
}

// the column-wise concatenation [a (ca planes) | b (cb planes)] through the same BatchNorm into one scratch matrix:
// a JoinTable and a BatchNorm in front of a convolution whose kernel has no split pass (planes multiples of four)
__global__ void k_scale_shift_act_join_to(const float *__restrict__ a, int ca, const float *__restrict__ b, int cb,
                                          float *__restrict__ y, long long n_rows, const float *__restrict__ scale,
                                          const float *__restrict__ shift, float leak) {
  const int pv = (ca + cb) / 4, av = ca / 4;
  const long long total = n_rows * pv;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / pv;
    const int q = (int)(i % pv), c = q * 4;
    float4 v = q < av ? __ldg(reinterpret_cast<const float4 *>(a + r * ca + c))
                      : __ldg(reinterpret_cast<const float4 *>(b + r * cb + (c - ca)));
    if (scale) {
      const float4 sc = __ldg(reinterpret_cast<const float4 *>(scale + c)), sh = __ldg(reinterpret_cast<const float4 *>(shift + c));
      v.x = __fadd_rn(__fmul_rn(v.x, sc.x), sh.x), v.y = __fadd_rn(__fmul_rn(v.y, sc.y), sh.y);
      v.z = __fadd_rn(__fmul_rn(v.z, sc.z), sh.z), v.w = __fadd_rn(__fmul_rn(v.w, sc.w), sh.w);
      v.x *= (v.x > 0.f) ? 1.f : leak, v.y *= (v.y > 0.f) ? 1.f : leak;
      v.z *= (v.z > 0.f) ? 1.f : leak, v.w *= (v.w > 0.f) ? 1.f : leak;
    }
    reinterpret_cast<float4 *>(y)[i] = v;
  }
}

// W, x -> scale = gamma / sqrt(var + eps), shift = beta - mean * scale, with the roundings of the
// stand-alone BatchNorm kernel (CPU/BatchNormalization.cpp:41-46 of the reference)
__global__ void k_bn_fold(const float *__restrict__ mean, const float *__restrict__ var, const float *__restrict__ gamma,
                          const float *__restrict__ beta, float eps, int planes, float *__restrict__ scale,
                          float *__restrict__ shift) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= planes) return;
  const float w = powf(var[c] + eps, -0.5f) * (gamma ? gamma[c] : 1.f);
  scale[c] = w;
  shift[c] = __fadd_rn(__fmul_rn(-mean[c], w), beta ? beta[c] : 0.f);
}

// pre_scale / pre_shift / pre_leak (optional): an eval-mode BatchNorm and its leaky ReLU in FRONT of the
// convolution, in[r][p] <- act(in[r][p] * pre_scale[p] + pre_shift[p]).  The tcgen05 kernels that split their input
// rows before the launch apply it in that pass; for every other kernel it is applied into a scratch copy of the
// input first (what the stand-alone operator would have done).
int conv_forward_dispatch(const float *in, long long rows_in, float *out, long long rows_out, const float *weight,
                          const float *bias, const int *table, int K, int cin, int cout, int groups, int precision,
                          int *flags, cudaStream_t stream, const float *bn_scale, const float *bn_shift, float leak,
                          const float *pre_scale, const float *pre_shift, float pre_leak, const float *in_b,
                          int planes_a) {
  bool fused = true;  // did the kernel apply the optional BatchNorm epilogue itself?
  // TF32X3 is the fp32-accuracy mode: each shape runs whichever fp32-class kernel is fastest.
  // With 32 or 64 output planes (and first layers) that is the row-stationary kernel of
  // conv_rows.cu on the warp-level tensor path; other narrow shapes take the pipelined kernel of
  // conv_pipe.cu with three tf32 mma.sync passes on compacted 16-pair tiles.  The tcgen05 tile costs
  // the same per 8 input planes and 256 rows whatever Cout and however few of the rows have a
  // rule, so it only pays from SCN_X3_MIN_COUT output planes on.
  const int x3_min_cout = getenv("SCN_X3_MIN_COUT") ? atoi(getenv("SCN_X3_MIN_COUT")) : 65;
  const bool narrow_x3 = precision == SCN_PRECISION_TF32X3 && cout < x3_min_cout;
  // The persistent kernel runs one CTA per SM over whole tiles; with fewer tiles than SMs the
  // per-tile kernel is used instead, which splits a tile's filter offsets over several CTAs.
  const bool force_persistent = getenv("SCN_TC_PERSISTENT") && atoi(getenv("SCN_TC_PERSISTENT")) != 0;
  const long long wide_min_rows = getenv("SCN_WIDE_MIN_ROWS") ? atoll(getenv("SCN_WIDE_MIN_ROWS")) : 148 * 256;
  const bool few_tiles = rows_out <= wide_min_rows && !force_persistent;
  const bool use_rows = !(getenv("SCN_X3_ROWS") && atoi(getenv("SCN_X3_ROWS")) == 0);
  const bool rows_thin = narrow_x3 && use_rows && conv_rows_thin_supported(out, bias, cin, cout, groups);
  // the row-stationary kernel also has the single-pass modes (32 / 64 output planes)
  const bool rows = (narrow_x3 || precision == SCN_PRECISION_TF32 || precision == SCN_PRECISION_BF16) && use_rows &&
                    conv_rows_supported(in, out, weight, bias, K, cin, cout, groups);
  const bool pipe_mma = narrow_x3 && cin % 8 == 0 && conv_pipe_supported(in, out, weight, bias, K, cin, cout);
  // a narrow shape none of the three takes (more than 32 filter offsets, groups ...) goes on to tcgen05
  const bool tensor = precision != SCN_PRECISION_FP32 && !(rows_thin || rows || pipe_mma);
  const bool to_wide = tensor && !few_tiles && conv_wide_supported(K, cin, cout, groups, precision, rows_in);
  const bool to_tma = tensor && !to_wide && !few_tiles && conv_tma_supported(K, cin, cout, groups, precision, rows_in);
  const bool to_tc = tensor && !to_wide && !to_tma && conv_tc_supported(cin, cout, groups, precision);
  float *pre_copy = nullptr;
  const bool splits = to_wide || (to_tc && conv_tc_splits_rows(precision, cin, rows_in, rows_out));
  if (in_b && rows_in > 0 && !splits) {
    // a joined input (in_b: the input is [in (planes_a) | in_b]; groups == 1) for a kernel without a split pass:
    // the concatenation, normalised if a BatchNorm comes with it, is written to a scratch matrix first
    SCN_REQUIRE(groups == 1 && planes_a % 4 == 0 && (cin - planes_a) % 4 == 0 && (uintptr_t)in % 16 == 0 &&
                    (uintptr_t)in_b % 16 == 0,
                SCN_ERR_UNSUPPORTED, "joined input: plane counts must be multiples of four");
    const long long total = rows_in * (long long)cin;
    SCN_TRY(device_alloc((void **)&pre_copy, sizeof(float) * (size_t)total, stream));
    SCN_LAUNCH(k_scale_shift_act_join_to, (unsigned)std::min<long long>(ceil_div(total / 4, 256), 148 * 16), 256, 0, stream,
               in, planes_a, in_b, cin - planes_a, pre_copy, rows_in, pre_scale, pre_shift, pre_leak);
    in = pre_copy;
    in_b = nullptr;
    pre_scale = pre_shift = nullptr;
  }
  if (pre_scale && rows_in > 0 && !splits) {
    const long long total = rows_in * (long long)cin * groups;
    SCN_TRY(device_alloc((void **)&pre_copy, sizeof(float) * (size_t)total, stream));
    const int vec = (cin * groups) % 4 == 0 && (uintptr_t)in % 16 == 0 && (uintptr_t)pre_scale % 16 == 0 &&
                    (uintptr_t)pre_shift % 16 == 0;
    SCN_LAUNCH(k_scale_shift_act_to, (unsigned)std::min<long long>(ceil_div(total / (vec ? 4 : 1), 256), 148 * 16), 256, 0,
               stream, in, pre_copy, rows_in, cin * groups, pre_scale, pre_shift, pre_leak, vec);
    in = pre_copy;
    pre_scale = pre_shift = nullptr;
  }
  const int status = [&]() -> int {
  if (rows_thin) {
    SCN_TRY(conv_forward_rows_thin(in, rows_in, out, rows_out, weight, bias, bn_scale, bn_shift, leak, table, K, cin,
                                   cout, flags, stream));
    g_last_kernel = SCN_KERNEL_CONV_ROWS;
  } else if (rows) {
    SCN_TRY(conv_forward_rows(in, rows_in, out, rows_out, weight, bias, bn_scale, bn_shift, leak, table, K, cin, cout,
                              precision, flags, stream));
    g_last_kernel = SCN_KERNEL_CONV_ROWS;
  } else if (pipe_mma) {
    SCN_TRY(conv_forward_pipe(in, rows_in, out, rows_out, weight, bias, table, K, cin, cout, groups, 1,
                              flags, stream));
    g_last_kernel = SCN_KERNEL_CONV_PIPE_MMA;
    fused = false;
  } else if (to_wide) {
    SCN_TRY(conv_forward_wide(in, rows_in, out, rows_out, weight, bias, bn_scale, bn_shift, bn_scale ? leak : 1.f, table,
                              K, cin, cout, precision, flags, stream, pre_scale, pre_shift, pre_leak, in_b, planes_a));
    g_last_kernel = SCN_KERNEL_CONV_WIDE;
  } else if (to_tma) {
    SCN_TRY(conv_forward_tma(in, rows_in, out, rows_out, weight, bias, table, K, cin, cout,
                             precision, flags, stream));
    g_last_kernel = SCN_KERNEL_CONV_TC_PERSISTENT;
    fused = false;
  } else if (to_tc) {
    SCN_TRY(conv_forward_tc(in, rows_in, out, rows_out, weight, bias, bn_scale, bn_shift, leak, table, K, cin, cout,
                            precision, flags, stream, pre_scale, pre_shift, pre_leak, in_b, planes_a));
    g_last_kernel = SCN_KERNEL_CONV_TC;
  } else {
    SCN_TRY(conv_forward_simt(in, rows_in, out, rows_out, weight, bias, table, K, cin, cout,
                              groups, flags, stream));
    g_last_kernel = SCN_KERNEL_CONV_SIMT;
    fused = false;
  }
  return SCN_OK;
  }();
  device_free(pre_copy, stream);
  SCN_TRY(status);
  if (bn_scale && !fused && rows_out > 0) {
    const long long total = rows_out * (long long)cout * groups;
    SCN_LAUNCH(k_scale_shift_act, (unsigned)std::min<long long>(ceil_div(total, 256), 148 * 16), 256, 0, stream, out,
               rows_out, cout * groups, bn_scale, bn_shift, leak);
    SCN_CUDA_CHECK(cudaGetLastError());
  }
  return SCN_OK;
}

// `disjoint` (only with `transposed`): every output row has exactly one rule (filter = stride).
// `disjoint` additionally promises that every output row HAS a rule: the caller clears it when the
// fine grid may hold rows that are in no map (earlier duplicates under input mode 0), whose output
// the scatter form would leave unwritten while the gather form and the reference give them the bias.
static int run_conv(scn_metadata *md, Rulebook &rb, bool transposed, const float *in, float *out,
                    const float *weight, const float *bias, int n_in_planes, int n_out_planes, int groups,
                    int precision, cudaStream_t stream, double *macs, bool disjoint = false,
                    const float *bn_scale = nullptr, const float *bn_shift = nullptr, float leak = 1.f,
                    const float *pre_scale = nullptr, const float *pre_shift = nullptr, float pre_leak = 1.f,
                    const float *in_b = nullptr, int planes_a = 0) {
  SCN_REQUIRE(!bn_scale == !bn_shift && !pre_scale == !pre_shift, SCN_ERR_BAD_ARG,
              "scale and shift of a fused BatchNorm come together");
  SCN_REQUIRE(groups >= 1 && n_in_planes >= 1 && n_out_planes >= 1 && n_in_planes % groups == 0 &&
                  n_out_planes % groups == 0,
              SCN_ERR_BAD_ARG, "planes %d -> %d not divisible into %d groups", n_in_planes, n_out_planes, groups);
  SCN_REQUIRE(precision >= SCN_PRECISION_FP32 && precision <= SCN_PRECISION_TF32X3, SCN_ERR_BAD_ARG,
              "unknown precision %d", precision);
  SCN_REQUIRE(weight, SCN_ERR_BAD_ARG, "null weight");
  int cin = n_in_planes / groups, cout = n_out_planes / groups;
  long long rows_in = transposed ? rb.n_out : rb.n_in;
  long long rows_out = transposed ? rb.n_in : rb.n_out;
  const int *table = rb.nbr;
  // the transposed layer with one rule per output row runs from its input side, on the table as built
  const bool scatter = transposed && disjoint && precision == SCN_PRECISION_TF32X3 && rows_in > 0 &&
                       !(getenv("SCN_X3_ROWS") && atoi(getenv("SCN_X3_ROWS")) == 0) &&
                       !(getenv("SCN_ROWS_SCATTER") && atoi(getenv("SCN_ROWS_SCATTER")) == 0) &&
                       conv_rows_supported(in, out, weight, bias, rb.n_offsets, cin, cout, groups);
  if (transposed && !scatter) {
    SCN_TRY(rulebook_transposed(rb, stream));
    table = rb.tnbr;
  }
  if (rows_out > 0) {
    SCN_REQUIRE(out && (in || rows_in == 0), SCN_ERR_BAD_ARG, "null features");
    if (!md->flags_dev) {
      SCN_TRY(device_alloc((void **)&md->flags_dev, sizeof(int), stream));
      SCN_CUDA_CHECK(cudaMemsetAsync(md->flags_dev, 0, sizeof(int), stream));
    }
  }
  if (rows_out > 0 && scatter) {
    SCN_TRY(conv_forward_rows_scatter(in, rows_in, out, rows_out, weight, bias, bn_scale, bn_shift, leak, rb.nbr,
                                      rb.n_offsets, cin, cout, md->flags_dev, stream));
    g_last_kernel = SCN_KERNEL_CONV_ROWS;
  } else if (rows_out > 0) {
    SCN_TRY(conv_forward_dispatch(in, rows_in, out, rows_out, weight, bias, table, rb.n_offsets, cin, cout, groups,
                                  precision, md->flags_dev, stream, bn_scale, bn_shift, leak, pre_scale, pre_shift,
                                  pre_leak, in_b, planes_a));
  }
  if (macs) {  // the reference's return value: rules x ip x op x groups (CPU/Convolution.cpp:141)
    if (g_deferred_counts.load()) {
      // do not wait for the rule totals here: -(ip x op x groups) and a ticket for the total
      SCN_TRY(rulebook_counts_async(rb, stream));
      if (rb.total_rules < 0) {
        count_ticket_release(md->last_ticket);
        md->last_ticket = rb.ticket;
        rb.ticket->refs.fetch_add(1);
        *macs = -(double)cin * cout * groups;
        return SCN_OK;
      }
    } else {
      SCN_TRY(rulebook_counts(rb, stream));
    }
    *macs = (double)rb.total_rules * cin * cout * groups;
  }
  return SCN_OK;
}
}  // namespace scn

using namespace scn;

extern "C" {

int scn_last_conv_kernel(void) { return g_last_kernel; }

int scn_set_weight_token(uint64_t token) {
  g_weight_token = token;
  return SCN_OK;
}

int scn_release_weight_token(uint64_t token, void *stream) {
  if (token == 0) return SCN_OK;
  int current = -1;
  cudaGetDevice(&current);
  std::lock_guard<std::mutex> lock(g_weight_mu);
  for (auto it = g_weight_images.begin(); it != g_weight_images.end();) {
    if (it->first.token == token) {
      if (it->first.device != current) cudaSetDevice(it->first.device);
      device_free(it->second, it->first.device == current ? (cudaStream_t)stream : nullptr);
      if (it->first.device != current) cudaSetDevice(current);
      it = g_weight_images.erase(it);
    } else {
      ++it;
    }
  }
  return SCN_OK;
}

int scn_set_backward_precision(int precision) {
  SCN_REQUIRE(precision >= SCN_PRECISION_FP32 && precision <= SCN_PRECISION_TF32X3, SCN_ERR_BAD_ARG,
              "unknown precision %d", precision);
  g_backward_precision.store(precision);
  return SCN_OK;
}

int scn_set_deferred_counts(int on) {
  g_deferred_counts.store(on ? 1 : 0);
  return SCN_OK;
}

int scn_md_take_count_ticket(scn_metadata *md, void **ticket) {
  SCN_REQUIRE(md && ticket, SCN_ERR_BAD_ARG, "null argument");
  *ticket = md->last_ticket;  // the reference held for the caller moves to the caller
  md->last_ticket = nullptr;
  return SCN_OK;
}

int scn_count_ticket_total(void *ticket, int64_t *total) {
  SCN_REQUIRE(ticket && total, SCN_ERR_BAD_ARG, "null argument");
  long long t = 0;
  SCN_TRY(count_ticket_total((CountTicket *)ticket, &t));
  *total = t;
  return SCN_OK;
}

int scn_count_ticket_release(void *ticket) {
  count_ticket_release((CountTicket *)ticket);
  return SCN_OK;
}

int scn_submanifold_convolution_forward(scn_metadata *md, const int64_t *spatial_size,
                                        const int64_t *filter_size, const float *in_features,
                                        float *out_features, const float *weight, const float *bias,
                                        int n_in_planes, int n_out_planes, int groups, int precision,
                                        void *stream_, double *macs) {
  cudaStream_t stream = (cudaStream_t)stream_;
  SCN_REQUIRE(md && spatial_size && filter_size, SCN_ERR_BAD_ARG, "null argument");
  Rulebook *rb = nullptr;
  SCN_TRY(get_submanifold_rulebook(md, spatial_size, filter_size, stream, &rb));
  return run_conv(md, *rb, false, in_features, out_features, weight, bias, n_in_planes, n_out_planes,
                  groups, precision, stream, macs);
}

int scn_convolution_forward(scn_metadata *md, const int64_t *input_size, const int64_t *output_size,
                            const int64_t *filter_size, const int64_t *filter_stride,
                            const float *in_features, float *out_features, const float *weight,
                            const float *bias, int n_in_planes, int n_out_planes, int groups,
                            int precision, void *stream_, double *macs) {
  cudaStream_t stream = (cudaStream_t)stream_;
  SCN_REQUIRE(md && input_size && output_size && filter_size && filter_stride, SCN_ERR_BAD_ARG, "null argument");
  Rulebook *rb = nullptr;
  SCN_TRY(get_strided_rulebook(md, input_size, output_size, filter_size, filter_stride, stream, &rb));
  return run_conv(md, *rb, false, in_features, out_features, weight, bias, n_in_planes, n_out_planes,
                  groups, precision, stream, macs);
}

int scn_deconvolution_forward(scn_metadata *md, const int64_t *input_size, const int64_t *output_size,
                              const int64_t *filter_size, const int64_t *filter_stride,
                              const float *in_features, float *out_features, const float *weight,
                              const float *bias, int n_in_planes, int n_out_planes, int groups,
                              int precision, void *stream_, double *macs) {
  cudaStream_t stream = (cudaStream_t)stream_;
  SCN_REQUIRE(md && input_size && output_size && filter_size && filter_stride, SCN_ERR_BAD_ARG, "null argument");
  Rulebook *rb = nullptr;
  // the rulebook of the matching Convolution: fine (this op's output) -> coarse (this op's input)
  SCN_TRY(get_strided_rulebook(md, output_size, input_size, filter_size, filter_stride, stream, &rb));
  bool disjoint = true;  // filter = stride: the children of different coarse sites and offsets never coincide
  for (int d = 0; d < md->dim; ++d) disjoint &= filter_size[d] == filter_stride[d];
  const Grid *fine = find_grid(md, output_size);
  disjoint &= fine && !fine->may_have_blank_rows;
  return run_conv(md, *rb, true, in_features, out_features, weight, bias, n_in_planes, n_out_planes,
                  groups, precision, stream, macs, disjoint);
}

/* ---- convolutions with the eval-mode BatchNorm (+ leaky ReLU) that follows them applied in the store ---- */

int scn_batchnorm_fold(const float *running_mean, const float *running_var, const float *weight, const float *bias,
                       double eps, int n_planes, float *scale, float *shift, void *stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  SCN_REQUIRE(running_mean && running_var && scale && shift && n_planes >= 1, SCN_ERR_BAD_ARG, "null argument");
  SCN_LAUNCH(k_bn_fold, (unsigned)ceil_div(n_planes, 128), 128, 0, stream, running_mean, running_var, weight, bias,
             (float)eps, n_planes, scale, shift);
  SCN_CUDA_CHECK(cudaGetLastError());
  return SCN_OK;
}

int scn_submanifold_convolution_bn_forward(scn_metadata *md, const int64_t *spatial_size, const int64_t *filter_size,
                                           const float *in_features, float *out_features, const float *weight,
                                           const float *bias, const float *bn_scale, const float *bn_shift,
                                           double leakiness, int n_in_planes, int n_out_planes, int groups,
                                           int precision, void *stream_, double *macs) {
  cudaStream_t stream = (cudaStream_t)stream_;
  SCN_REQUIRE(md && spatial_size && filter_size && bn_scale && bn_shift, SCN_ERR_BAD_ARG, "null argument");
  Rulebook *rb = nullptr;
  SCN_TRY(get_submanifold_rulebook(md, spatial_size, filter_size, stream, &rb));
  return run_conv(md, *rb, false, in_features, out_features, weight, bias, n_in_planes, n_out_planes, groups,
                  precision, stream, macs, false, bn_scale, bn_shift, (float)leakiness);
}

int scn_convolution_bn_forward(scn_metadata *md, const int64_t *input_size, const int64_t *output_size,
                               const int64_t *filter_size, const int64_t *filter_stride, const float *in_features,
                               float *out_features, const float *weight, const float *bias, const float *bn_scale,
                               const float *bn_shift, double leakiness, int n_in_planes, int n_out_planes, int groups,
                               int precision, void *stream_, double *macs) {
  cudaStream_t stream = (cudaStream_t)stream_;
  SCN_REQUIRE(md && input_size && output_size && filter_size && filter_stride && bn_scale && bn_shift, SCN_ERR_BAD_ARG,
              "null argument");
  Rulebook *rb = nullptr;
  SCN_TRY(get_strided_rulebook(md, input_size, output_size, filter_size, filter_stride, stream, &rb));
  return run_conv(md, *rb, false, in_features, out_features, weight, bias, n_in_planes, n_out_planes, groups,
                  precision, stream, macs, false, bn_scale, bn_shift, (float)leakiness);
}

int scn_submanifold_convolution_joined_forward(scn_metadata *md, const int64_t *spatial_size, const int64_t *filter_size,
                                               const float *in_a, int planes_a, const float *in_b, int planes_b,
                                               float *out_features, const float *weight, const float *bias,
                                               const float *pre_scale, const float *pre_shift, double pre_leakiness,
                                               const float *bn_scale, const float *bn_shift, double leakiness,
                                               int n_out_planes, int precision, void *stream_, double *macs) {
  cudaStream_t stream = (cudaStream_t)stream_;
  SCN_REQUIRE(md && spatial_size && filter_size, SCN_ERR_BAD_ARG, "null argument");
  SCN_REQUIRE(planes_a >= 8 && planes_b >= 4 && planes_a % 8 == 0 && planes_b % 4 == 0, SCN_ERR_UNSUPPORTED,
              "joined input: %d + %d planes unsupported (a multiple of eight, then a multiple of four)", planes_a, planes_b);
  Rulebook *rb = nullptr;
  SCN_TRY(get_submanifold_rulebook(md, spatial_size, filter_size, stream, &rb));
  SCN_REQUIRE(rb->n_in == 0 || (in_a && in_b), SCN_ERR_BAD_ARG, "null features");
  return run_conv(md, *rb, false, in_a, out_features, weight, bias, planes_a + planes_b, n_out_planes, 1, precision,
                  stream, macs, false, bn_scale, bn_shift, (float)leakiness, pre_scale, pre_shift, (float)pre_leakiness,
                  in_b, planes_a);
}

int scn_convolution_bn_bn_forward(scn_metadata *md, const int64_t *input_size, const int64_t *output_size,
                                  const int64_t *filter_size, const int64_t *filter_stride, const float *in_features,
                                  float *out_features, const float *weight, const float *bias, const float *pre_scale,
                                  const float *pre_shift, double pre_leakiness, const float *bn_scale,
                                  const float *bn_shift, double leakiness, int n_in_planes, int n_out_planes, int groups,
                                  int precision, void *stream_, double *macs) {
  cudaStream_t stream = (cudaStream_t)stream_;
  SCN_REQUIRE(md && input_size && output_size && filter_size && filter_stride && pre_scale && pre_shift, SCN_ERR_BAD_ARG,
              "null argument");
  Rulebook *rb = nullptr;
  SCN_TRY(get_strided_rulebook(md, input_size, output_size, filter_size, filter_stride, stream, &rb));
  return run_conv(md, *rb, false, in_features, out_features, weight, bias, n_in_planes, n_out_planes, groups,
                  precision, stream, macs, false, bn_scale, bn_shift, (float)leakiness, pre_scale, pre_shift,
                  (float)pre_leakiness);
}

int scn_deconvolution_bn_forward(scn_metadata *md, const int64_t *input_size, const int64_t *output_size,
                                 const int64_t *filter_size, const int64_t *filter_stride, const float *in_features,
                                 float *out_features, const float *weight, const float *bias, const float *bn_scale,
                                 const float *bn_shift, double leakiness, int n_in_planes, int n_out_planes,
                                 int groups, int precision, void *stream_, double *macs) {
  cudaStream_t stream = (cudaStream_t)stream_;
  SCN_REQUIRE(md && input_size && output_size && filter_size && filter_stride && bn_scale && bn_shift, SCN_ERR_BAD_ARG,
              "null argument");
  Rulebook *rb = nullptr;
  SCN_TRY(get_strided_rulebook(md, output_size, input_size, filter_size, filter_stride, stream, &rb));
  bool disjoint = true;
  for (int d = 0; d < md->dim; ++d) disjoint &= filter_size[d] == filter_stride[d];
  const Grid *fine = find_grid(md, output_size);
  disjoint &= fine && !fine->may_have_blank_rows;
  return run_conv(md, *rb, true, in_features, out_features, weight, bias, n_in_planes, n_out_planes, groups,
                  precision, stream, macs, disjoint, bn_scale, bn_shift, (float)leakiness);
}
}
