// fp32 sparse convolution, output stationary, software-pipelined.
//
// Same arithmetic and the same dense rulebook as k_conv_simt (conv_simt.cu; the reference's
// per-offset gather / GEMM / scatter-add is CPU/Convolution.cpp:137-148 and
// CUDA/Convolution.cu:57-233,618-642).  A CTA of 128 threads owns 128 output rows for the
// whole filter:
//
//   prologue  the four warps compact the tile's rules of every filter offset (ballots over
//             coalesced reads of the dense rulebook) into per-offset pair lists in shared memory;
//             offsets without a rule in the tile disappear from the step list
//   steps     one step = (offset, batch of <= 64 pairs, 32-plane chunk), listed once per tile.  The
//             input rows of the batch and the W[k] slab of the chunk travel with 16-byte cp.async
//             into a ring of three stages, two steps ahead of the arithmetic; there is ONE block
//             barrier per step and no per-step bookkeeping beyond two counters
//   compute   thread = (pair group 0..15) x (plane group 0..7): PM pairs x NPL planes in registers,
//             PM = ceil(pairs / 16) chosen per step, so every thread works whatever the fill of
//             the tile; input values are broadcast float4 reads, W values float4 reads
//   fold      after the last chunk the micro-tile is added into the tile accumulator in shared
//             memory (one rule per (offset, output row): no two threads share a row in a step)
//
// Output rows are written once, bias added.  Needs 16-byte aligned rows (cin, cout multiples of
// 4) and at most 32 filter offsets; conv_simt.cu keeps the general kernel.
#include <algorithm>

#include "metadata.cuh"
#include "tc_ptx.cuh"

namespace scn {

constexpr int kPRows = 128;              // output rows per CTA
constexpr int kPThreads = 128;
constexpr int kPCap = 64;                // pairs per step
constexpr int kPChunk = 32;              // input planes per step
constexpr int kPAStride = kPChunk + 4;   // stage row stride (floats): 4 pair groups of a warp hit 4 bank quads
#ifndef SCN_PIPE_STAGES
#define SCN_PIPE_STAGES 3
#endif
constexpr int kPStages = SCN_PIPE_STAGES;  // ring of stages: copies run kPStages - 1 steps ahead of the arithmetic
constexpr int kPMaxK = 32;
constexpr int kPMaxGroups = 2 * kPMaxK;  // (offset, batch of <= 64 pairs) groups of a tile

template <int NPL>
struct PipeSmem {
  float acc[kPRows][NPL * 8];                // tile accumulator
  float a[kPStages][kPCap][kPAStride];       // gathered input rows of a step: [pair][plane]
  float w[kPStages][kPChunk][NPL * 8];       // W[k][c0 .. c0+32][n0 .. n0+BN]
  int cnt[kPMaxK];                           // pairs per offset
  int groups[kPMaxGroups];                   // offset | first pair << 8 | pairs << 16, in execution order
  int n_groups;
  // followed by: int pin[K][128] (pair -> input row), unsigned char prow[K][128] (pair -> local output row)
};

static size_t pipe_smem_bytes(int npl, int K) {
  size_t fixed = npl == 4 ? sizeof(PipeSmem<4>) : sizeof(PipeSmem<8>);
  return fixed + (size_t)K * kPRows * 5;
}

template <int PM, int NPL>
__device__ __forceinline__ void pipe_chunk(float (&acc)[4][NPL], const float *a_thr, const float *w_thr, int kmax) {
  constexpr int WS = NPL * 8;
#pragma unroll 2
  for (int kk = 0; kk < kmax; kk += 4) {
    float4 w[4][NPL / 4];
#pragma unroll
    for (int q = 0; q < 4; ++q)
#pragma unroll
      for (int h = 0; h < NPL / 4; ++h) w[q][h] = *reinterpret_cast<const float4 *>(w_thr + (kk + q) * WS + h * 32);
#pragma unroll
    for (int j = 0; j < PM; ++j) {
      const float4 a4 = *reinterpret_cast<const float4 *>(a_thr + j * 16 * kPAStride + kk);
#pragma unroll
      for (int h = 0; h < NPL / 4; ++h) {
        float *c = &acc[j][h * 4];
        c[0] = fmaf(a4.x, w[0][h].x, c[0]);
        c[1] = fmaf(a4.x, w[0][h].y, c[1]);
        c[2] = fmaf(a4.x, w[0][h].z, c[2]);
        c[3] = fmaf(a4.x, w[0][h].w, c[3]);
        c[0] = fmaf(a4.y, w[1][h].x, c[0]);
        c[1] = fmaf(a4.y, w[1][h].y, c[1]);
        c[2] = fmaf(a4.y, w[1][h].z, c[2]);
        c[3] = fmaf(a4.y, w[1][h].w, c[3]);
        c[0] = fmaf(a4.z, w[2][h].x, c[0]);
        c[1] = fmaf(a4.z, w[2][h].y, c[1]);
        c[2] = fmaf(a4.z, w[2][h].z, c[2]);
        c[3] = fmaf(a4.z, w[2][h].w, c[3]);
        c[0] = fmaf(a4.w, w[3][h].x, c[0]);
        c[1] = fmaf(a4.w, w[3][h].y, c[1]);
        c[2] = fmaf(a4.w, w[3][h].z, c[2]);
        c[3] = fmaf(a4.w, w[3][h].w, c[3]);
      }
    }
  }
}

template <int NPL>
__global__ void __launch_bounds__(kPThreads)
k_conv_pipe(const float *__restrict__ in, int ld_in, long long n_in, float *__restrict__ out, int ld_out,
            long long n_out, const float *__restrict__ weight, long long w_offset_stride,
            long long w_group_stride, const float *__restrict__ bias, const int *__restrict__ nbr, int K,
            int cin, int cout, int *flags) {
  constexpr int BN = NPL * 8;
  constexpr unsigned kFull = 0xffffffffu;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  PipeSmem<NPL> &S = *reinterpret_cast<PipeSmem<NPL> *>(smem_raw);
  int(*pin)[kPRows] = reinterpret_cast<int(*)[kPRows]>(smem_raw + sizeof(PipeSmem<NPL>));
  unsigned char(*prow)[kPRows] =
      reinterpret_cast<unsigned char(*)[kPRows]>(smem_raw + sizeof(PipeSmem<NPL>) + (size_t)K * kPRows * 4);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tx = tid & 7, ty = tid >> 3;
  const long long row0 = (long long)blockIdx.x * kPRows;
  const int n0 = blockIdx.y * BN;
  const int g = blockIdx.z;
  in += (long long)g * cin;
  out += (long long)g * cout;
  weight += (long long)g * w_group_stride;
  if (bias) bias += (long long)g * cout;

  // ---- prologue: pair lists of every offset ---------------------------------------------------
  for (int i = tid; i < kPRows * BN / 4; i += kPThreads)
    reinterpret_cast<float4 *>(&S.acc[0][0])[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  {
    constexpr int kPer = kPMaxK / 4;  // offsets per warp
    int v[kPer][4];
#pragma unroll
    for (int u = 0; u < kPer; ++u) {
      const int k = warp + u * 4;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const long long r = row0 + i * 32 + lane;
        v[u][i] = (k < K && r < n_out) ? __ldg(nbr + (long long)k * n_out + r) : -1;
      }
    }
#pragma unroll
    for (int u = 0; u < kPer; ++u) {
      const int k = warp + u * 4;
      if (k >= K) break;
      int base = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        int idx = v[u][i];
        if (idx >= n_in) {
          atomicOr(flags, FLAG_BAD_ROW);
          idx = -1;
        }
        const unsigned m = __ballot_sync(kFull, idx >= 0);
        if (idx >= 0) {
          const int p = base + __popc(m & ((1u << lane) - 1u));
          pin[k][p] = idx;
          prow[k][p] = (unsigned char)(i * 32 + lane);
        }
        base += __popc(m);
      }
      if (lane == 0) S.cnt[k] = base;
    }
  }
  __syncthreads();

  // ---- group list: (offset with rules, batch of <= 64 pairs); lane k of warp 0 places offset k ------
  if (warp == 0) {
    const int c = lane < K ? S.cnt[lane] : 0;
    const int nb = (c + kPCap - 1) / kPCap;  // 0, 1 or 2 batches
    int incl = nb;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int o = __shfl_up_sync(kFull, incl, d);
      if (lane >= d) incl += o;
    }
    const int first = incl - nb;
    for (int b = 0; b < nb; ++b) S.groups[first + b] = lane | (b * kPCap) << 8 | min(kPCap, c - b * kPCap) << 16;
    if (lane == 31) S.n_groups = incl;
  }
  __syncthreads();

  // ---- steps: (group, 32-plane chunk), flattened; copies of step s+2 are issued during step s ------
  const int nch = (cin + kPChunk - 1) / kPChunk;
  const int n_steps = S.n_groups * nch;
  constexpr int PPR = BN / 4;               // 16-byte pieces per W row
  constexpr int RSTEP = kPThreads / PPR;    // W rows per pass of the CTA
  const int w_cc = (tid % PPR) * 4, w_r0 = tid / PPR;
  const bool w_col_ok = n0 + w_cc < cout;
  const long long w_thr = (long long)w_r0 * cout + n0 + w_cc;
  // one cp.async group per call, empty or not, so wait_group's count stays fixed
  auto issue = [&](int g, int c, int stage) {
    if (g < S.n_groups) {
      const int d = S.groups[g];
      const int k = d & 0xFF, base = (d >> 8) & 0xFF, P = d >> 16;
      const float *wk = weight + (long long)k * w_offset_stride + (long long)c * kPChunk * cout + w_thr;
      const int rows_left = cin - c * kPChunk;  // W rows of this chunk that exist
#pragma unroll
      for (int i = 0; i < kPChunk / RSTEP; ++i) {
        const int r = w_r0 + i * RSTEP;
        const bool ok = w_col_ok && r < rows_left;
        cp_async16(smem_u32(&S.w[stage][r][w_cc]), ok ? wk + (long long)i * RSTEP * cout : weight, ok ? 16u : 0u);
      }
      const int c0 = c * kPChunk + tx * 4;
      if (c0 < cin) {
        const int *pk = &pin[k][base];
        const float *col = in + c0;
#pragma unroll
        for (int i = 0; i < kPCap / 16; ++i) {
          const int p = ty + 16 * i;
          if (p < P) cp_async16(smem_u32(&S.a[stage][p][tx * 4]), col + (long long)pk[p] * ld_in, 16u);
        }
      }
    }
    cp_async_commit();
  };
  int gi = 0, ci = 0;  // next step to issue
  auto advance_issue = [&] {
    if (++ci == nch) {
      ci = 0;
      ++gi;
    }
  };
#pragma unroll
  for (int st = 0; st < kPStages - 1; ++st) {
    issue(gi, ci, st);
    advance_issue();
  }

  float acc[4][NPL];
  int stage = 0, gc = 0, c = 0;  // stage, group and chunk of the step being computed
  for (int s = 0; s < n_steps; ++s) {
    cp_async_wait<kPStages - 2>();  // all but the newest kPStages - 2 groups: the copies of step s have landed
    __syncthreads();     // ... for every thread; and the previous step is consumed
    issue(gi, ci, stage == 0 ? kPStages - 1 : stage - 1);
    advance_issue();

    const int d = S.groups[gc];
    const int k = d & 0xFF, base = (d >> 8) & 0xFF, P = d >> 16;
    const int pm = (P + 15) >> 4;
    const int kmax = min(kPChunk, cin - c * kPChunk);
    if (c == 0) {
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int e = 0; e < NPL; ++e) acc[j][e] = 0.f;
    }
    const float *a_thr = &S.a[stage][ty][0];
    const float *w_thr_s = &S.w[stage][0][tx * 4];
    switch (pm) {
      case 1: pipe_chunk<1, NPL>(acc, a_thr, w_thr_s, kmax); break;
      case 2: pipe_chunk<2, NPL>(acc, a_thr, w_thr_s, kmax); break;
      case 3: pipe_chunk<3, NPL>(acc, a_thr, w_thr_s, kmax); break;
      default: pipe_chunk<4, NPL>(acc, a_thr, w_thr_s, kmax); break;
    }
    if (c == nch - 1) {
      const unsigned char *pr = &prow[k][base];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int p = j * 16 + ty;
        if (p < P) {
          float *dst = &S.acc[pr[p]][tx * 4];
#pragma unroll
          for (int h = 0; h < NPL / 4; ++h) {
            float4 t = *reinterpret_cast<float4 *>(dst + h * 32);
            t.x += acc[j][h * 4 + 0];
            t.y += acc[j][h * 4 + 1];
            t.z += acc[j][h * 4 + 2];
            t.w += acc[j][h * 4 + 3];
            *reinterpret_cast<float4 *>(dst + h * 32) = t;
          }
        }
      }
    }
    if (++c == nch) {
      c = 0;
      ++gc;
    }
    stage = stage + 1 == kPStages ? 0 : stage + 1;
  }
  cp_async_wait<0>();
  __syncthreads();

  // ---- write the tile once ----------------------------------------------------------------------
  for (int i = tid; i < kPRows * (BN / 4); i += kPThreads) {
    const int r = i / (BN / 4), cc = (i % (BN / 4)) * 4;
    const long long row = row0 + r;
    const int n = n0 + cc;
    if (row >= n_out || n >= cout) continue;
    float4 v = *reinterpret_cast<const float4 *>(&S.acc[r][cc]);
    if (bias) {
      const float4 b = __ldg(reinterpret_cast<const float4 *>(bias + n));
      v.x += b.x;
      v.y += b.y;
      v.z += b.z;
      v.w += b.w;
    }
    *reinterpret_cast<float4 *>(out + row * ld_out + n) = v;
  }
}

template <int NPL>
static int launch_pipe(const float *in, int ld_in, long long n_in, float *out, int ld_out, long long n_out,
                       const float *weight, const float *bias, const int *table, int K, int cin, int cout,
                       int groups, int *flags, cudaStream_t stream) {
  static int configured[64] = {0};
  int dev = 0;
  SCN_CUDA_CHECK(cudaGetDevice(&dev));
  const size_t smem = pipe_smem_bytes(NPL, K);
  if (dev >= 64 || configured[dev] < (int)smem) {
    SCN_CUDA_CHECK(cudaFuncSetAttribute(k_conv_pipe<NPL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (dev < 64) configured[dev] = (int)smem;
  }
  dim3 grid((unsigned)ceil_div(n_out, (long long)kPRows), (unsigned)ceil_div(cout, NPL * 8), (unsigned)groups);
  auto kernel = k_conv_pipe<NPL>;
  SCN_LAUNCH(kernel, grid, kPThreads, smem, stream, in, ld_in, n_in, out, ld_out, n_out, weight, (long long)groups * cin * cout, (long long)cin * cout, bias, table, K, cin, cout, flags);
  SCN_CUDA_CHECK(cudaGetLastError());
  return SCN_OK;
}

bool conv_pipe_supported(const float *in, const float *out, const float *weight, const float *bias, int K, int cin,
                         int cout) {
  return K <= kPMaxK && cin % 4 == 0 && cout % 4 == 0 && (uintptr_t)in % 16 == 0 && (uintptr_t)out % 16 == 0 &&
         (uintptr_t)weight % 16 == 0 && (uintptr_t)bias % 16 == 0;
}

// out [n_out, groups*cout] = bias + sum_k in[table[k][.]] @ W[k]; cin / cout are per group.
int conv_forward_pipe(const float *in, long long n_in, float *out, long long n_out, const float *weight,
                      const float *bias, const int *table, int K, int cin, int cout, int groups, int *flags,
                      cudaStream_t stream) {
  if (n_out == 0) return SCN_OK;
  const int ld_in = cin * groups, ld_out = cout * groups;
  if (cout <= 32)
    return launch_pipe<4>(in, ld_in, n_in, out, ld_out, n_out, weight, bias, table, K, cin, cout, groups, flags, stream);
  return launch_pipe<8>(in, ld_in, n_in, out, ld_out, n_out, weight, bias, table, K, cin, cout, groups, flags, stream);
}

}  // namespace scn
