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
#include <stdlib.h>

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
  float acc[kPRows][NPL * 8 + 4];            // tile accumulator; +4: the rows a warp folds into spread over the banks
  float a[kPStages][kPCap][kPAStride];       // gathered input rows of a step: [pair][plane]
  float w[kPStages][kPChunk][NPL * 8];       // W[k][c0 .. c0+32][n0 .. n0+BN], column n of row r at n ^ ((r & 3) << 3)
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
__device__ __forceinline__ void pipe_chunk(float (&acc)[4][NPL], const float *a_thr, const float *w_row0, int col0,
                                           int kmax) {
  constexpr int WS = NPL * 8;
#pragma unroll 2
  for (int kk = 0; kk < kmax; kk += 4) {
    float4 w[4][NPL / 4];
#pragma unroll
    for (int q = 0; q < 4; ++q)
#pragma unroll
      for (int h = 0; h < NPL / 4; ++h)  // columns of row r are stored at col ^ ((r & 3) << 3); kk % 4 == 0
        w[q][h] = *reinterpret_cast<const float4 *>(w_row0 + (kk + q) * WS + ((h * 32 + col0) ^ (q << 3)));
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

// ---- warp-level tensor path (three tf32 passes) on the same pipeline ---------------------------
// D(16x8, fp32) += A(16x8, tf32, row) * B(8x8, tf32, col); lane = 4 g + t holds
//   a0 A[g][t] a1 A[g+8][t] a2 A[g][t+4] a3 A[g+8][t+4], b0 B[t][g] b1 B[t+4][g],
//   d0 D[g][2t] d1 D[g][2t+1] d2 D[g+8][2t] d3 D[g+8][2t+1].
__device__ __forceinline__ void mma_m16n8k8_tf32(float (&d)[4], const unsigned (&a)[4], const unsigned (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ void split_tf32(float x, unsigned &hi, unsigned &lo) {
  hi = __float_as_uint(x) & 0xFFFFE000u;
  lo = __float_as_uint(x - __uint_as_float(hi));
}

// One chunk: MT tiles of 16 pairs x the warp's NT tiles of 8 planes (planes n_w .. n_w + 8 NT).
template <int MT, int NT>
__device__ __forceinline__ void pipe_chunk_mma(float (&d)[4][NT][4], const float *a_stage, const float *w_row0,
                                               int WS, int n_w, int kmax, int lane) {
  const int g = lane >> 2, t = lane & 3;
  // a whole 32-plane chunk is the common case: unrolled, so that the loads of the next 8 planes
  // are issued ahead of this block's instructions
#pragma unroll
  for (int k0 = 0; k0 < kPChunk; k0 += 8) {
    if (k0 >= kmax) break;
    unsigned bh[NT][2], bl[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int col = (n_w + nt * 8 + g) ^ (t << 3);  // rows k0+t and k0+t+4 share (r & 3) = t
      split_tf32(w_row0[(k0 + t) * WS + col], bh[nt][0], bl[nt][0]);
      split_tf32(w_row0[(k0 + t + 4) * WS + col], bh[nt][1], bl[nt][1]);
    }
    // all fragments first, then the three passes tile by tile: consecutive instructions write
    // different accumulators
    unsigned ah[MT][4], al[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      const float *ap = a_stage + (mt * 16 + g) * kPAStride + k0 + t;
      split_tf32(ap[0], ah[mt][0], al[mt][0]);
      split_tf32(ap[8 * kPAStride], ah[mt][1], al[mt][1]);
      split_tf32(ap[4], ah[mt][2], al[mt][2]);
      split_tf32(ap[8 * kPAStride + 4], ah[mt][3], al[mt][3]);
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) mma_m16n8k8_tf32(d[mt][nt], al[mt], bh[nt]);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) mma_m16n8k8_tf32(d[mt][nt], ah[mt], bl[nt]);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) mma_m16n8k8_tf32(d[mt][nt], ah[mt], bh[nt]);
  }
}

template <int NPL, bool MMA>
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
  for (int i = tid; i < kPRows * (BN + 4) / 4; i += kPThreads)
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
        cp_async16(smem_u32(&S.w[stage][r][w_cc ^ ((r & 3) << 3)]), ok ? wk + (long long)i * RSTEP * cout : weight, ok ? 16u : 0u);
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

  float acc[4][NPL];          // FMA micro-tile
  float dm[4][BN / 32][4];    // MMA fragments
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
    if (!MMA) {
      if (c == 0) {
  #pragma unroll
        for (int j = 0; j < 4; ++j)
  #pragma unroll
          for (int e = 0; e < NPL; ++e) acc[j][e] = 0.f;
      }
      const float *a_thr = &S.a[stage][ty][0];
      const float *w_row0 = &S.w[stage][0][0];
      switch (pm) {
        case 1: pipe_chunk<1, NPL>(acc, a_thr, w_row0, tx * 4, kmax); break;
        case 2: pipe_chunk<2, NPL>(acc, a_thr, w_row0, tx * 4, kmax); break;
        case 3: pipe_chunk<3, NPL>(acc, a_thr, w_row0, tx * 4, kmax); break;
        default: pipe_chunk<4, NPL>(acc, a_thr, w_row0, tx * 4, kmax); break;
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
    } else {
      constexpr int NT = BN / 32;
      if (c == 0) {
#pragma unroll
        for (int mt = 0; mt < 4; ++mt)
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) dm[mt][nt][0] = dm[mt][nt][1] = dm[mt][nt][2] = dm[mt][nt][3] = 0.f;
      }
      const float *a_stage = &S.a[stage][0][0];
      const float *w_row0 = &S.w[stage][0][0];
      const int n_w = warp * NT * 8;
      switch (pm) {
        case 1: pipe_chunk_mma<1, NT>(dm, a_stage, w_row0, BN, n_w, kmax, lane); break;
        case 2: pipe_chunk_mma<2, NT>(dm, a_stage, w_row0, BN, n_w, kmax, lane); break;
        case 3: pipe_chunk_mma<3, NT>(dm, a_stage, w_row0, BN, n_w, kmax, lane); break;
        default: pipe_chunk_mma<4, NT>(dm, a_stage, w_row0, BN, n_w, kmax, lane); break;
      }
      if (c == nch - 1) {
        const unsigned char *pr = &prow[k][base];
        const int gq = lane >> 2, t2 = (lane & 3) * 2;
#pragma unroll
        for (int mt = 0; mt < 4; ++mt) {
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const int p = mt * 16 + half * 8 + gq;
            if (mt < pm && p < P) {
              float *dst = &S.acc[pr[p]][n_w + t2];
#pragma unroll
              for (int nt = 0; nt < NT; ++nt) {
                float2 v = *reinterpret_cast<float2 *>(dst + nt * 8);
                v.x += dm[mt][nt][half * 2 + 0];
                v.y += dm[mt][nt][half * 2 + 1];
                *reinterpret_cast<float2 *>(dst + nt * 8) = v;
              }
            }
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

template <int NPL, bool MMA>
static int launch_pipe(const float *in, int ld_in, long long n_in, float *out, int ld_out, long long n_out,
                       const float *weight, const float *bias, const int *table, int K, int cin, int cout,
                       int groups, int *flags, cudaStream_t stream) {
  static int configured[64] = {0};
  int dev = 0;
  SCN_CUDA_CHECK(cudaGetDevice(&dev));
  const size_t smem = pipe_smem_bytes(NPL, K);
  if (dev >= 64 || configured[dev] < (int)smem) {
    SCN_CUDA_CHECK(cudaFuncSetAttribute(k_conv_pipe<NPL, MMA>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (dev < 64) configured[dev] = (int)smem;
  }
  dim3 grid((unsigned)ceil_div(n_out, (long long)kPRows), (unsigned)ceil_div(cout, NPL * 8), (unsigned)groups);
  auto kernel = k_conv_pipe<NPL, MMA>;
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
// three_pass_mma: the arithmetic runs as three tf32 mma.sync passes (fp32-class accuracy) instead of fp32 FMA.
int conv_forward_pipe(const float *in, long long n_in, float *out, long long n_out, const float *weight,
                      const float *bias, const int *table, int K, int cin, int cout, int groups, int three_pass_mma,
                      int *flags, cudaStream_t stream) {
  if (n_out == 0) return SCN_OK;
  const int ld_in = cin * groups, ld_out = cout * groups;
  const bool mma = three_pass_mma && cin % 8 == 0;
  if (cout <= 32)
    return mma ? launch_pipe<4, true>(in, ld_in, n_in, out, ld_out, n_out, weight, bias, table, K, cin, cout, groups, flags, stream)
               : launch_pipe<4, false>(in, ld_in, n_in, out, ld_out, n_out, weight, bias, table, K, cin, cout, groups, flags, stream);
  return mma ? launch_pipe<8, true>(in, ld_in, n_in, out, ld_out, n_out, weight, bias, table, K, cin, cout, groups, flags, stream)
             : launch_pipe<8, false>(in, ld_in, n_in, out, ld_out, n_out, weight, bias, table, K, cin, cout, groups, flags, stream);
}

}  // namespace scn
