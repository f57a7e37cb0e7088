// Tensor-core sparse convolution for sm_100a: tcgen05.mma with the accumulator in TMEM.
//
// Output stationary, like the fp32 kernel: a CTA owns 256 consecutive output rows for the whole
// filter, so their accumulators live in tensor memory from the first filter offset to the last
// and every output row is written to HBM exactly once.
//
// Orientation.  A tcgen05.mma instruction costs max(56, N / 2) cycles whatever its M and kind (measured
// by scn_tc_probe_mma: 128 cycles at N = 256, a floor of 56 below N = 112), so the wide dimension has
// to be N.  Channel counts are small (32 ... 224) while rows are plentiful, hence the product is
// computed transposed:
//     D^T[Cout x 256 rows] += W[k]^T[Cout x Cin-slice] * G^T[Cin-slice x 256 rows]
// i.e. the MMA's A operand (M = 128 TMEM lanes) is the weight slab, its B operand (N = 256) the
// gathered input rows.  TMEM lane = output plane, TMEM column = row of the tile.
//
// For every filter offset k for which the tile has at least one rule, and every slice of 32
// (or 16) input planes:
//   G  = the 256 input rows named by the dense rulebook column (offset k, rows of the tile),
//        gathered with 16-byte cp.async copies straight into the tensor core's K-major
//        core-matrix layout in shared memory; a row without a rule is zero-filled by the copy
//        itself (src-size 0), so it contributes nothing;
//   W  = W[k][slice][:] -- prepared once per call in exactly its shared-memory image, so one
//        bulk copy (cp.async.bulk, completion on an mbarrier) brings the whole slab;
//   one elected thread issues slice/8 (tf32) or slice/16 (bf16) tcgen05.mma instructions of
//   shape 128 x 256 x 8|16 per 128 output planes; completion is tracked with tcgen05.commit.
// The gather runs ahead of the tensor core through a ring of shared-memory stages; producer
// warps and the MMA-issuing warp meet only on mbarriers (no block-wide sync in the main loop).
//
// Arithmetic modes:
//   TF32    one pass, operands truncated to tf32 by the tensor core            (1e-2 class)
//   BF16    operands rounded to bf16, fp32 accumulate                          (1e-2 class)
//   BF16X3  the fp32-class mode in its default form: a = h + m with h = bf16(a), m = bf16(a - h);
//           D += W_h*G_h + W_h*G_m + W_m*G_h, fp32 accumulate (what is dropped is 2^-17 of a product;
//           half the instructions of TF32X3)
//           In both bf16 modes the input rows are split once by a pass before the launch and the
//           producers copy them with cp.async (arrival on completion), as in conv_wide.cu; on the
//           smallest levels and in the allocation-free entry point they are read as fp32 and split
//           in the producers' registers instead.
//   TF32X3  the other form (SCN_X3_FORM=tf32): a = a_hi + a_lo with a_hi the tf32 truncation,
//           D += W_hi*G_hi + W_hi*G_lo + W_lo*G_hi
//
// Every wait on an mbarrier is bounded; on expiry the kernel raises FLAG_TC_TIMEOUT, stops
// issuing work, drains its own copies, frees its tensor memory and returns.
#include <cuda_bf16.h>

#include <stdlib.h>

#include <algorithm>

#include "metadata.cuh"
#include "tc_ptx.cuh"

namespace scn {


constexpr int kTcRows = 256;     // output rows per CTA = N of the MMA = TMEM columns per plane tile
constexpr int kTcPlanes = 128;   // output planes per MMA = M = TMEM lanes
constexpr int kTcThreads = 288;  // 8 producer/epilogue warps + 1 MMA warp
constexpr int kProducerThreads = 256;
constexpr int kMmaWarp = kProducerThreads / 32;
constexpr int kTcMaxOffsets = 128;

// Instruction descriptor: D fp32, A/B both tf32 or both bf16, both K-major, M = 128, N = 256.
__host__ __device__ inline unsigned instr_desc(bool bf16) {
  unsigned fmt = bf16 ? 1u : 2u;
  return (1u << 4) | (fmt << 7) | (fmt << 10) | ((unsigned)(kTcRows >> 3) << 17) | ((unsigned)(kTcPlanes >> 4) << 24);
}

// ---------------------------------------------------------------------------------------------
// weight preparation: W [K][Cin][Cout] fp32 -> per (offset, slice) the shared-memory image of the
// weight operand (Cout rows, K-major core matrices over the slice's input planes), high part
// and -- for TF32X3 -- low part.  image(k, c) at ((k * n_slices + c) * parts + part) * tile bytes.
// ---------------------------------------------------------------------------------------------
__global__ void k_prepare_weights(const float *__restrict__ w, unsigned char *__restrict__ out, int K, int cin,
                                  int cout, int kc, int mode) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  long long total = (long long)K * cin * cout;
  if (idx >= total) return;
  int n = (int)(idx % cout);
  int c = (int)((idx / cout) % cin);
  int k = (int)(idx / ((long long)cout * cin));
  float v = w[idx];
  int slice = c / kc, kk = c % kc;
  int n_slices = cin / kc;
  int parts = (mode == TC_TF32X3 || mode == TC_BF16X3) ? 2 : 1;
  if (mode == TC_BF16 || mode == TC_BF16X3) {
    size_t tile = (size_t)cout * kc * 2;
    size_t off = (size_t)(n / 8) * (kc / 8) * 128 + (size_t)(kk / 8) * 128 + (n % 8) * 16 + (kk % 8) * 2;
    unsigned char *base = out + (((size_t)k * n_slices + slice) * parts) * tile;
    const __nv_bfloat16 h = __float2bfloat16_rn(v);
    *reinterpret_cast<__nv_bfloat16 *>(base + off) = h;
    if (mode == TC_BF16X3)  // what the rounding left over, again as bf16
      *reinterpret_cast<__nv_bfloat16 *>(base + tile + off) = __float2bfloat16_rn(v - __bfloat162float(h));
  } else {
    size_t tile = (size_t)cout * kc * 4;
    size_t off = (size_t)(n / 8) * (kc / 4) * 128 + (size_t)(kk / 4) * 128 + (n % 8) * 16 + (kk % 4) * 4;
    unsigned char *base = out + (((size_t)k * n_slices + slice) * parts) * tile;
    float hi = __uint_as_float(__float_as_uint(v) & 0xFFFFE000u);
    *reinterpret_cast<float *>(base + off) = (mode == TC_TF32X3) ? hi : v;
    if (mode == TC_TF32X3) *reinterpret_cast<float *>(base + tile + off) = v - hi;
  }
}

int prepare_weights(const float *w, unsigned char *out, int K, int cin, int cout, int kc, int mode,
                    cudaStream_t stream) {
  long long total = (long long)K * cin * cout;
  SCN_LAUNCH(k_prepare_weights, (unsigned)ceil_div(total, 256), 256, 0, stream, w, out, K, cin, cout, kc, mode);
  SCN_CUDA_CHECK(cudaGetLastError());
  return SCN_OK;
}

// ---------------------------------------------------------------------------------------------
// main kernel
// ---------------------------------------------------------------------------------------------
struct TcParams {
  const float *in;
  // bf16 modes, optional: the input rows as bf16 parts (per row and 32-plane block [32 h | 32 m], made by
  // split_rows_bf16 before the launch).  The producers then only copy (cp.async, arrival on completion)
  // instead of reading fp32 rows into registers and splitting them for every output row that gathers them.
  const unsigned char *in_split;
  long long n_in;
  int ld_in;
  float *out;
  long long n_out;
  int ld_out;
  const unsigned char *wprep;
  const float *bias;
  const float *bn_scale, *bn_shift;  // optional fused eval-mode BatchNorm: out = act((acc + bias) * scale + shift)
  float leak;                        // act(y) = y > 0 ? y : y * leak (1 = identity)
  const int *nbr;  // [K][n_out]
  int K, cin, cout;
  int kc;          // input planes per step (32 or 16)
  int n_stages;
  int lookahead;   // steps the gather runs ahead of the tensor core (<= n_stages - 1)
  int tmem_cols;   // 256 per 128 output planes
  int n_split;     // CTAs per tile (grid.y): each takes a contiguous range of the filter offsets
  float *partial;  // [n_split][n_out][cout] partial sums when n_split > 1 (k_sum_partials adds them up)
  int *flags;
  int drop_arrival;  // test hook (scn_test_drop_barrier_arrival): CTA 0 leaves out one arrival on full_g[0]
};

__device__ __forceinline__ void cp_async_wait_dyn(int n) {
  switch (n) {
    case 0: cp_async_wait<0>(); break;
    case 1: cp_async_wait<1>(); break;
    case 2: cp_async_wait<2>(); break;
    default: cp_async_wait<3>(); break;
  }
}

// Warp roles.  Warps 0-7 are the gather producers (and, afterwards, the epilogue); warp 8
// owns tensor memory, streams the weight slabs and issues the MMAs.  The roles meet only on
// mbarriers:
//   full_g[s]  one arrival per producer warp: the rows of stage s are in shared memory (and
//              fenced for the async proxy)
//   full_w[s]  transaction barrier of the weight slab's bulk copy
//   empty[s]   tcgen05.commit: the MMAs that read stage s have finished
//   acc_full   tcgen05.commit after the last MMA of the tile
template <int MODE>
__global__ void __launch_bounds__(kTcThreads) k_conv_tc(TcParams P) {
  constexpr bool kBf16 = (MODE == TC_BF16 || MODE == TC_BF16X3);     // operands are bf16, converted while staging
  constexpr bool kSplit = (MODE == TC_TF32X3 || MODE == TC_BF16X3);  // two parts per operand, three products
  constexpr int kEsize = kBf16 ? 2 : 4;
  constexpr int kPerPiece = 16 / kEsize;  // elements per 16-byte piece
  constexpr int kMmaK = 32 / kEsize;      // K per instruction (32 bytes)
  // plain tf32 needs no pass over the gathered rows, so the copies themselves can signal the
  // barrier when they land (cp.async.mbarrier.arrive.noinc): the producers never wait for data
  constexpr bool kAsyncArrive = (MODE == TC_TF32);

  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const long long row0 = (long long)blockIdx.x * kTcRows;
  const int K = P.K, kc = P.kc, NS = P.n_stages, L = P.lookahead;
  const int n_slices = P.cin / kc;
  const int pieces_per_row = kc / kPerPiece;
  const unsigned g_bytes = kTcRows * kc * kEsize;
  const unsigned w_bytes = P.cout * kc * kEsize;
  const unsigned stage_bytes = (g_bytes + w_bytes) * (kSplit ? 2 : 1);
  const unsigned sbo = pieces_per_row * 128;
  const int n_mt = (P.cout + kTcPlanes - 1) / kTcPlanes;  // plane tiles of 128
  // offsets of this CTA; with n_split > 1 the tile's sum over offsets is finished by k_sum_partials
  const int k_begin = (int)(((long long)blockIdx.y * K) / P.n_split);
  const int k_end = (int)(((long long)(blockIdx.y + 1) * K) / P.n_split);
  float *const out_base = P.partial ? P.partial + (size_t)blockIdx.y * P.n_out * P.ld_out : P.out;
  const float *const bias_base = P.partial ? nullptr : P.bias;

  // shared memory carve-up: [stages][W | W_lo | G | G_lo] | idx [K][256] | control.  The weight
  // slab comes first: an MMA always reads 128 weight rows, and when Cout is not a multiple of
  // 128 the rows past the slab are whatever follows it -- the gathered rows of the same stage,
  // in bounds and harmless (they only reach TMEM lanes that are never read back).
  unsigned char *stage_base = smem;
  int *sh_idx = reinterpret_cast<int *>(smem + (size_t)NS * stage_bytes);
  unsigned long long *bars = reinterpret_cast<unsigned long long *>(sh_idx + (size_t)K * kTcRows);
  unsigned long long *full_g = bars;            // [NS]
  unsigned long long *full_w = bars + NS;       // [NS]
  unsigned long long *empty = bars + 2 * NS;    // [NS]
  unsigned long long *acc_full = bars + 3 * NS;
  int *sh_steps = reinterpret_cast<int *>(bars + 3 * NS + 1);  // [K] offsets with at least one rule
  int *sh_has = sh_steps + kTcMaxOffsets;                       // [K]
  unsigned *sh_tmem = reinterpret_cast<unsigned *>(sh_has + kTcMaxOffsets);
  int *sh_nk = reinterpret_cast<int *>(sh_tmem + 1);
  volatile int *sh_abort = sh_nk + 1;
  const unsigned w_off = 0, g_off = w_bytes * (kSplit ? 2 : 1);

  // ---- prologue: barriers, tensor memory, rulebook columns of this tile ----------------------
  if (tid == 0) {
    for (int s = 0; s < NS; ++s) {
      mbar_init(&full_g[s], (kAsyncArrive || (kBf16 && P.in_split)) ? kProducerThreads : kProducerThreads / 32);
      mbar_init(&full_w[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_full, 1);
    *sh_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kMmaWarp) tmem_alloc(sh_tmem, (unsigned)P.tmem_cols);
  for (int k = k_begin + warp; k < k_end; k += kTcThreads / 32) {
    bool any = false;
#pragma unroll
    for (int i = 0; i < kTcRows / 32; ++i) {
      int r = lane + 32 * i;
      long long row = row0 + r;
      int v = (row < P.n_out) ? __ldg(P.nbr + (long long)k * P.n_out + row) : -1;
      if (v >= P.n_in) {
        atomicOr(P.flags, FLAG_BAD_ROW);
        v = -1;
      }
      sh_idx[k * kTcRows + r] = v;
      any |= (v >= 0);
    }
    any = __any_sync(0xffffffffu, any);
    if (lane == 0) sh_has[k] = any;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (tid == 0) {
    int n = 0;
    for (int k = k_begin; k < k_end; ++k)
      if (sh_has[k]) sh_steps[n++] = k;
    *sh_nk = n;
  }
  __syncthreads();
  const unsigned tmem_base = *sh_tmem;
  const int S = *sh_nk * n_slices;

  if (warp < kMmaWarp) {
    // =================================== gather producers =====================================
    // Piece p = tid + 256 i of a stage is the 16-byte piece j of tile row r with
    //   r = (p & 7) + 8 * (p / (8 * pieces_per_row)),  j = (p >> 3) % pieces_per_row,
    // so a quarter warp fills one 128-byte core matrix and a warp reads 64 contiguous bytes of
    // 8 rows.  pieces_per_row is a power of two (2, 4 or 8): j is fixed per thread and the rows
    // step by 32 * 8 / pieces_per_row; a thread owns pieces_per_row pieces of every stage.
    const int lg = 31 - __clz(pieces_per_row);
    const int j = (tid >> 3) & (pieces_per_row - 1);
    const int r_base = (tid & 7) + 8 * (tid >> (3 + lg));
    const int r_step = 8 * ((kProducerThreads / 8) >> lg);
    const unsigned off_base = g_off + (unsigned)(r_base >> 3) * sbo + j * 128 + (r_base & 7) * 16;
    const unsigned off_step = (unsigned)(r_step >> 3) * sbo;
    const int n_mine = pieces_per_row;
    // running counters instead of divisions: ring stage / round of the step being issued (s)
    // and of the step being completed (c = s - L), offset index and slice of step s
    int st = 0, round = 0, ki = 0, slice = 0;
    int st_c = 0;
    const bool copy_only = kBf16 && P.in_split != nullptr;  // rows split before the launch: see TcParams
    if (kBf16 && !copy_only) {
      // bf16 operands are made in registers, so the gather cannot run ahead through the ring like the
      // cp.async one.  It runs ahead through registers instead: the loads of step s + 1 are issued
      // before step s is converted and stored (two register buffers, the loop handles two steps per
      // turn), which hides the L2 latency of every step but the first behind the previous one's work.
      constexpr int kMine = 4;  // pieces per thread and step: 32 input planes / 8 per 16-byte bf16 piece
      float4 xa[kMine][2], xb[kMine][2];
      unsigned va = 0, vb = 0;  // which pieces of the buffer hold a real row
      auto load_step = [&](float4 (&x)[kMine][2], unsigned &valid) {
        const int k = sh_steps[ki];
        const int *idx = sh_idx + k * kTcRows + r_base;
        const float *col = P.in + slice * kc + j * kPerPiece;
        valid = 0;
#pragma unroll
        for (int i = 0; i < kMine; ++i)
          if (i < n_mine) {
            const int src_row = idx[i * r_step];
            if (src_row >= 0) {
              const float4 *src = reinterpret_cast<const float4 *>(col + (long long)src_row * P.ld_in);
              x[i][0] = __ldg(src);
              x[i][1] = __ldg(src + 1);
              valid |= 1u << i;
            }
          }
        if (++slice == n_slices) {
          slice = 0;
          ++ki;
        }
      };
      auto store_step = [&](const float4 (&x)[kMine][2], unsigned valid, int step) -> bool {
        if (round > 0) {  // one lane polls, the warp follows
          int freed = 1;
          if (lane == 0) freed = mbar_wait(&empty[st], (unsigned)((round - 1) & 1)) ? 1 : 0;
          if (!__shfl_sync(0xffffffffu, freed, 0)) return false;
        }
        unsigned char *sa = stage_base + (size_t)st * stage_bytes;
#pragma unroll
        for (int i = 0; i < kMine; ++i)
          if (i < n_mine) {
            // 8 input floats -> one 16-byte piece of 8 bf16; the three-term form also stores what the
            // rounding left over, as a second bf16 tile
            uint4 packed = make_uint4(0, 0, 0, 0), rest = make_uint4(0, 0, 0, 0);
            if (valid & (1u << i)) {
              split_bf16_pair(x[i][0].x, x[i][0].y, packed.x, rest.x);
              split_bf16_pair(x[i][0].z, x[i][0].w, packed.y, rest.y);
              split_bf16_pair(x[i][1].x, x[i][1].y, packed.z, rest.z);
              split_bf16_pair(x[i][1].z, x[i][1].w, packed.w, rest.w);
            }
            const unsigned off = off_base + i * off_step;
            *reinterpret_cast<uint4 *>(sa + off) = packed;
            if (kSplit) *reinterpret_cast<uint4 *>(sa + g_bytes + off) = rest;
          }
        __syncwarp();
        // (test hook: one warp of CTA 0 never reports its first step, so the MMA thread's bounded wait runs out)
        const bool dropped = P.drop_arrival && blockIdx.x == 0 && blockIdx.y == 0 && warp == 0 && step == 0;
        if (lane == 0 && !dropped) mbar_arrive(&full_g[st]);  // one arrival per warp (release)
        if (++st == NS) {
          st = 0;
          ++round;
        }
        return true;
      };
      if (S > 0) load_step(xa, va);
      for (int s = 0; s < S; s += 2) {
        if (*sh_abort) break;
        if (s + 1 < S) load_step(xb, vb);
        if (!store_step(xa, va, s)) {
          *sh_abort = 1;
          break;
        }
        if (s + 1 < S) {
          if (s + 2 < S) load_step(xa, va);
          if (!store_step(xb, vb, s + 1)) {
            *sh_abort = 1;
            break;
          }
        }
      }
    } else {
    for (int s = 0; s < S + L; ++s) {
      if (*sh_abort) break;
      if (s < S) {
        if (round > 0) {  // one lane polls, the warp follows
          int freed = 1;
          if (lane == 0) freed = mbar_wait(&empty[st], (unsigned)((round - 1) & 1)) ? 1 : 0;
          freed = __shfl_sync(0xffffffffu, freed, 0);
          if (!freed) {
            *sh_abort = 1;
            break;
          }
        }
        const int k = sh_steps[ki];
        unsigned char *sa = stage_base + (size_t)st * stage_bytes;
        const unsigned sa_u32 = smem_u32(sa);
        const int *idx = sh_idx + k * kTcRows + r_base;
        const float *col = P.in + slice * kc + j * kPerPiece;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          if (i < n_mine) {
            const int src_row = idx[i * r_step];
            const unsigned off = off_base + i * off_step;
            if (kBf16 && copy_only) {
              // plane p = slice * kc + 8 j of the row: block p / 32 of [32 h | 32 m], piece (p % 32) / 8
              if (src_row >= 0) {
                const int p = slice * kc + j * kPerPiece;
                const unsigned char *src = P.in_split + (size_t)src_row * P.ld_in * 4 + (size_t)(p >> 5) * 128 + ((p & 31) >> 3) * 16;
                cp_async16(sa_u32 + off, src, 16u);
                if (kSplit) cp_async16(sa_u32 + g_bytes + off, src + 64, 16u);
              } else {
                *reinterpret_cast<uint4 *>(sa + off) = make_uint4(0, 0, 0, 0);
                if (kSplit) *reinterpret_cast<uint4 *>(sa + g_bytes + off) = make_uint4(0, 0, 0, 0);
              }
            } else if (!kBf16) {
              // The copy pipe moves one 16-byte lane request per cycle, so a zero-filling copy
              // costs as much as a real one; a missing row is zeroed with a plain 128-bit store
              // (32 lanes per 4 cycles) instead and only real rows go through cp.async.
              if (src_row >= 0)
                cp_async16(sa_u32 + off, col + (long long)src_row * P.ld_in, 16u);
              else
                *reinterpret_cast<uint4 *>(sa + off) = make_uint4(0, 0, 0, 0);
            } else {
              // bf16: 8 input floats -> one 16-byte piece of 8 bf16, converted in registers; the
              // three-term form also stores what the rounding left over, as a second bf16 tile
              uint4 packed = make_uint4(0, 0, 0, 0), rest = make_uint4(0, 0, 0, 0);
              if (src_row >= 0) {
                const float4 *src = reinterpret_cast<const float4 *>(col + (long long)src_row * P.ld_in);
                float4 x = __ldg(src), y = __ldg(src + 1);
                split_bf16_pair(x.x, x.y, packed.x, rest.x);
                split_bf16_pair(x.z, x.w, packed.y, rest.y);
                split_bf16_pair(y.x, y.y, packed.z, rest.z);
                split_bf16_pair(y.z, y.w, packed.w, rest.w);
              }
              *reinterpret_cast<uint4 *>(sa + off) = packed;
              if (kSplit) *reinterpret_cast<uint4 *>(sa + g_bytes + off) = rest;
            }
          }
        }
        if (kAsyncArrive || copy_only)
          asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(&full_g[st])) : "memory");
        if (++slice == n_slices) {
          slice = 0;
          ++ki;
        }
        if (++st == NS) {
          st = 0;
          ++round;
        }
      }
      if (kAsyncArrive || copy_only) continue;
      cp_async_commit();
      if (s >= L) {
        // step c = s - L: its rows have landed once only L groups are still pending
        cp_async_wait_dyn(L);
        unsigned char *sa = stage_base + (size_t)st_c * stage_bytes;
        if (kSplit && !kBf16) {
          // low parts of the pieces this thread copied: g_lo = g - trunc_tf32(g)
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            if (i < n_mine) {
              const unsigned off = off_base + i * off_step;
              float4 a = *reinterpret_cast<const float4 *>(sa + off);
              float4 lo;
              lo.x = a.x - __uint_as_float(__float_as_uint(a.x) & 0xFFFFE000u);
              lo.y = a.y - __uint_as_float(__float_as_uint(a.y) & 0xFFFFE000u);
              lo.z = a.z - __uint_as_float(__float_as_uint(a.z) & 0xFFFFE000u);
              lo.w = a.w - __uint_as_float(__float_as_uint(a.w) & 0xFFFFE000u);
              *reinterpret_cast<float4 *>(sa + g_bytes + off) = lo;
            }
          }
        }
        // No proxy fence here: with copies of later steps still in flight it would wait for all
        // of them and serialise the gather.  The consumer fences after it has acquired the barrier.
        __syncwarp();
        // (test hook: one warp of CTA 0 never reports its first step, so the MMA thread's bounded wait runs out)
        const bool dropped = P.drop_arrival && blockIdx.x == 0 && blockIdx.y == 0 && warp == 0 && s == L;
        if (lane == 0 && !dropped) mbar_arrive(&full_g[st_c]);  // one arrival per warp (release)
        if (++st_c == NS) st_c = 0;
      }
    }
    }
    cp_async_wait<0>();

    // ================================ epilogue (same 8 warps) ==================================
    // TMEM lane = output plane, column = tile row.  A warp may read only the 32 lanes of its
    // quadrant (warp id mod 4); the two warps of a quadrant take alternate 16-row chunks.  The 32
    // lanes of a warp hold 32 consecutive planes of one row: a 128-byte coalesced store.
    bool have_acc = false;
    if (S > 0 && !*sh_abort) {
      have_acc = mbar_wait(acc_full, 0);
      if (!have_acc) *sh_abort = 1;
    }
    have_acc = __all_sync(0xffffffffu, have_acc);  // tcgen05.ld below is warp-collective
    tc_fence_after();
    const int quad = warp & 3;
    if (S == 0 || have_acc) {
      for (int mt = 0; mt < n_mt; ++mt) {
        const int plane0 = mt * kTcPlanes + quad * 32;
        if (plane0 >= P.cout) break;
        const int plane = plane0 + lane;
        const bool plane_ok = plane < P.cout;
        const float b = (bias_base && plane_ok) ? bias_base[plane] : 0.f;
        // the fused BatchNorm belongs to the finished sum: with split offsets k_sum_partials applies it
        const bool epi = P.bn_scale && !P.partial && plane_ok;
        const float sc = epi ? P.bn_scale[plane] : 1.f, sh = epi ? P.bn_shift[plane] : 0.f;
        const float leak = epi ? P.leak : 1.f;
        for (int n0 = (warp >> 2) * 16; n0 < kTcRows; n0 += 32) {
          if (row0 + n0 >= P.n_out) break;
          float v[16];
          if (have_acc) {
            tmem_ld16(tmem_base + ((unsigned)(quad * 32) << 16) + (unsigned)(mt * kTcRows + n0), v);
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = 0.f;
          }
          if (plane_ok) {
            float *dst = out_base + (row0 + n0) * P.ld_out + plane;
#pragma unroll
            for (int i = 0; i < 16; ++i)
              if (row0 + n0 + i < P.n_out) {
                float y = v[i] + b;
                if (epi) {
                  y = __fadd_rn(__fmul_rn(y, sc), sh);
                  y *= (y > 0.f) ? 1.f : leak;
                }
                dst[(long long)i * P.ld_out] = y;
              }
          }
        }
      }
    }
  } else if (warp == kMmaWarp && lane == 0) {
    // ============================ weight slabs + MMA issue (one thread) =======================
    const unsigned idesc = instr_desc(kBf16);
    const unsigned total_w = w_bytes * (kSplit ? 2 : 1);
    bool ok = true;
    // running counters (no divisions): weight-slab loader and MMA issuer each walk the steps
    int w_st = 0, w_round = 0, w_ki = 0, w_slice = 0;
    auto load_next_w = [&]() {
      if (w_round > 0 && !mbar_wait(&empty[w_st], (unsigned)((w_round - 1) & 1))) {
        ok = false;
        return;
      }
      const int k = sh_steps[w_ki];
      unsigned char *sw = stage_base + (size_t)w_st * stage_bytes + w_off;
      mbar_expect_tx(&full_w[w_st], total_w);
      bulk_copy_g2s(smem_u32(sw), P.wprep + ((size_t)k * n_slices + w_slice) * total_w, total_w, &full_w[w_st]);
      if (++w_slice == n_slices) {
        w_slice = 0;
        ++w_ki;
      }
      if (++w_st == NS) {
        w_st = 0;
        ++w_round;
      }
    };
    const int Lw = L > 0 ? L : 1;  // the weight slabs always run at least one step ahead
    for (int s = 0; s < Lw && s < S && ok; ++s) load_next_w();
    int st = 0, round = 0;
    const int n_mma = kc / kMmaK;
    for (int step = 0; step < S && ok; ++step) {
      if (*sh_abort) break;
      if (step + Lw < S) load_next_w();
      const unsigned ph = (unsigned)(round & 1);
      if (!ok || !mbar_wait(&full_w[st], ph) || !mbar_wait(&full_g[st], ph)) {
        ok = false;
        break;
      }
      // the producers' generic-proxy writes were acquired through full_g; order them before the
      // tensor core's async-proxy reads
      fence_proxy_async_smem();
      tc_fence_after();
      const unsigned w_addr = smem_u32(stage_base + (size_t)st * stage_bytes) + w_off;
      const unsigned g_addr = smem_u32(stage_base + (size_t)st * stage_bytes) + g_off;
      for (int jj = 0; jj < n_mma; ++jj) {
        const unsigned long long dg = smem_desc(g_addr + jj * 256, 128, sbo);
        const unsigned long long dg_lo = smem_desc(g_addr + g_bytes + jj * 256, 128, sbo);
        const unsigned acc = (step > 0 || jj > 0) ? 1u : 0u;
        for (int mt = 0; mt < n_mt; ++mt) {
          const unsigned d = tmem_base + (unsigned)(mt * kTcRows);
          const unsigned w_mt = w_addr + (unsigned)mt * (kTcPlanes / 8) * sbo + jj * 256;
          const unsigned long long dw = smem_desc(w_mt, 128, sbo);
          tc_mma<kBf16>(d, dw, dg, idesc, acc);
          if (kSplit) {
            const unsigned long long dw_lo = smem_desc(w_mt + w_bytes, 128, sbo);
            tc_mma<kBf16>(d, dw, dg_lo, idesc, 1u);
            tc_mma<kBf16>(d, dw_lo, dg, idesc, 1u);
          }
        }
      }
      tc_commit(&empty[st]);
      if (step == S - 1) tc_commit(acc_full);
      if (++st == NS) {
        st = 0;
        ++round;
      }
    }
    if (!ok) *sh_abort = 1;
  }
  tc_fence_before();
  __syncthreads();
  if (*sh_abort && tid == 0) atomicOr(P.flags, FLAG_TC_TIMEOUT);
  if (warp == kMmaWarp) tmem_dealloc(tmem_base, (unsigned)P.tmem_cols);
}

// out[i] = bias[i % cout] + sum over s of partial[s][i], in the fixed order s = 0, 1, ...: the result
// does not depend on which CTA finished first.
__global__ void k_sum_partials(const float4 *__restrict__ partial, int n_split, long long n4, const float *__restrict__ bias,
                               const float *__restrict__ bn_scale, const float *__restrict__ bn_shift, float leak,
                               int cout, float4 *__restrict__ out) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n4) return;
  const int plane = (int)((i * 4) % cout);
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int s = 0; s < n_split; ++s) {
    const float4 v = partial[(long long)s * n4 + i];
    acc.x += v.x;
    acc.y += v.y;
    acc.z += v.z;
    acc.w += v.w;
  }
  if (bias) {  // added last, as the unsplit kernel adds it to the finished sum
    const float4 b = __ldg(reinterpret_cast<const float4 *>(bias + plane));
    acc.x += b.x;
    acc.y += b.y;
    acc.z += b.z;
    acc.w += b.w;
  }
  if (bn_scale) {
    const float4 sc = __ldg(reinterpret_cast<const float4 *>(bn_scale + plane));
    const float4 sh = __ldg(reinterpret_cast<const float4 *>(bn_shift + plane));
    acc.x = __fadd_rn(__fmul_rn(acc.x, sc.x), sh.x);
    acc.y = __fadd_rn(__fmul_rn(acc.y, sc.y), sh.y);
    acc.z = __fadd_rn(__fmul_rn(acc.z, sc.z), sh.z);
    acc.w = __fadd_rn(__fmul_rn(acc.w, sc.w), sh.w);
    acc.x *= (acc.x > 0.f) ? 1.f : leak;
    acc.y *= (acc.y > 0.f) ? 1.f : leak;
    acc.z *= (acc.z > 0.f) ? 1.f : leak;
    acc.w *= (acc.w > 0.f) ? 1.f : leak;
  }
  out[i] = acc;
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
// set by scn_test_drop_barrier_arrival, consumed by the next conv_forward_tc of the calling thread
static thread_local int g_drop_arrival = 0;

static int tc_mode_of(int precision) {
  switch (precision) {
    case SCN_PRECISION_TF32: return TC_TF32;
    case SCN_PRECISION_BF16: return TC_BF16;
    case SCN_PRECISION_TF32X3: return split_mode_of_env();
    default: return -1;
  }
}

bool conv_tc_supported(int cin, int cout, int groups, int precision) {
  if (tc_mode_of(precision) < 0) return false;
  return groups == 1 && cin % 16 == 0 && cout % 8 == 0 && cout >= 8 && cout <= 256;
}

struct TcPlan {
  int kc, stages, lookahead;
  size_t smem;
};

// conv_wide.cu: in [n][cin] fp32 -> out, per row and 32-plane block, the 32 h = bf16(x) then the 32 m = bf16(x - h)
int split_rows_bf16(const float *in, unsigned char *out, long long n_rows, int cin, cudaStream_t stream,
                    const float *pre_scale = nullptr, const float *pre_shift = nullptr, float pre_leak = 1.f,
                    const float *in_b = nullptr, int planes_a = 0);

static int env_int(const char *name, int dflt) {
  const char *v = getenv(name);
  return v ? atoi(v) : dflt;
}

// A tile costs K * Cin/16 x 3 tensor-core instructions of 128 cycles however few rows it holds,
// so a level with fewer tiles than the GPU has SMs leaves most tensor cores idle for the whole
// call.  Such calls split every tile's filter offsets over n CTAs; the CTAs write partial sums
// and k_sum_partials adds them in a fixed order.  n minimises (waves of CTAs) x (offsets per
// CTA + a fixed cost of about 1.5 offsets for a CTA's prologue and epilogue).
// SCN_TC_SPLIT forces the factor (1 = never split).
static int split_factor(long long n_out, int K, int cout) {
  const int forced = env_int("SCN_TC_SPLIT", 0);
  if (forced > 0) return std::max(1, std::min(forced, K));
  const long long tiles = ceil_div(n_out, kTcRows);
  const long long slots = 148 * (cout <= kTcPlanes ? 2 : 1);  // tensor memory: 256 columns per 128 planes
  if (tiles >= 4 * slots) return 1;
  int best = 1;
  double best_cost = 1e30;
  for (int n = 1; n <= K; ++n) {
    const double cost = (double)ceil_div(tiles * n, slots) * ((double)ceil_div(K, n) + 1.5);
    if (cost < best_cost - 1e-9) {
      best_cost = cost;
      best = n;
    }
  }
  return best;
}

// Picks the slice width, ring depth and lookahead.  Two CTAs per SM are preferred (one tile's
// prologue and epilogue then overlap the other's main loop) when tensor memory allows it
// (Cout <= 128: 256 columns each) and the ring keeps at least three stages; otherwise one CTA
// with a deeper ring.  SCN_TC_STAGES / SCN_TC_KC / SCN_TC_LOOKAHEAD override the choice.
static bool plan(int mode, int K, int cin, int cout, TcPlan &pl) {
  const int esize = (mode == TC_BF16 || mode == TC_BF16X3) ? 2 : 4;
  const int parts = (mode == TC_TF32X3 || mode == TC_BF16X3) ? 2 : 1;
  const size_t control = (size_t)K * kTcRows * 4 + 16 * 8 + 2 * kTcMaxOffsets * 4 + 64;
  const size_t one_cta = 200 * 1024, two_ctas = 110 * 1024;
  const int force_kc = env_int("SCN_TC_KC", 0), force_ns = env_int("SCN_TC_STAGES", 0);
  TcPlan best{};
  bool found = false;
  for (int pass = 0; pass < 2 && !found; ++pass) {  // pass 0: two CTAs per SM, pass 1: one
    if (pass == 0 && (cout > kTcPlanes || force_ns)) continue;
    const size_t budget = pass == 0 ? two_ctas : one_cta;
    for (int kc : {32, 16}) {
      if (cin % kc) continue;
      if (force_kc && kc != force_kc) continue;
      size_t stage = ((size_t)kTcRows * kc * esize + (size_t)cout * kc * esize) * parts;
      if (control + 2 * stage > budget) continue;
      int stages = force_ns ? force_ns : (int)std::min<size_t>(4, (budget - control) / stage);
      if (control + (size_t)stages * stage > 220 * 1024) continue;
      if (stages < 3 && !force_ns && (pass == 0 || (kc == 32 && cin % 16 == 0 && !force_kc))) continue;
      best.kc = kc;
      best.stages = stages;
      best.smem = (size_t)stages * stage + control;
      found = true;
      break;
    }
  }
  if (!found) return false;
  // The gather may run `lookahead` steps ahead; a stage is refilled only after its MMAs have
  // finished, so the ring needs lookahead + 2 stages to keep the producers from waiting on the
  // tensor core's round trip every step.  bf16 converts in registers with blocking loads, so
  // running ahead buys nothing there.
  best.lookahead = (mode == TC_BF16 || mode == TC_BF16X3)
                       ? 0
                       : std::max(1, std::min(env_int("SCN_TC_LOOKAHEAD", best.stages - 2), best.stages - 1));
  pl = best;
  return true;
}

// cudaFuncSetAttribute is per device: done once for every device the library is used on.
static int configure_tc_kernels() {
  static bool configured[64] = {false};
  int dev = 0;
  SCN_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && configured[dev]) return SCN_OK;
  SCN_CUDA_CHECK(cudaFuncSetAttribute(k_conv_tc<TC_TF32>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
  SCN_CUDA_CHECK(cudaFuncSetAttribute(k_conv_tc<TC_BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
  SCN_CUDA_CHECK(cudaFuncSetAttribute(k_conv_tc<TC_TF32X3>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
  SCN_CUDA_CHECK(cudaFuncSetAttribute(k_conv_tc<TC_BF16X3>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
  if (dev >= 0 && dev < 64) configured[dev] = true;
  return SCN_OK;
}

// Will conv_forward_tc split the rows before the launch (and so be able to take a BatchNorm in front into that pass)?
bool conv_tc_splits_rows(int precision, int cin, long long n_in, long long n_out) {
  const int mode = tc_mode_of(precision);
  const int copy_env = env_int("SCN_TC_COPY", -1);
  return (mode == TC_BF16 || mode == TC_BF16X3) && cin % 32 == 0 && n_in > 0 && !g_drop_arrival &&
         (copy_env < 0 ? n_out >= 4096 : copy_env != 0);
}

// pre_scale / pre_shift / pre_leak (optional, only where conv_tc_splits_rows says yes): an eval-mode BatchNorm and its
// leaky ReLU in front of the convolution, applied in the split pass
int conv_forward_tc(const float *in, long long n_in, float *out, long long n_out, const float *weight,
                    const float *bias, const float *bn_scale, const float *bn_shift, float leak, const int *table,
                    int K, int cin, int cout, int precision, int *flags, cudaStream_t stream, const float *pre_scale,
                    const float *pre_shift, float pre_leak, const float *in_b, int planes_a) {
  if (n_out == 0) return SCN_OK;
  int mode = tc_mode_of(precision);
  SCN_REQUIRE(mode >= 0 && K <= kTcMaxOffsets, SCN_ERR_UNSUPPORTED, "tensor-core path: unsupported precision/filter");
  SCN_REQUIRE((uintptr_t)in % 16 == 0, SCN_ERR_BAD_ARG, "tensor-core path needs a 16-byte aligned input matrix");
  TcPlan pl;
  SCN_REQUIRE(plan(mode, K, cin, cout, pl), SCN_ERR_UNSUPPORTED, "tensor-core path: tile does not fit shared memory");
  const int esize = (mode == TC_BF16 || mode == TC_BF16X3) ? 2 : 4;
  const int parts = (mode == TC_TF32X3 || mode == TC_BF16X3) ? 2 : 1;
  size_t wbytes = (size_t)K * cin * cout * esize * parts;
  WeightImage wi;
  bool build = true;
  SCN_TRY(weight_image_get(WIMG_TC, K, cin, cout, pl.kc * 16 + mode, wbytes, stream, &wi, &build));
  unsigned char *wprep = (unsigned char *)wi.ptr;
  long long total = (long long)K * cin * cout;
  if (build)
    SCN_LAUNCH(k_prepare_weights, (unsigned)ceil_div(total, 256), 256, 0, stream, weight, wprep, K, cin, cout, pl.kc, mode);

  // bf16 modes: the rows are split into their bf16 parts once, before the launch (a row is gathered by up to K
  // output rows), and the producers copy.  Not for the run the test hook asked for (its dropped arrival is a
  // warp's, and the copying producers arrive per thread) and not for the smallest levels, where the extra launch
  // costs more than it saves (224 -> 224 planes: 0.058 ms with register producers against 0.098 at 1.4 k rows, 0.093
  // against 0.082 at 6.4 k, 0.349 against 0.280 for 320 -> 160 at 23 k).  SCN_TC_COPY=0 / 1 forces the choice.
  unsigned char *split = nullptr;
  const bool copy_only = conv_tc_splits_rows(precision, cin, n_in, n_out);
  SCN_REQUIRE(copy_only || (!pre_scale && !in_b), SCN_ERR_UNSUPPORTED,
              "a BatchNorm or a join in front needs the split pass");
  if (copy_only) {
    SCN_TRY(device_alloc((void **)&split, (size_t)n_in * cin * 4, stream));
    const int st = split_rows_bf16(in, split, n_in, cin, stream, pre_scale, pre_shift, pre_leak, in_b, planes_a);
    if (st != SCN_OK) {
      device_free(split, stream);
      return st;
    }
  }
  TcParams P;
  P.in = in;
  P.in_split = split;
  P.n_in = n_in;
  P.ld_in = cin;
  P.out = out;
  P.n_out = n_out;
  P.ld_out = cout;
  P.wprep = wprep;
  P.bias = bias;
  P.bn_scale = bn_scale;
  P.bn_shift = bn_shift;
  P.leak = leak;
  P.nbr = table;
  P.K = K;
  P.cin = cin;
  P.cout = cout;
  P.kc = pl.kc;
  P.n_stages = pl.stages;
  P.lookahead = pl.lookahead;
  P.tmem_cols = kTcRows * (int)ceil_div(cout, kTcPlanes);
  P.flags = flags;
  P.drop_arrival = g_drop_arrival;
  g_drop_arrival = 0;
  const bool vec_ok = (uintptr_t)out % 16 == 0 && (uintptr_t)bias % 16 == 0;  // k_sum_partials moves float4
  P.n_split = vec_ok ? split_factor(n_out, K, cout) : 1;
  P.partial = nullptr;
  if (P.n_split > 1) SCN_TRY(device_alloc((void **)&P.partial, (size_t)P.n_split * n_out * cout * sizeof(float), stream));
  dim3 grid((unsigned)ceil_div(n_out, kTcRows), (unsigned)P.n_split);
  SCN_TRY(configure_tc_kernels());
  if (mode == TC_TF32)
    SCN_LAUNCH(k_conv_tc<TC_TF32>, grid, kTcThreads, pl.smem, stream, P);
  else if (mode == TC_BF16)
    SCN_LAUNCH(k_conv_tc<TC_BF16>, grid, kTcThreads, pl.smem, stream, P);
  else if (mode == TC_BF16X3)
    SCN_LAUNCH(k_conv_tc<TC_BF16X3>, grid, kTcThreads, pl.smem, stream, P);
  else
    SCN_LAUNCH(k_conv_tc<TC_TF32X3>, grid, kTcThreads, pl.smem, stream, P);
  const cudaError_t launch_err = cudaGetLastError();
  device_free(split, stream);
  SCN_CUDA_CHECK(launch_err);
  if (P.n_split > 1) {
    const long long n4 = n_out * cout / 4;  // cout is a multiple of 8
    SCN_LAUNCH(k_sum_partials, (unsigned)ceil_div(n4, 256), 256, 0, stream, reinterpret_cast<const float4 *>(P.partial), P.n_split, n4, bias, bn_scale, bn_shift, leak, cout, reinterpret_cast<float4 *>(out));
    SCN_CUDA_CHECK(cudaGetLastError());
    SCN_TRY(device_free(P.partial, stream));
  }
  SCN_TRY(weight_image_put(wi, stream));
  return SCN_OK;
}


// ---------------------------------------------------------------------------------------------
// Allocation-free variant
// ---------------------------------------------------------------------------------------------
// conv_forward_tc stages the prepared weight image in memory it takes from the stream-ordered
// allocator.  Some hosts cannot do that at the point where they run the convolution: code
// that is replaying a fixed sequence of launches, a real-time loop that must not enter the
// driver's allocator, a process whose memory budget was handed out up front.  For them the
// same kernel pair runs with the image in a fixed array that is part of the library image:
// every GPU that loads the library carries these 8 MiB until the process exits.
constexpr size_t kStaticWeightBytes = 8u << 20;
static __device__ __align__(256) unsigned char g_static_weight_image[kStaticWeightBytes];

// In host code the array's name is only a handle; the device address comes from the runtime,
// once per device, with that device current.
static void *g_static_weight_ptr[64] = {nullptr};

static int static_weight_image(void **ptr) {
  int dev = 0;
  SCN_CUDA_CHECK(cudaGetDevice(&dev));
  SCN_REQUIRE(dev >= 0 && dev < 64, SCN_ERR_UNSUPPORTED, "device index %d unsupported", dev);
  if (!g_static_weight_ptr[dev]) {
    void *p = nullptr;
    SCN_CUDA_CHECK(cudaGetSymbolAddress(&p, g_static_weight_image));
    SCN_REQUIRE(p, SCN_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
    g_static_weight_ptr[dev] = p;
  }
  *ptr = g_static_weight_ptr[dev];
  return SCN_OK;
}

}  // namespace scn

extern "C" int scn_test_drop_barrier_arrival(void) {
  scn::g_drop_arrival = 1;
  return SCN_OK;
}

extern "C" int scn_submanifold_convolution_forward_static(scn_metadata *md, const int64_t *spatial_size,
                                                          const int64_t *filter_size, const float *in_features,
                                                          float *out_features, const float *weight,
                                                          const float *bias, int n_in_planes, int n_out_planes,
                                                          int precision, void *stream_) {
  using namespace scn;
  cudaStream_t stream = (cudaStream_t)stream_;
  SCN_REQUIRE(md && spatial_size && filter_size && weight, SCN_ERR_BAD_ARG, "null argument");
  const int mode = tc_mode_of(precision);
  SCN_REQUIRE(mode >= 0 && conv_tc_supported(n_in_planes, n_out_planes, 1, precision), SCN_ERR_UNSUPPORTED,
              "the allocation-free entry point runs the tensor-core kernel only: precision tf32 / bf16 / tf32x3, "
              "n_in_planes %% 16 == 0, n_out_planes %% 8 == 0, n_out_planes <= 256 (got %d -> %d, precision %d)",
              n_in_planes, n_out_planes, precision);
  // the rulebook must exist already: building it would allocate
  auto it = md->sub_rules.find(make_key(md->dim, spatial_size, filter_size));
  SCN_REQUIRE(it != md->sub_rules.end() && it->second.built, SCN_ERR_NO_GRID,
              "rulebook not built yet: call scn_md_submanifold_rulebook (which allocates) beforehand");
  SCN_REQUIRE(md->flags_dev, SCN_ERR_NO_GRID, "metadata has no device state yet");
  Rulebook &rb = it->second;
  const int K = rb.n_offsets, cin = n_in_planes, cout = n_out_planes;
  if (rb.n_out == 0) return SCN_OK;
  SCN_REQUIRE(in_features && out_features, SCN_ERR_BAD_ARG, "null features");
  SCN_REQUIRE(K <= kTcMaxOffsets && (uintptr_t)in_features % 16 == 0, SCN_ERR_UNSUPPORTED,
              "filter volume above %d or input matrix not 16-byte aligned", kTcMaxOffsets);
  TcPlan pl;
  SCN_REQUIRE(plan(mode, K, cin, cout, pl), SCN_ERR_UNSUPPORTED, "tile does not fit shared memory");
  const int esize = (mode == TC_BF16 || mode == TC_BF16X3) ? 2 : 4;
  const int parts = (mode == TC_TF32X3 || mode == TC_BF16X3) ? 2 : 1;
  const size_t wbytes = (size_t)K * cin * cout * esize * parts;
  SCN_REQUIRE(wbytes <= kStaticWeightBytes, SCN_ERR_UNSUPPORTED,
              "prepared weights need %zu bytes, the built-in buffer holds %zu (filter volume x n_in x n_out x %d)",
              wbytes, kStaticWeightBytes, esize * parts);
  void *image = nullptr;
  SCN_TRY(static_weight_image(&image));
  // the image is rewritten in full for this call's shape; nothing in it has to start at zero
  const long long total = (long long)K * cin * cout;
  SCN_LAUNCH(k_prepare_weights, (unsigned)ceil_div(total, 256), 256, 0, stream, weight, (unsigned char *)image, K, cin,
             cout, pl.kc, mode);
  TcParams P;
  P.in = in_features;
  P.in_split = nullptr;  // no allocation here: the producers split in registers
  P.n_in = rb.n_in;
  P.ld_in = cin;
  P.out = out_features;
  P.n_out = rb.n_out;
  P.ld_out = cout;
  P.wprep = (const unsigned char *)image;
  P.bias = bias;
  P.bn_scale = P.bn_shift = nullptr;
  P.leak = 1.f;
  P.nbr = rb.nbr;
  P.K = K;
  P.cin = cin;
  P.cout = cout;
  P.kc = pl.kc;
  P.n_stages = pl.stages;
  P.lookahead = pl.lookahead;
  P.tmem_cols = kTcRows * (int)ceil_div(cout, kTcPlanes);
  P.n_split = 1;  // splitting needs scratch for the partial sums
  P.partial = nullptr;
  P.flags = md->flags_dev;
  P.drop_arrival = 0;
  const unsigned grid = (unsigned)ceil_div(rb.n_out, kTcRows);
  SCN_TRY(configure_tc_kernels());  // attribute calls: no allocation
  if (mode == TC_TF32)
    SCN_LAUNCH(k_conv_tc<TC_TF32>, grid, kTcThreads, pl.smem, stream, P);
  else if (mode == TC_BF16)
    SCN_LAUNCH(k_conv_tc<TC_BF16>, grid, kTcThreads, pl.smem, stream, P);
  else if (mode == TC_BF16X3)
    SCN_LAUNCH(k_conv_tc<TC_BF16X3>, grid, kTcThreads, pl.smem, stream, P);
  else
    SCN_LAUNCH(k_conv_tc<TC_TF32X3>, grid, kTcThreads, pl.smem, stream, P);
  SCN_CUDA_CHECK(cudaGetLastError());
  return SCN_OK;
}
