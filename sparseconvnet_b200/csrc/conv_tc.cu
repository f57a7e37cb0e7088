// Tensor-core sparse convolution for sm_100a: tcgen05.mma with the accumulator in TMEM.
//
// Output stationary, like the fp32 kernel: a CTA owns 128 consecutive output rows for the whole
// filter, so the accumulator tile D[128 x Cout] (fp32) lives in tensor memory from the first
// filter offset to the last and every output row is written to HBM exactly once.  For every
// filter offset k for which the tile has at least one rule, and every 32-plane slice of the
// input planes:
//   A  = the 128 input rows named by the dense rulebook column (offset k, rows of the tile),
//        gathered with 16-byte cp.async copies straight into the tensor core's K-major
//        core-matrix layout in shared memory; a row without a rule is zero-filled by the copy
//        itself (src-size 0), so it contributes nothing;
//   B  = W[k][slice][:] -- prepared once per call in exactly that shared-memory image, so one
//        bulk-copy (cp.async.bulk, completion on an mbarrier) brings the whole slab;
//   D += A * B  issued by one elected thread: Cin-slice/8 (tf32) or /16 (bf16) tcgen05.mma
//        instructions of shape 128 x Cout x 8|16, completion tracked with tcgen05.commit.
// The gather runs up to three steps ahead of the tensor core through a ring of shared-memory
// stages; producer warps and the MMA-issuing warp meet only on mbarriers (no block-wide sync in
// the main loop).
//
// Arithmetic modes:
//   TF32    one pass, operands truncated to tf32 by the tensor core            (1e-2 class)
//   BF16    operands rounded to bf16 while staging, fp32 accumulate            (1e-2 class)
//   TF32X3  split a = a_hi + a_lo (both tf32-representable): D += A_hi*B_hi + A_lo*B_hi +
//           A_hi*B_lo, fp32 accumulate -- recovers fp32-class accuracy (error ~2^-21 per
//           product) on the tensor pipe, for the reference's fp32 parity bar.
//
// Every wait on an mbarrier is bounded; on expiry the kernel raises FLAG_TC_TIMEOUT, stops
// issuing work, drains its own copies, frees its tensor memory and returns.
#include <cuda_bf16.h>

#include <stdlib.h>

#include <algorithm>

#include "metadata.cuh"

namespace scn {

enum TcMode : int { TC_TF32 = 0, TC_BF16 = 1, TC_TF32X3 = 2 };

constexpr int kTcRows = 128;     // M of the MMA tile = TMEM lanes
constexpr int kTcThreads = 160;  // 4 producer/epilogue warps + 1 MMA warp
constexpr int kTcMaxOffsets = 128;
constexpr unsigned kWaitLimit = 1u << 20;

// ---------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ unsigned smem_u32(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned long long *bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long *bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait: returns false if the phase did not complete within the iteration limit.
__device__ __forceinline__ bool mbar_wait(unsigned long long *bar, unsigned parity) {
  unsigned addr = smem_u32(bar);
  for (unsigned it = 0; it < kWaitLimit; ++it) {
    unsigned done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}
__device__ __forceinline__ void cp_async16(unsigned dst, const void *src, unsigned src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulk_copy_g2s(unsigned dst, const void *src, unsigned bytes, unsigned long long *bar) {
  asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_alloc(unsigned *dst_smem, unsigned ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(unsigned taddr, unsigned ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_commit(unsigned long long *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
template <bool BF16>
__device__ __forceinline__ void tc_mma(unsigned d_tmem, unsigned long long a_desc, unsigned long long b_desc,
                                       unsigned idesc, unsigned accumulate) {
  if (BF16)
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  else
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// 32 lanes x 16 consecutive 32-bit columns: thread t of the warp gets lane (base lane + t).
__device__ __forceinline__ void tmem_ld16(unsigned taddr, float *v) {
  unsigned r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, "
      "[%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor, K-major, no swizzle: 8-row x 16-byte core matrices stored as
// contiguous 128-byte blocks; `lbo` = byte step between core matrices along K, `sbo` = byte
// step between 8-row groups along M/N; version field 1 (Blackwell).
__device__ __forceinline__ unsigned long long smem_desc(unsigned addr, unsigned lbo, unsigned sbo) {
  unsigned long long d = 0;
  d |= (unsigned long long)((addr >> 4) & 0x3FFF);
  d |= (unsigned long long)((lbo >> 4) & 0x3FFF) << 16;
  d |= (unsigned long long)((sbo >> 4) & 0x3FFF) << 32;
  d |= 1ull << 46;
  return d;
}
// Instruction descriptor: D fp32, A/B both tf32 or both bf16, both K-major, M = 128, N = n.
__host__ __device__ inline unsigned instr_desc(bool bf16, int n) {
  unsigned fmt = bf16 ? 1u : 2u;
  return (1u << 4) | (fmt << 7) | (fmt << 10) | ((unsigned)(n >> 3) << 17) | ((unsigned)(kTcRows >> 4) << 24);
}

// ---------------------------------------------------------------------------------------------
// weight preparation: W [K][Cin][Cout] fp32 -> per (offset, slice) the shared-memory image of the
// B operand (N = Cout rows, K-major core matrices), high part and -- for TF32X3 -- low part.
// image(k, c) at ((k * n_slices + c) * parts + part) * cout * kc * esize bytes.
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
  int parts = mode == TC_TF32X3 ? 2 : 1;
  if (mode == TC_BF16) {
    size_t tile = (size_t)cout * kc * 2;
    size_t off = (size_t)(n / 8) * (kc / 8) * 128 + (size_t)(kk / 8) * 128 + (n % 8) * 16 + (kk % 8) * 2;
    *reinterpret_cast<__nv_bfloat16 *>(out + ((size_t)k * n_slices + slice) * tile + off) = __float2bfloat16_rn(v);
  } else {
    size_t tile = (size_t)cout * kc * 4;
    size_t off = (size_t)(n / 8) * (kc / 4) * 128 + (size_t)(kk / 4) * 128 + (n % 8) * 16 + (kk % 4) * 4;
    unsigned char *base = out + (((size_t)k * n_slices + slice) * parts) * tile;
    float hi = __uint_as_float(__float_as_uint(v) & 0xFFFFE000u);
    *reinterpret_cast<float *>(base + off) = (mode == TC_TF32X3) ? hi : v;
    if (mode == TC_TF32X3) *reinterpret_cast<float *>(base + tile + off) = v - hi;
  }
}

// ---------------------------------------------------------------------------------------------
// main kernel
// ---------------------------------------------------------------------------------------------
struct TcParams {
  const float *in;
  long long n_in;
  int ld_in;
  float *out;
  long long n_out;
  int ld_out;
  const unsigned char *wprep;
  const float *bias;
  const int *nbr;  // [K][n_out]
  int K, cin, cout;
  int kc;          // input planes per step (32 or 16)
  int n_stages;
  int lookahead;   // steps the gather runs ahead of the tensor core (< n_stages)
  int tmem_cols;   // power of two >= cout, >= 32
  int *flags;
};

__device__ __forceinline__ void mbar_arrive(unsigned long long *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void cp_async_wait_dyn(int n) {
  switch (n) {
    case 0: cp_async_wait<0>(); break;
    case 1: cp_async_wait<1>(); break;
    case 2: cp_async_wait<2>(); break;
    default: cp_async_wait<3>(); break;
  }
}

// Warp roles.  Warps 0-3 (128 threads, one per tile row in the epilogue) are the gather
// producers; warp 4 owns tensor memory, streams the weight slabs and issues the MMAs.  The
// roles meet only on mbarriers:
//   full_a[s]  128 producer arrivals: the rows of stage s are in shared memory (and fenced for
//              the async proxy)
//   full_w[s]  transaction barrier of the weight slab's bulk copy
//   empty[s]   tcgen05.commit: the MMAs that read stage s have finished
//   acc_full   tcgen05.commit after the last MMA of the tile
constexpr int kProducerThreads = 128;

template <int MODE>
__global__ void __launch_bounds__(kTcThreads) k_conv_tc(TcParams P) {
  constexpr bool kBf16 = (MODE == TC_BF16);
  constexpr bool kSplit = (MODE == TC_TF32X3);
  constexpr int kEsize = kBf16 ? 2 : 4;
  constexpr int kPerPiece = 16 / kEsize;  // elements per 16-byte piece
  constexpr int kMmaK = 32 / kEsize;      // K per instruction (32 bytes)

  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const long long row0 = (long long)blockIdx.x * kTcRows;
  const int K = P.K, kc = P.kc, NS = P.n_stages, L = P.lookahead;
  const int n_slices = P.cin / kc;
  const int pieces_per_row = kc / kPerPiece;
  const unsigned a_bytes = kTcRows * kc * kEsize;
  const unsigned w_bytes = P.cout * kc * kEsize;
  const unsigned stage_bytes = (a_bytes + w_bytes) * (kSplit ? 2 : 1);
  const unsigned sbo = pieces_per_row * 128;

  // shared memory carve-up: [stages][A | A_lo | W | W_lo] | idx [K][128] | control
  unsigned char *stage_base = smem;
  int *sh_idx = reinterpret_cast<int *>(smem + (size_t)NS * stage_bytes);
  unsigned long long *bars = reinterpret_cast<unsigned long long *>(sh_idx + (size_t)K * kTcRows);
  unsigned long long *full_a = bars;            // [NS]
  unsigned long long *full_w = bars + NS;       // [NS]
  unsigned long long *empty = bars + 2 * NS;    // [NS]
  unsigned long long *acc_full = bars + 3 * NS;
  int *sh_steps = reinterpret_cast<int *>(bars + 3 * NS + 1);  // [K] offsets with at least one rule
  int *sh_has = sh_steps + kTcMaxOffsets;                       // [K]
  unsigned *sh_tmem = reinterpret_cast<unsigned *>(sh_has + kTcMaxOffsets);
  int *sh_nk = reinterpret_cast<int *>(sh_tmem + 1);
  volatile int *sh_abort = sh_nk + 1;

  // ---- prologue: barriers, tensor memory, rulebook columns of this tile ----------------------
  if (tid == 0) {
    for (int s = 0; s < NS; ++s) {
      mbar_init(&full_a[s], kProducerThreads);
      mbar_init(&full_w[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_full, 1);
    *sh_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 4) tmem_alloc(sh_tmem, (unsigned)P.tmem_cols);
  for (int k = warp; k < K; k += kTcThreads / 32) {
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
    for (int k = 0; k < K; ++k)
      if (sh_has[k]) sh_steps[n++] = k;
    *sh_nk = n;
  }
  __syncthreads();
  const unsigned tmem_base = *sh_tmem;
  const int S = *sh_nk * n_slices;

  if (warp < 4) {
    // =================================== gather producers =====================================
    // Piece p = tid + 128 i of a stage is the 16-byte piece j of tile row r with
    //   r = (p & 7) + 8 * (p / (8 * pieces_per_row)),  j = (p >> 3) % pieces_per_row,
    // so a quarter warp fills one 128-byte core matrix and a warp reads 64 contiguous bytes of
    // 8 rows.  pieces_per_row is a power of two (2, 4 or 8): j is fixed per thread and the rows
    // step by 16 * 8 / pieces_per_row.
    const int lg = 31 - __clz(pieces_per_row);
    const int j = (tid >> 3) & (pieces_per_row - 1);
    const int r_base = (tid & 7) + 8 * (tid >> (3 + lg));
    const int r_step = 8 * (16 >> lg);
    const unsigned off_base = (unsigned)(r_base >> 3) * sbo + j * 128 + (r_base & 7) * 16;
    const unsigned off_step = (unsigned)(r_step >> 3) * sbo;
    const int n_mine = pieces_per_row;  // pieces of this thread per stage
    for (int s = 0; s < S + L; ++s) {
      if (*sh_abort) break;
      if (s < S) {
        const int st = s % NS, use = s / NS;
        if (use > 0 && !mbar_wait(&empty[st], (unsigned)((use - 1) & 1))) {
          *sh_abort = 1;
          break;
        }
        const int k = sh_steps[s / n_slices], slice = s % n_slices;
        unsigned char *sa = stage_base + (size_t)st * stage_bytes;
        const unsigned sa_u32 = smem_u32(sa);
        const int *idx = sh_idx + k * kTcRows + r_base;
        const float *col = P.in + slice * kc + j * kPerPiece;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          if (i < n_mine) {
            const int src_row = idx[i * r_step];
            const unsigned off = off_base + i * off_step;
            if (!kBf16) {
              cp_async16(sa_u32 + off, col + (long long)(src_row < 0 ? 0 : src_row) * P.ld_in, src_row < 0 ? 0u : 16u);
            } else {
              // bf16: 8 input floats -> one 16-byte piece of 8 bf16, converted in registers
              uint4 packed = make_uint4(0, 0, 0, 0);
              if (src_row >= 0) {
                const float4 *src = reinterpret_cast<const float4 *>(col + (long long)src_row * P.ld_in);
                float4 x = __ldg(src), y = __ldg(src + 1);
                __nv_bfloat162 b0 = __floats2bfloat162_rn(x.x, x.y), b1 = __floats2bfloat162_rn(x.z, x.w);
                __nv_bfloat162 b2 = __floats2bfloat162_rn(y.x, y.y), b3 = __floats2bfloat162_rn(y.z, y.w);
                packed.x = *reinterpret_cast<unsigned *>(&b0);
                packed.y = *reinterpret_cast<unsigned *>(&b1);
                packed.z = *reinterpret_cast<unsigned *>(&b2);
                packed.w = *reinterpret_cast<unsigned *>(&b3);
              }
              *reinterpret_cast<uint4 *>(sa + off) = packed;
            }
          }
        }
      }
      cp_async_commit();
      if (s >= L) {
        const int c = s - L;  // the step whose rows have landed once only L groups are pending
        cp_async_wait_dyn(L);
        unsigned char *sa = stage_base + (size_t)(c % NS) * stage_bytes;
        if (kSplit) {
          // low parts of the pieces this thread copied: a_lo = a - trunc_tf32(a)
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
              *reinterpret_cast<float4 *>(sa + a_bytes + off) = lo;
            }
          }
        }
        fence_proxy_async_smem();  // this thread's shared-memory writes -> visible to the tensor core
        mbar_arrive(&full_a[c % NS]);
      }
    }
    cp_async_wait<0>();

    // ================================ epilogue (same 4 warps) ==================================
    bool have_acc = false;
    if (S > 0 && !*sh_abort) {
      have_acc = mbar_wait(acc_full, 0);
      if (!have_acc) *sh_abort = 1;
    }
    have_acc = __all_sync(0xffffffffu, have_acc);  // tcgen05.ld below is warp-collective
    tc_fence_after();
    const long long row = row0 + warp * 32 + lane;
    const bool store = row < P.n_out && (S == 0 || have_acc);
    for (int c0 = 0; c0 < P.cout; c0 += 16) {
      float v[16];
      if (have_acc) {
        tmem_ld16(tmem_base + ((unsigned)(warp * 32) << 16) + (unsigned)c0, v);
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = 0.f;
      }
      if (store) {
        float *dst = P.out + row * P.ld_out + c0;
#pragma unroll
        for (int i = 0; i < 16; i += 4) {
          float4 o;
          o.x = v[i] + (P.bias ? P.bias[c0 + i] : 0.f);
          o.y = v[i + 1] + (P.bias ? P.bias[c0 + i + 1] : 0.f);
          o.z = v[i + 2] + (P.bias ? P.bias[c0 + i + 2] : 0.f);
          o.w = v[i + 3] + (P.bias ? P.bias[c0 + i + 3] : 0.f);
          *reinterpret_cast<float4 *>(dst + i) = o;
        }
      }
    }
  } else if (warp == 4 && lane == 0) {
    // ============================ weight slabs + MMA issue (one thread) =======================
    const unsigned idesc = instr_desc(kBf16, P.cout);
    const unsigned total_w = w_bytes * (kSplit ? 2 : 1);
    bool ok = true;
    auto load_w = [&](int s) {
      const int st = s % NS, use = s / NS;
      if (use > 0 && !mbar_wait(&empty[st], (unsigned)((use - 1) & 1))) {
        ok = false;
        return;
      }
      const int k = sh_steps[s / n_slices], slice = s % n_slices;
      unsigned char *sw = stage_base + (size_t)st * stage_bytes + (kSplit ? 2 * a_bytes : a_bytes);
      mbar_expect_tx(&full_w[st], total_w);
      bulk_copy_g2s(smem_u32(sw), P.wprep + ((size_t)k * n_slices + slice) * total_w, total_w, &full_w[st]);
    };
    const int Lw = L > 0 ? L : 1;  // the weight slabs always run at least one step ahead
    for (int s = 0; s < Lw && s < S && ok; ++s) load_w(s);
    for (int step = 0; step < S && ok; ++step) {
      if (*sh_abort) break;
      if (step + Lw < S) load_w(step + Lw);
      const int st = step % NS;
      const unsigned ph = (unsigned)((step / NS) & 1);
      if (!ok || !mbar_wait(&full_w[st], ph) || !mbar_wait(&full_a[st], ph)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const unsigned a_addr = smem_u32(stage_base + (size_t)st * stage_bytes);
      const unsigned w_addr = a_addr + (kSplit ? 2 * a_bytes : a_bytes);
      const int n_mma = kc / kMmaK;
      for (int j = 0; j < n_mma; ++j) {
        unsigned long long da = smem_desc(a_addr + j * 256, 128, sbo);
        unsigned long long db = smem_desc(w_addr + j * 256, 128, sbo);
        tc_mma<kBf16>(tmem_base, da, db, idesc, (step > 0 || j > 0) ? 1u : 0u);
        if (kSplit) {
          unsigned long long da_lo = smem_desc(a_addr + a_bytes + j * 256, 128, sbo);
          unsigned long long db_lo = smem_desc(w_addr + w_bytes + j * 256, 128, sbo);
          tc_mma<kBf16>(tmem_base, da_lo, db, idesc, 1u);
          tc_mma<kBf16>(tmem_base, da, db_lo, idesc, 1u);
        }
      }
      tc_commit(&empty[st]);
      if (step == S - 1) tc_commit(acc_full);
    }
    if (!ok) *sh_abort = 1;
  }
  tc_fence_before();
  __syncthreads();
  if (*sh_abort && tid == 0) atomicOr(P.flags, FLAG_TC_TIMEOUT);
  if (warp == 4) tmem_dealloc(tmem_base, (unsigned)P.tmem_cols);
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
static int tc_mode_of(int precision) {
  switch (precision) {
    case SCN_PRECISION_TF32: return TC_TF32;
    case SCN_PRECISION_BF16: return TC_BF16;
    case SCN_PRECISION_TF32X3: return TC_TF32X3;
    default: return -1;
  }
}

bool conv_tc_supported(int cin, int cout, int groups, int precision) {
  if (tc_mode_of(precision) < 0) return false;
  return groups == 1 && cin % 32 == 0 && cout % 16 == 0 && cout >= 16 && cout <= 256;
}

struct TcPlan {
  int kc, stages, lookahead;
  size_t smem;
};

static int env_int(const char *name, int dflt) {
  const char *v = getenv(name);
  return v ? atoi(v) : dflt;
}

// Picks the slice width, ring depth and lookahead.  Two CTAs per SM are preferred (one tile's
// prologue and epilogue then overlap the other's main loop) as long as the ring keeps at least
// three stages; otherwise one CTA with a deeper ring.  SCN_TC_STAGES / SCN_TC_KC /
// SCN_TC_LOOKAHEAD override the choice (tuning knobs).
static bool plan(int mode, int K, int cin, int cout, TcPlan &pl) {
  const int esize = mode == TC_BF16 ? 2 : 4;
  const size_t control = (size_t)K * kTcRows * 4 + 16 * 8 + 2 * kTcMaxOffsets * 4 + 64;
  const size_t one_cta = 200 * 1024, two_ctas = 110 * 1024;
  int force_kc = env_int("SCN_TC_KC", 0), force_ns = env_int("SCN_TC_STAGES", 0);
  for (int kc : {32, 16}) {
    if (cin % kc) continue;
    if (force_kc && kc != force_kc) continue;
    if (mode == TC_BF16 && kc == 16) continue;
    size_t stage = ((size_t)kTcRows * kc * esize + (size_t)cout * kc * esize) * (mode == TC_TF32X3 ? 2 : 1);
    if (control + 2 * stage > one_cta) continue;
    int stages = (int)std::min<size_t>(4, (two_ctas - std::min(control, two_ctas)) / stage);
    if (stages < 3) stages = (int)std::min<size_t>(4, (one_cta - control) / stage);
    if (force_ns) stages = force_ns;
    if (stages < 2 || control + (size_t)stages * stage > 220 * 1024) continue;
    if (stages < 3 && kc == 32 && cin % 16 == 0 && mode != TC_BF16 && !force_kc && !force_ns) continue;
    pl.kc = kc;
    pl.stages = stages;
    // bf16 converts in registers with blocking loads, so running ahead buys nothing there
    // The gather may run `lookahead` steps ahead; a stage is refilled only after its MMAs have
    // finished, so the ring needs lookahead + 2 stages to keep the producers from waiting on the
    // tensor core's round trip every step.  bf16 converts in registers with blocking loads, so
    // running ahead buys nothing there.
    pl.lookahead = mode == TC_BF16 ? 0 : std::max(1, std::min(env_int("SCN_TC_LOOKAHEAD", stages - 2), stages - 1));
    pl.smem = (size_t)stages * stage + control;
    return true;
  }
  return false;
}

int conv_forward_tc(const float *in, long long n_in, float *out, long long n_out, const float *weight,
                    const float *bias, const int *table, int K, int cin, int cout, int precision, int *flags,
                    cudaStream_t stream) {
  if (n_out == 0) return SCN_OK;
  int mode = tc_mode_of(precision);
  SCN_REQUIRE(mode >= 0 && K <= kTcMaxOffsets, SCN_ERR_UNSUPPORTED, "tensor-core path: unsupported precision/filter");
  SCN_REQUIRE(((uintptr_t)in % 16 == 0) && ((uintptr_t)out % 16 == 0), SCN_ERR_BAD_ARG,
              "tensor-core path needs 16-byte aligned feature matrices");
  TcPlan pl;
  SCN_REQUIRE(plan(mode, K, cin, cout, pl), SCN_ERR_UNSUPPORTED, "tensor-core path: tile does not fit shared memory");
  const int esize = mode == TC_BF16 ? 2 : 4;
  const int parts = mode == TC_TF32X3 ? 2 : 1;
  size_t wbytes = (size_t)K * cin * cout * esize * parts;
  unsigned char *wprep = nullptr;
  SCN_TRY(device_alloc((void **)&wprep, wbytes, stream));
  long long total = (long long)K * cin * cout;
  SCN_LAUNCH(k_prepare_weights, (unsigned)ceil_div(total, 256), 256, 0, stream, weight, wprep, K, cin, cout, pl.kc, mode);

  TcParams P;
  P.in = in;
  P.n_in = n_in;
  P.ld_in = cin;
  P.out = out;
  P.n_out = n_out;
  P.ld_out = cout;
  P.wprep = wprep;
  P.bias = bias;
  P.nbr = table;
  P.K = K;
  P.cin = cin;
  P.cout = cout;
  P.kc = pl.kc;
  P.n_stages = pl.stages;
  P.lookahead = pl.lookahead;
  P.tmem_cols = (int)std::max<unsigned long long>(32, next_pow2((unsigned long long)cout));
  P.flags = flags;
  unsigned grid = (unsigned)ceil_div(n_out, kTcRows);
  static bool configured[3] = {false, false, false};
  if (!configured[mode]) {
    SCN_CUDA_CHECK(cudaFuncSetAttribute(k_conv_tc<TC_TF32>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    SCN_CUDA_CHECK(cudaFuncSetAttribute(k_conv_tc<TC_BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    SCN_CUDA_CHECK(cudaFuncSetAttribute(k_conv_tc<TC_TF32X3>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    configured[0] = configured[1] = configured[2] = true;
  }
  if (mode == TC_TF32)
    SCN_LAUNCH(k_conv_tc<TC_TF32>, grid, kTcThreads, pl.smem, stream, P);
  else if (mode == TC_BF16)
    SCN_LAUNCH(k_conv_tc<TC_BF16>, grid, kTcThreads, pl.smem, stream, P);
  else
    SCN_LAUNCH(k_conv_tc<TC_TF32X3>, grid, kTcThreads, pl.smem, stream, P);
  SCN_CUDA_CHECK(cudaGetLastError());
  SCN_TRY(device_free(wprep, stream));
  return SCN_OK;
}

}  // namespace scn
