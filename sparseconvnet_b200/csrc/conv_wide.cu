// Persistent tcgen05 sparse convolution with bf16 operands: the kernel for wide layers (more than 64
// output planes) on levels with many rows, in the fp32-class three-term form and in the single-pass
// bf16 mode.
//
// Same mathematics and orientation as conv_tc.cu / conv_tma.cu (output stationary,
// D^T[planes x 256 rows] += W_k^T G_k^T with the accumulators in TMEM; the reference's per-offset
// gather / GEMM / scatter-add is CPU/Convolution.cpp:137-148, CUDA/Convolution.cu:57-233).  What is
// different is how the gathered rows reach the tensor core.  A tcgen05.mma of 128 x 256 x 16 bf16
// takes 128 cycles (measured by scn_tc_probe_mma: max(56, N / 2) cycles whatever M and kind), so a
// 32-plane step of the three-term form is 6 instructions = 768 cycles, and everything else has to
// fit under that:
//
//   * a pass before the launch (k_wide_split_rows) writes every input row once as its two bf16 parts,
//     h = bf16(x) and m = bf16(x - h), per 32-plane slice [32 h | 32 m]: the same 128 bytes as the fp32
//     slice.  A row is gathered by up to K output rows; it is converted once instead of K times;
//   * the twelve producer warps only copy: for every (tile row, 16-byte piece) one cp.async per part
//     straight into the K-major core-matrix layout the instruction reads, with zero fill where the tile
//     row has no rule for the offset.  Nothing passes through registers, nothing is converted, there is
//     no list of hits; a thread's arrival at the step's barrier is tied to the completion of its own
//     copies (cp.async.mbarrier.arrive), so the only thing a producer ever waits for is a free ring
//     slot.  (The form this replaced read fp32 rows into registers, split them there and stored both
//     tiles: 0.44 against 0.37 ms on 96 -> 96 planes at 154 k rows, the pass before the launch included);
//   * a step is 44-48 KB (two bf16 tiles + the two weight slabs), so the ring holds four steps;
//   * per filter offset the 256 row-owning threads publish their rulebook entry and one barrier (which
//     also carries the decision to stop) makes them visible; offsets for which the tile has no rule
//     cost that barrier and nothing else;
//   * one thread issues the MMAs (h h, h m, m h per 16 planes) into one of two TMEM accumulators
//     while four epilogue warps drain the other (tcgen05.ld -> bias -> optional per-plane
//     scale / shift / leaky ReLU of a following BatchNorm -> coalesced stores, each row once).
//
// Error of the three-term form: the dropped products m m and x_l w (x_l = x - h - m) are 2^-17 of a
// product; measured 5e-6 to 9e-6 of the largest output per layer against the reference's CPU
// operator, 3e-5 through the four 81-offset layers of the 4-D stack -- better than the three-pass
// tf32 split on the same instruction, whose high part is a truncation.
//
// What bounds it now: shared-memory bandwidth.  A step moves 32 KB of gathered tiles and 12-24 KB of
// weights in and lets the tensor core read 72 KB of operands out (each of the six instructions reads its
// 4 KB weight block and its 8 KB row block): about 120 KB per 768 cycles against the 128 bytes per cycle
// an SM's shared memory delivers.  96 -> 96 planes at 154 k rows runs at 1 700 cycles per step, the
// zero rows of a tile (60 % at that level) included.
//
// Every wait is bounded: on expiry the role raises the abort flag, everybody leaves their loops,
// tensor memory is freed and the host sees FLAG_TC_TIMEOUT through scn_md_poll_errors.
#include <stdlib.h>

#include <algorithm>

#include "metadata.cuh"
#include "tc_ptx.cuh"

namespace scn {

namespace {

constexpr int kWMaxRows = 256; // output rows per tile = MMA N: 256 or 128 (template parameter ROWS)
constexpr int kWPlanes = 128;  // output planes per MMA = M
constexpr int kWSlice = 32;    // input planes per step
constexpr int kWMaxStages = 8;
// warps 0 .. PW-1 produce (PW a multiple of four), the next four drain accumulators (their warp id mod 4
// selects the TMEM lane quadrant), the last issues the MMAs.  One CTA per SM with the whole shared memory
// and all 512 TMEM columns.
enum : int { W_LAST_OF_TILE = 1, W_LAST_OF_CTA = 2 };

struct WideParams {
  const float *in;
  const unsigned char *in_split;  // the input rows as bf16 parts: per row and 32-plane slice [32 h | 32 m]
  int ld_in;
  long long n_in;
  float *out;
  long long n_out;
  int ld_out;
  const unsigned char *wprep;  // per (offset, slice): [W_h | W_m] (three-term) or [W_h], bf16 core-matrix images
  const float *bias;
  const float *bn_scale, *bn_shift;  // optional: out = (acc + bias) * scale[plane] + shift[plane]
  float leak;                        // then out = out > 0 ? out : out * leak (1 = identity)
  const int *nbr;                    // [K][n_out]
  int K, cin, cout;
  int n_stages;
  long long n_tiles;
  int tile_rows;  // output rows per tile (the MMA's N): a multiple of 16, at most the kernel's ROWS
  int *flags;
};

__host__ __device__ inline unsigned wide_idesc(int rows) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(rows >> 3) << 17) | ((unsigned)(kWPlanes >> 4) << 24);
}

// TERMS 3: h h + h m + m h (fp32-class); 1: h h (plain bf16).  ROWS: rows of a tile in the shared-memory and TMEM
// layouts.  PW: producer warps.  TRC: the tile height of this launch as a constant (0: read from the parameters --
// with the height known to the compiler the kernel is 6 % faster: 4.33 against 4.63 ms on 64 -> 64 planes, 81 offsets,
// 1.5 M rows).
template <int TERMS, int ROWS, int PW, int TRC>
__global__ void __launch_bounds__((PW + 5) * 32, 1) k_conv_wide(WideParams P) {
  constexpr int kWProducerWarps = PW, kWProducers = PW * 32;
  constexpr int kWEpilogue0 = PW, kWMmaWarp = PW + 4;
  constexpr unsigned kTmemCols = 512u;
  constexpr int kParts = TERMS == 3 ? 2 : 1;
  constexpr int kWRows = ROWS;
  // A bf16 tile of gathered rows [ROWS x 32 planes] is stored as four planes of 16-byte pieces (piece j =
  // 8 input planes of every row): piece j of row r at j * kWLbo + r * 16.  That is the K-major
  // core-matrix layout with 128 bytes between 8-row groups and kWLbo between the K pieces; the 32
  // bytes of padding in kWLbo put the four pieces of a row on different banks, so the four lanes that
  // copy one row's part (its 64 contiguous bytes: one line per row and copy instruction) write
  // without conflicting with one another.
  constexpr unsigned kWLbo = kWRows * 16 + 32;
  constexpr unsigned kWTile = 4 * kWLbo;  // bytes of one tile (a multiple of 128)
  constexpr int kWOwners = ROWS / 32;           // warps whose threads own one tile row each for the rulebook reads
  constexpr int kWItems = (ROWS * 4 + kWProducers - 1) / kWProducers;  // (row, piece) items per thread and step
  extern __shared__ __align__(1024) unsigned char smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int NS = P.n_stages;
  const int n_slices = P.cin / kWSlice;
  const unsigned w_bytes = (unsigned)P.cout * kWSlice * 2;  // one bf16 weight slab
  const unsigned total_w = w_bytes * kParts;
  // step: [W_h (| W_m) | pad | G_h (| G_m)].  The weight slabs come first because an MMA always reads
  // 128 weight rows: with fewer output planes the rows past the slab are whatever follows it -- in
  // bounds, and they only reach TMEM lanes that are never read back.
  const unsigned w_region = (total_w + 1023u) & ~1023u;
  const unsigned stage_bytes = w_region + kWTile * kParts;  // a multiple of 128
  const int n_mt = (P.cout + kWPlanes - 1) / kWPlanes;
  const int n_acc = (2 * n_mt * kWRows <= (int)kTmemCols) ? 2 : 1;  // accumulator buffers in TMEM

  unsigned char *ctl = smem + (size_t)NS * stage_bytes;
  unsigned long long *full = reinterpret_cast<unsigned long long *>(ctl);  // [NS] rows stored, slab landed
  unsigned long long *empty = full + kWMaxStages;                          // [NS] MMAs done
  unsigned long long *acc_full = empty + kWMaxStages;                      // [2]
  unsigned long long *acc_empty = acc_full + 2;                            // [2]
  int *meta = reinterpret_cast<int *>(acc_empty + 2);                      // [NS] step flags
  unsigned *sh_tmem = reinterpret_cast<unsigned *>(meta + kWMaxStages);
  volatile int *sh_abort = reinterpret_cast<volatile int *>(sh_tmem + 1);
  int *ent = reinterpret_cast<int *>(ctl + 512);  // [2][256] input row of every tile row for the group's offset, or -1
  int *warp_cnt = ent + 2 * kWMaxRows;            // [2][8] rows with a rule per owner warp

  if (tid == 0) {
    for (int s = 0; s < NS; ++s) {
      mbar_init(&full[s], kWProducers + 1);  // every producer thread (its copies landed) + the slab
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);
    }
    *sh_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kWMmaWarp) tmem_alloc(sh_tmem, kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem_base = *sh_tmem;
  const long long my_tiles =
      ((long long)blockIdx.x < P.n_tiles) ? (P.n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  // Rows per tile: the shared-memory and TMEM layouts are those of ROWS rows; a launch may use fewer (the host
  // picks the height that gives every SM the same number of tiles), then the tail of each buffer stays unused.
  const int TR = TRC ? TRC : P.tile_rows;

  if (warp < kWProducerWarps) {
    // =============================== producers: copy the gathered rows ==========================
    int st = 0, round = 0;
    bool ok = true;
    // barrier + OR over the producers: every producer thread gets the same answer, so they leave
    // the loop together (a warp that left alone would strand the others at the next barrier)
    auto producer_vote = [](bool x) -> bool {
      unsigned r;
      asm volatile(
          "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 p, %1, 0;\n\tbar.red.or.pred q, 1, %2, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
          : "=r"(r)
          : "r"((unsigned)x), "n"(kWProducers)
          : "memory");
      return r != 0;
    };
    // waits until ring slot `s` (in ring round `rnd`) is free; all lanes get the answer
    auto slot_free = [&](int s, int rnd) -> bool {
      if (rnd == 0) return true;
      int freed = 1;
      if (lane == 0) freed = mbar_wait(&empty[s], (unsigned)((rnd - 1) & 1)) ? 1 : 0;
      return __shfl_sync(0xffffffffu, freed, 0) != 0;
    };
    auto entry = [&](long long tile, int k) -> int {
      const long long r = tile * TR + tid;
      return (tid < TR && tile < P.n_tiles && r < P.n_out) ? __ldg(P.nbr + (long long)k * P.n_out + r) : -1;
    };
    // flattened (tile, offset) walk with a two-deep prefetch of the row owner's rulebook entry
    long long tile_a = blockIdx.x;
    int k_a = 0;
    auto advance = [&](long long &tile, int &k) {
      if (++k == P.K) {
        k = 0;
        tile += gridDim.x;
      }
    };
    long long tile_b = tile_a, tile_c;
    int k_b = k_a, k_c;
    advance(tile_b, k_b);
    tile_c = tile_b;
    k_c = k_b;
    advance(tile_c, k_c);
    int v0 = entry(tile_a, k_a), v1 = entry(tile_b, k_b), v2;
    int issued_in_tile = 0;
    {
      // entries and warp counts of a group are published before the group's barrier and read after it;
      // the next group's are written while slow threads may still read this one's: two copies, by parity
      int par = 0;
      for (long long t = 0; t < my_tiles; par ^= 1) {
        v2 = entry(tile_c, k_c);
        const bool hit = (unsigned)v0 < (unsigned)P.n_in;
        if (v0 >= 0 && !hit) atomicOr(P.flags, FLAG_BAD_ROW);
        const unsigned hits = __ballot_sync(0xffffffffu, hit);
        if (warp < kWOwners) {
          ent[par * kWRows + tid] = hit ? v0 : -1;
          if (lane == 0) warp_cnt[par * 8 + warp] = __popc(hits);
        }
        if (producer_vote(!ok || *sh_abort)) break;
        int total = 0;
#pragma unroll
        for (int w = 0; w < kWOwners; ++w) total += warp_cnt[par * 8 + w];
        const bool tile_end = (k_a == P.K - 1);
        const bool zero_step = tile_end && total == 0 && issued_in_tile == 0;  // a tile must get one step
        if (total > 0 || zero_step) {
          // this thread's (row, 16-byte piece) items: four consecutive lanes take the four pieces of a row
          unsigned off[kWItems], size[kWItems];
          const unsigned char *src[kWItems];
#pragma unroll
          for (int i = 0; i < kWItems; ++i) {
            const int it = tid + i * kWProducers;
            const int r = (it >> 2) & (kWRows - 1), j = it & 3;
            const bool in_tile = it < kWRows * 4 && r < TR;
            const int v = in_tile ? ent[par * kWRows + r] : -1;
            off[i] = in_tile ? (unsigned)j * kWLbo + (unsigned)r * 16u : 0xFFFFFFFFu;
            size[i] = v >= 0 ? 16u : 0u;
            src[i] = P.in_split + (v >= 0 ? (size_t)v * P.ld_in * 4 : 0) + j * 16;
          }
          for (int s0 = 0; s0 < n_slices && ok; ++s0) {
            if (!slot_free(st, round)) {
              ok = false;
              break;
            }
            const unsigned stage = smem_u32(smem) + (unsigned)st * stage_bytes;
            if (tid == 0) {
              meta[st] = 0;
              mbar_expect_tx(&full[st], total_w);
              bulk_copy_g2s(stage, P.wprep + ((size_t)k_a * n_slices + s0) * total_w, total_w, &full[st]);
            }
            const unsigned g = stage + w_region;
#pragma unroll
            for (int i = 0; i < kWItems; ++i)
              if (off[i] != 0xFFFFFFFFu) {
                const unsigned char *q = src[i] + (size[i] ? (size_t)s0 * (kWSlice * 4) : 0);
                cp_async16(g + off[i], q, size[i]);
                if (TERMS == 3) cp_async16(g + kWTile + off[i], q + (size[i] ? 64 : 0), size[i]);
              }
            // this thread's arrival happens when its copies above have landed
            asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(&full[st])) : "memory");
            if (++st == NS) {
              st = 0;
              ++round;
            }
          }
          ++issued_in_tile;
        }
        if (tile_end && ok) {
          if (slot_free(st, round)) {
            if (tid == 0) {
              meta[st] = W_LAST_OF_TILE | (t == my_tiles - 1 ? W_LAST_OF_CTA : 0);
              mbar_arrive(&full[st]);  // stands in for the slab's transaction arrival
            }
            mbar_arrive(&full[st]);
            if (++st == NS) {
              st = 0;
              ++round;
            }
          } else {
            ok = false;
          }
          issued_in_tile = 0;
          ++t;
        }
        v0 = v1;
        v1 = v2;
        tile_a = tile_b;
        k_a = k_b;
        tile_b = tile_c;
        k_b = k_c;
        advance(tile_c, k_c);
      }
      // copies still in flight must land before the CTA's shared memory goes away
      asm volatile("cp.async.wait_all;" ::: "memory");
    }
    if (!ok) *sh_abort = 1;
  } else if (warp == kWMmaWarp) {
    // ==================================== MMA issue (one thread) ===============================
    if (lane == 0) {
      const unsigned idesc = wide_idesc(TR);
      const unsigned stage0 = smem_u32(smem);
      int st = 0, round = 0;
      bool ok = true;
      for (long long t = 0; t < my_tiles && ok; ++t) {
        const int ab = (n_acc == 2) ? (int)(t & 1) : 0;
        const long long use = (n_acc == 2) ? (t >> 1) : t;
        if (use > 0 && !mbar_wait(&acc_empty[ab], (unsigned)((use - 1) & 1))) {
          ok = false;
          break;
        }
        tc_fence_after();
        bool first = true;
        for (;;) {
          if (*sh_abort) {
            ok = false;
            break;
          }
          if (!mbar_wait(&full[st], (unsigned)(round & 1))) {
            ok = false;
            break;
          }
          // the producers' generic-proxy stores were acquired through the barrier; order them before
          // the tensor core's async-proxy reads
          fence_proxy_async_smem();
          tc_fence_after();
          const int flags = meta[st];
          if (flags & W_LAST_OF_TILE) {  // marker slot: no data, just the end of the tile
            tc_commit(&empty[st]);
            tc_commit(&acc_full[ab]);
            if (++st == NS) {
              st = 0;
              ++round;
            }
            break;
          }
          const unsigned w_addr = stage0 + (unsigned)st * stage_bytes;
          const unsigned g_addr = w_addr + w_region;
#pragma unroll
          for (int jj = 0; jj < 2; ++jj) {  // two K = 16 instructions per 32-plane step and product
            const unsigned long long dg_h = smem_desc(g_addr + jj * 2 * kWLbo, kWLbo, 128);
            const unsigned long long dg_m = smem_desc(g_addr + kWTile + jj * 2 * kWLbo, kWLbo, 128);
            const unsigned acc = (first && jj == 0) ? 0u : 1u;
            for (int mt = 0; mt < n_mt; ++mt) {
              const unsigned d = tmem_base + (unsigned)((ab * n_mt + mt) * kWRows);
              const unsigned w_mt = w_addr + (unsigned)mt * (kWPlanes / 8) * 512u + jj * 256;
              const unsigned long long dw_h = smem_desc(w_mt, 128, 512);
              tc_mma<true>(d, dw_h, dg_h, idesc, acc);
              if (TERMS == 3) {
                const unsigned long long dw_m = smem_desc(w_mt + w_bytes, 128, 512);
                tc_mma<true>(d, dw_h, dg_m, idesc, 1u);
                tc_mma<true>(d, dw_m, dg_h, idesc, 1u);
              }
            }
          }
          first = false;
          tc_commit(&empty[st]);
          if (++st == NS) {
            st = 0;
            ++round;
          }
        }
      }
      if (!ok) *sh_abort = 1;
    }
  } else if (warp >= kWEpilogue0 && warp < kWEpilogue0 + 4) {
    // ========================================= epilogue =======================================
    // TMEM lane = output plane, column = tile row; warp q of this group reads lanes 32q..32q+31
    // (the quadrant its warp id selects).  The 32 lanes hold 32 consecutive planes of one row:
    // a 128-byte coalesced store per row.
    const int quad = warp & 3;
    for (long long t = 0; t < my_tiles; ++t) {
      const int ab = (n_acc == 2) ? (int)(t & 1) : 0;
      const long long use = (n_acc == 2) ? (t >> 1) : t;
      int got = 1;
      if (lane == 0) got = (!*sh_abort && mbar_wait(&acc_full[ab], (unsigned)(use & 1))) ? 1 : 0;
      got = __shfl_sync(0xffffffffu, got, 0);
      if (!got) {
        *sh_abort = 1;
        break;
      }
      tc_fence_after();
      const long long row0 = (blockIdx.x + t * gridDim.x) * TR;
      const long long row_end = min(P.n_out, row0 + TR);
      for (int mt = 0; mt < n_mt; ++mt) {
        const int plane0 = mt * kWPlanes + quad * 32;
        if (plane0 >= P.cout) break;
        const int plane = plane0 + lane;
        const bool plane_ok = plane < P.cout;
        const float b = (P.bias && plane_ok) ? P.bias[plane] : 0.f;
        const float sc = (P.bn_scale && plane_ok) ? P.bn_scale[plane] : 1.f;
        const float sh = (P.bn_scale && plane_ok) ? P.bn_shift[plane] : 0.f;
        const float leak = P.leak;
#pragma unroll
        for (int n0 = 0; n0 < kWRows; n0 += 32) {
          if (n0 >= TR || row0 + n0 >= row_end) break;
          float v[32];
          tmem_ld32(tmem_base + ((unsigned)(quad * 32) << 16) + (unsigned)((ab * n_mt + mt) * kWRows + n0), v);
          if (plane_ok) {
            float *dst = P.out + (row0 + n0) * P.ld_out + plane;
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (row0 + n0 + i < row_end) {
                float y = v[i] + b;
                if (P.bn_scale) {  // separate multiply and add, as the stand-alone BatchNorm kernel rounds them
                  y = __fadd_rn(__fmul_rn(y, sc), sh);
                  y *= (y > 0.f) ? 1.f : leak;
                }
                dst[(long long)i * P.ld_out] = y;
              }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[ab]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (*sh_abort && tid == 0) atomicOr(P.flags, FLAG_TC_TIMEOUT);
  if (warp == kWMmaWarp) tmem_dealloc(tmem_base, kTmemCols);
}

// in [n][cin] fp32 -> out, per row and 32-plane slice: the 32 h = bf16(x) then the 32 m = bf16(x - h)
// (128 bytes, the size of the fp32 slice).  One thread per 8 planes: 32 bytes in, 16 + 16 out.
// pre_scale / pre_shift (optional): x is first taken through an eval-mode BatchNorm and its leaky ReLU,
// x <- act(x * scale[plane] + shift[plane]) with the roundings of the stand-alone operator: a BatchNorm in front of
// the convolution costs no pass of its own.
__device__ __forceinline__ float wide_pre_bn(float x, float sc, float sh, float leak) {
  const float y = __fadd_rn(__fmul_rn(x, sc), sh);
  return y * (y > 0.f ? 1.f : leak);
}

// in_b (optional): the input is the column-wise concatenation [in (planes_a) | in_b (cin - planes_a)] of two
// matrices (a JoinTable in front of the layer), read from where the two lie; planes_a a multiple of eight.
__global__ void __launch_bounds__(256)
k_wide_split_rows(const float *__restrict__ in, unsigned char *__restrict__ out, long long n_pieces, int cin,
                  const float *__restrict__ pre_scale, const float *__restrict__ pre_shift, float pre_leak,
                  const float *__restrict__ in_b, int planes_a) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n_pieces) return;
  const int ppr = cin / 8;  // pieces per row
  const long long row = idx / ppr;
  const int piece = (int)(idx % ppr), slice = piece >> 2, j = piece & 3;
  const float *src = !in_b ? in + row * cin + piece * 8
                           : (piece * 8 < planes_a ? in + row * planes_a + piece * 8
                                                   : in_b + row * (cin - planes_a) + (piece * 8 - planes_a));
  const float4 *p = reinterpret_cast<const float4 *>(src);
  float4 a = __ldg(p), b = __ldg(p + 1);
  if (pre_scale) {
    const float4 s0 = __ldg(reinterpret_cast<const float4 *>(pre_scale + piece * 8)), s1 = __ldg(reinterpret_cast<const float4 *>(pre_scale + piece * 8) + 1);
    const float4 h0 = __ldg(reinterpret_cast<const float4 *>(pre_shift + piece * 8)), h1 = __ldg(reinterpret_cast<const float4 *>(pre_shift + piece * 8) + 1);
    a.x = wide_pre_bn(a.x, s0.x, h0.x, pre_leak), a.y = wide_pre_bn(a.y, s0.y, h0.y, pre_leak);
    a.z = wide_pre_bn(a.z, s0.z, h0.z, pre_leak), a.w = wide_pre_bn(a.w, s0.w, h0.w, pre_leak);
    b.x = wide_pre_bn(b.x, s1.x, h1.x, pre_leak), b.y = wide_pre_bn(b.y, s1.y, h1.y, pre_leak);
    b.z = wide_pre_bn(b.z, s1.z, h1.z, pre_leak), b.w = wide_pre_bn(b.w, s1.w, h1.w, pre_leak);
  }
  uint4 h, m;
  split_bf16_pair(a.x, a.y, h.x, m.x);
  split_bf16_pair(a.z, a.w, h.y, m.y);
  split_bf16_pair(b.x, b.y, h.z, m.z);
  split_bf16_pair(b.z, b.w, h.w, m.w);
  unsigned char *q = out + (size_t)row * cin * 4 + (size_t)slice * (kWSlice * 4) + j * 16;
  *reinterpret_cast<uint4 *>(q) = h;
  *reinterpret_cast<uint4 *>(q + 64) = m;
}

size_t wide_stage_bytes(int terms, int cout, int rows) {
  const int parts = terms == 3 ? 2 : 1;
  const size_t w = (size_t)cout * kWSlice * 2 * parts;
  return ((w + 1023) & ~(size_t)1023) + (size_t)4 * (rows * 16 + 32) * parts;
}
// Rows per tile.  Measured alternatives that lost: 128-row tiles (N = 128 instructions are as efficient, but every
// tile brings its own weight slabs: a third more operand bytes per row through shared memory; 0.47 against 0.36 ms on
// 96 -> 96 planes at 154 k rows with the copy-only producers, 0.65 against 0.56 with the earlier ones), 24 producer
// warps (0.45 against 0.44 ms) and two CTAs per SM with half the ring and one accumulator each (0.45 ms).
int wide_rows() { return 256; }
constexpr size_t kWideControlBytes = 4096;  // barriers, step flags, and the rulebook entries of two groups
constexpr size_t kWideSmemBudget = 226 * 1024;

}  // namespace

// The split pass on its own (also used by the per-tile kernel of conv_tc.cu): cin a multiple of 32, `out` holds
// n_rows * cin * 4 bytes.
int split_rows_bf16(const float *in, unsigned char *out, long long n_rows, int cin, cudaStream_t stream,
                    const float *pre_scale, const float *pre_shift, float pre_leak, const float *in_b, int planes_a) {
  SCN_REQUIRE(!in_b || (planes_a > 0 && planes_a < cin && planes_a % 8 == 0 && (uintptr_t)in_b % 16 == 0),
              SCN_ERR_BAD_ARG, "joined input: the first part must have a multiple of eight planes");
  const long long n_pieces = n_rows * (cin / 8);
  if (n_pieces <= 0) return SCN_OK;
  SCN_REQUIRE(!pre_scale || ((uintptr_t)pre_scale % 16 == 0 && (uintptr_t)pre_shift % 16 == 0), SCN_ERR_BAD_ARG,
              "scale / shift of the BatchNorm in front must be 16-byte aligned");
  SCN_LAUNCH(k_wide_split_rows, (unsigned)ceil_div(n_pieces, 256LL), 256, 0, stream, in, out, n_pieces, cin, pre_scale,
             pre_shift, pre_leak, in_b, planes_a);
  SCN_CUDA_CHECK(cudaGetLastError());
  return SCN_OK;
}

bool conv_wide_supported(int K, int cin, int cout, int groups, int precision, long long n_in) {
  (void)K;
  if (precision != SCN_PRECISION_TF32X3 && precision != SCN_PRECISION_BF16) return false;
  if (precision == SCN_PRECISION_TF32X3 && split_mode_of_env(TC_BF16X3) != TC_BF16X3) return false;
  if (getenv("SCN_CONV_WIDE") && atoi(getenv("SCN_CONV_WIDE")) == 0) return false;
  if (groups != 1 || cin % kWSlice != 0 || cout % 8 != 0 || cout < 8 || cout > 256 || n_in < 1) return false;
  const int terms = precision == SCN_PRECISION_TF32X3 ? 3 : 1;
  return (kWideSmemBudget - kWideControlBytes) / wide_stage_bytes(terms, cout, wide_rows()) >= 2;
}

// out [n_out, cout] = act((bias + sum_k in[table[k][.]] @ W[k]) * bn_scale + bn_shift); bn_scale may be
// null (then no scaling and, with leak == 1, no activation: the plain convolution).
int conv_forward_wide(const float *in, long long n_in, float *out, long long n_out, const float *weight,
                      const float *bias, const float *bn_scale, const float *bn_shift, float leak, const int *table,
                      int K, int cin, int cout, int precision, int *flags, cudaStream_t stream,
                      const float *pre_scale, const float *pre_shift, float pre_leak, const float *in_b, int planes_a) {
  if (n_out == 0) return SCN_OK;
  const int terms = precision == SCN_PRECISION_TF32X3 ? 3 : 1;
  SCN_REQUIRE((uintptr_t)in % 16 == 0, SCN_ERR_BAD_ARG, "tensor-core path needs a 16-byte aligned input matrix");
  SCN_REQUIRE(n_in < (1ll << 31) && n_out < (1ll << 31), SCN_ERR_UNSUPPORTED, "row count above 2^31");
  const int rows = wide_rows();
  const size_t stage = wide_stage_bytes(terms, cout, rows);
  const size_t budget = kWideSmemBudget;
  const int stages = (int)std::min<size_t>(kWMaxStages, (budget - kWideControlBytes) / stage);
  SCN_REQUIRE(stages >= 2, SCN_ERR_UNSUPPORTED, "tensor-core path: stage does not fit shared memory");
  const int parts = terms == 3 ? 2 : 1;
  const int mode = terms == 3 ? TC_BF16X3 : TC_BF16;
  WeightImage wi;
  bool build = true;
  SCN_TRY(weight_image_get(WIMG_TC, K, cin, cout, kWSlice * 16 + mode, (size_t)K * cin * cout * 2 * parts, stream, &wi,
                           &build));
  unsigned char *wprep = (unsigned char *)wi.ptr;
  if (build) SCN_TRY(prepare_weights(weight, wprep, K, cin, cout, kWSlice, mode, stream));

  // the input rows as bf16 parts, made once per call (every row is gathered by up to K output rows)
  unsigned char *split = nullptr;
  SCN_TRY(device_alloc((void **)&split, (size_t)n_in * cin * 4, stream));
  {
    const int st = split_rows_bf16(in, split, n_in, cin, stream, pre_scale, pre_shift, pre_leak, in_b, planes_a);
    if (st != SCN_OK) {
      device_free(split, stream);
      return st;
    }
  }
  WideParams P;
  P.in = in;
  P.in_split = split;
  P.ld_in = cin;
  P.n_in = n_in;
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
  P.n_stages = stages;
  P.flags = flags;
  static int n_sm[64] = {0};
  int dev = 0;
  SCN_CUDA_CHECK(cudaGetDevice(&dev));
  SCN_REQUIRE(dev >= 0 && dev < 64, SCN_ERR_UNSUPPORTED, "device index %d unsupported", dev);
  if (!n_sm[dev]) {
    int sms = 0;
    SCN_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const int b = (int)kWideSmemBudget;
#define SCN_WIDE_ATTR(TRC)                                                                                            \
  SCN_CUDA_CHECK(cudaFuncSetAttribute(k_conv_wide<1, 256, 12, TRC>, cudaFuncAttributeMaxDynamicSharedMemorySize, b)); \
  SCN_CUDA_CHECK(cudaFuncSetAttribute(k_conv_wide<3, 256, 12, TRC>, cudaFuncAttributeMaxDynamicSharedMemorySize, b));
    SCN_WIDE_ATTR(0) SCN_WIDE_ATTR(128) SCN_WIDE_ATTR(144) SCN_WIDE_ATTR(160) SCN_WIDE_ATTR(176) SCN_WIDE_ATTR(192)
    SCN_WIDE_ATTR(208) SCN_WIDE_ATTR(224) SCN_WIDE_ATTR(240) SCN_WIDE_ATTR(256)
#undef SCN_WIDE_ATTR
    n_sm[dev] = sms;
  }
  // Tile height: with w = the number of tiles of full height the busiest SM would get, the smallest multiple of 16
  // rows that still covers the level with w tiles per SM -- every SM then gets the same number of tiles (601 tiles
  // of 256 rows leave 5 on nine SMs and 4 on the rest; 740 tiles of 208 rows are 5 on each, a fifth fewer rows on
  // the longest SM).  SCN_WIDE_EVEN=0 keeps full-height tiles.
  P.tile_rows = rows;
  if (!(getenv("SCN_WIDE_EVEN") && atoi(getenv("SCN_WIDE_EVEN")) == 0)) {
    const long long waves = ceil_div(ceil_div(n_out, rows), n_sm[dev]);
    const long long even = ceil_div(ceil_div(n_out, waves * n_sm[dev]), 16) * 16;
    P.tile_rows = (int)std::max<long long>(64, std::min<long long>(rows, even));
  }
  P.n_tiles = ceil_div(n_out, P.tile_rows);
  const unsigned grid = (unsigned)std::min<long long>(P.n_tiles, n_sm[dev]);
  // one CTA per SM by construction: it asks for the whole shared memory and owns all 512 TMEM columns
  // the heights two or more tiles per SM lead to (128 rows and up) have kernels of their own
#define SCN_WIDE_LAUNCH(TRC)                                                                 \
  if (terms == 3)                                                                            \
    SCN_LAUNCH((k_conv_wide<3, 256, 12, TRC>), grid, 17 * 32, budget, stream, P);            \
  else                                                                                       \
    SCN_LAUNCH((k_conv_wide<1, 256, 12, TRC>), grid, 17 * 32, budget, stream, P);
  switch (P.tile_rows) {
    case 256: SCN_WIDE_LAUNCH(256) break;
    case 240: SCN_WIDE_LAUNCH(240) break;
    case 224: SCN_WIDE_LAUNCH(224) break;
    case 208: SCN_WIDE_LAUNCH(208) break;
    case 192: SCN_WIDE_LAUNCH(192) break;
    case 176: SCN_WIDE_LAUNCH(176) break;
    case 160: SCN_WIDE_LAUNCH(160) break;
    case 144: SCN_WIDE_LAUNCH(144) break;
    case 128: SCN_WIDE_LAUNCH(128) break;
    default: SCN_WIDE_LAUNCH(0) break;
  }
#undef SCN_WIDE_LAUNCH
  const cudaError_t launch_err = cudaGetLastError();
  device_free(split, stream);
  SCN_CUDA_CHECK(launch_err);
  SCN_TRY(weight_image_put(wi, stream));
  return SCN_OK;
}

}  // namespace scn
