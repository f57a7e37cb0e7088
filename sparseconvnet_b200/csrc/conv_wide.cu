// Persistent tcgen05 sparse convolution with bf16 operands made in registers: the kernel for wide
// layers (64 output planes and more) on levels with many rows, in the fp32-class three-term form
// and in the single-pass bf16 mode.
//
// Same mathematics and orientation as conv_tc.cu / conv_tma.cu (output stationary,
// D^T[planes x 256 rows] += W_k^T G_k^T with the accumulators in TMEM; the reference's per-offset
// gather / GEMM / scatter-add is CPU/Convolution.cpp:137-148, CUDA/Convolution.cu:57-233).  What is
// different is how the gathered rows reach the tensor core.  A tcgen05.mma of 128 x 256 x 16 bf16
// takes 128 cycles (measured by scn_tc_probe_mma: max(56, N / 2) cycles whatever M and kind), so a
// 32-plane step of the three-term form is 6 instructions = 768 cycles, and everything else has to
// fit under that:
//
//   * the fp32 rows never touch shared memory.  The twelve producer warps read the input rows that
//     have a rule with 128-bit loads into registers -- all loads of a (tile, offset) group's next
//     two steps are issued before the first is used, so a thread has up to 12 loads in flight --
//     split every value into h = bf16(x) and m = bf16(x - h), and store the two bf16 tiles straight
//     in the K-major core-matrix layout the instruction reads; rows without a rule get zero
//     stores.  Shared-memory traffic per step: 32 KB of stores + 72 KB of operand reads, against
//     32 + 64 + 144 KB when a raw fp32 tile is staged and converted by a second set of warps;
//   * a step is 44-48 KB (two bf16 tiles + the two weight slabs), so the ring holds four steps;
//   * per filter offset the 256 row-owning threads compact the rows that do have a rule (ballots +
//     one prefix over eight warp counts); offsets for which the tile has no rule cost nothing;
//   * one thread issues the MMAs (h h, h m, m h per 16 planes) into one of two TMEM accumulators
//     while four epilogue warps drain the other (tcgen05.ld -> bias -> optional per-plane
//     scale / shift / leaky ReLU of a following BatchNorm -> coalesced stores, each row once).
//
// Error of the three-term form: the dropped products m m and x_l w (x_l = x - h - m) are 2^-17 of a
// product; measured 5e-6 to 9e-6 of the largest output per layer against the reference's CPU
// operator, 3e-5 through the four 81-offset layers of the 4-D stack -- better than the three-pass
// tf32 split on the same instruction, whose high part is a truncation.
//
// Where the time goes (96 -> 96 planes, 154 k rows, 0.44 ms; the kernel it replaces took 0.75 ms): the
// MMA thread waits for full steps two thirds of the time; phase timers in the producers showed the work
// of a (tile, offset) group spread over its barriers, the list reads, the loads, the conversion and the
// zero stores with no single dominant term, and ncu shows no saturated pipe (tensor 38 %, LSU 34 %,
// issue slots 39 %): 2 900 warp instructions per step at 1.5 issued per clock.  What moved it: reading a
// row's 128 bytes with four neighbouring lanes (one line per row and load instruction instead of one
// sector per lane: 0.56 -> 0.44 ms) and two block barriers per group instead of three.
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
  int *flags;
};

__host__ __device__ inline unsigned wide_idesc(int rows) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(rows >> 3) << 17) | ((unsigned)(kWPlanes >> 4) << 24);
}

// TERMS 3: h h + h m + m h (fp32-class); 1: h h (plain bf16).  ROWS: output rows per tile.  PW: producer warps.
template <int TERMS, int ROWS, int PW>
__global__ void __launch_bounds__((PW + 5) * 32, 1) k_conv_wide(WideParams P) {
  constexpr int kWProducerWarps = PW, kWProducers = PW * 32;
  constexpr int kWEpilogue0 = PW, kWMmaWarp = PW + 4;
  constexpr int kWBatch = 2;  // steps whose loads are in flight together
  constexpr unsigned kTmemCols = 512u;
  constexpr int kParts = TERMS == 3 ? 2 : 1;
  constexpr int kWRows = ROWS;
  // A bf16 tile of gathered rows [ROWS x 32 planes] is stored as four planes of 16-byte pieces (piece j =
  // 8 input planes of every row): piece j of row r at j * kWLbo + r * 16.  That is the K-major
  // core-matrix layout with 128 bytes between 8-row groups and kWLbo between the K pieces; the 32
  // bytes of padding in kWLbo put the four pieces of a row on different banks, so the four lanes that
  // convert one row (they read its 128 contiguous bytes: one line per row and load instruction) store
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
  int *list_row = reinterpret_cast<int *>(ctl + 512);  // [256] tile rows with a rule, then
  int *list_idx = list_row + kWMaxRows;                // [256] their input rows
  int *list_miss = list_idx + kWMaxRows;               // [256] tile rows without a rule
  int *warp_cnt = list_miss + kWMaxRows;               // [8]

  if (tid == 0) {
    for (int s = 0; s < NS; ++s) {
      mbar_init(&full[s], kWProducerWarps + 1);
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

  if (warp < kWProducerWarps) {
    // =============================== producers: gather, split, store ===========================
    int st = 0, round = 0;
    bool ok = true;
    auto producer_sync = [] { asm volatile("bar.sync 1, %0;" ::"n"(kWProducers) : "memory"); };
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
      const long long r = tile * kWRows + tid;
      return (tid < kWRows && tile < P.n_tiles && r < P.n_out) ? __ldg(P.nbr + (long long)k * P.n_out + r) : -1;
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
    for (long long t = 0; t < my_tiles;) {
      v2 = entry(tile_c, k_c);
      const bool hit = (unsigned)v0 < (unsigned)P.n_in;
      if (v0 >= 0 && !hit) atomicOr(P.flags, FLAG_BAD_ROW);
      const unsigned hits = __ballot_sync(0xffffffffu, hit);
      // Two barriers per group.  The first also carries the decision to stop (a bounded wait ran out
      // somewhere): it is a reduction, so every producer gets the same answer.  Behind it the lists of
      // the previous group are free to be rewritten: nobody passes it before all have finished that group.
      if (lane == 0 && warp < kWOwners) warp_cnt[warp] = __popc(hits);
      if (producer_vote(!ok || *sh_abort)) break;
      int base = 0, total = 0;
#pragma unroll
      for (int w = 0; w < kWOwners; ++w) {
        const int cw = warp_cnt[w];
        if (w < warp) base += cw;
        total += cw;
      }
      const bool tile_end = (k_a == P.K - 1);
      const bool zero_step = tile_end && total == 0 && issued_in_tile == 0;  // a tile must get one step
      if (total > 0 || zero_step) {
        if (warp < kWOwners) {
          const unsigned lt = (1u << lane) - 1;
          if (hit) {
            const int pos = base + __popc(hits & lt);
            list_row[pos] = tid;
            list_idx[pos] = v0;
          } else {
            list_miss[32 * warp - base + __popc(~hits & lt)] = tid;
          }
        }
        producer_sync();
        const int n_miss = kWRows - total;
        const int n_hit_items = total * 4, n_miss_items = n_miss * 4;
        // This thread's items of every step of the group: (row, 16-byte piece) -> offset inside a bf16
        // tile, source.  Four consecutive lanes take the four pieces of one row.
        unsigned off[kWItems];
        const float *src[kWItems];
#pragma unroll
        for (int i = 0; i < kWItems; ++i) {
          const int it = tid + i * kWProducers;
          src[i] = nullptr;
          off[i] = 0;
          if (it < n_hit_items) {
            const int e = it >> 2, j = it & 3, r = list_row[e];
            off[i] = (unsigned)j * kWLbo + (unsigned)r * 16u;
            src[i] = P.in + (long long)list_idx[e] * P.ld_in + j * 8;
          }
        }
        for (int s0 = 0; s0 < n_slices && ok; s0 += kWBatch) {
          const int nb = min(kWBatch, n_slices - s0);
          // all loads of the batch first: up to kWItems x kWBatch x 2 128-bit loads in flight per thread
          float4 x[kWBatch][kWItems][2];
#pragma unroll
          for (int b = 0; b < kWBatch; ++b)
#pragma unroll
            for (int i = 0; i < kWItems; ++i)
              if (b < nb && src[i]) {
                const float4 *p = reinterpret_cast<const float4 *>(src[i] + (s0 + b) * kWSlice);
                x[b][i][0] = __ldg(p);
                x[b][i][1] = __ldg(p + 1);
              }
#pragma unroll
          for (int b = 0; b < kWBatch; ++b) {
            if (b >= nb || !ok) continue;
            if (!slot_free(st, round)) {
              ok = false;
              continue;
            }
            unsigned char *stage = smem + (size_t)st * stage_bytes;
            if (tid == 0) {
              meta[st] = 0;
              mbar_expect_tx(&full[st], total_w);
              bulk_copy_g2s(smem_u32(stage), P.wprep + ((size_t)k_a * n_slices + (s0 + b)) * total_w, total_w, &full[st]);
            }
            unsigned char *g = stage + w_region;
#pragma unroll
            for (int i = 0; i < kWItems; ++i)
              if (src[i]) {
                uint4 h, m;
                split_bf16_pair(x[b][i][0].x, x[b][i][0].y, h.x, m.x);
                split_bf16_pair(x[b][i][0].z, x[b][i][0].w, h.y, m.y);
                split_bf16_pair(x[b][i][1].x, x[b][i][1].y, h.z, m.z);
                split_bf16_pair(x[b][i][1].z, x[b][i][1].w, h.w, m.w);
                *reinterpret_cast<uint4 *>(g + off[i]) = h;
                if (TERMS == 3) *reinterpret_cast<uint4 *>(g + kWTile + off[i]) = m;
              }
            for (int it = tid; it < n_miss_items; it += kWProducers) {
              const unsigned o = (unsigned)(it & 3) * kWLbo + (unsigned)list_miss[it >> 2] * 16u;
              *reinterpret_cast<uint4 *>(g + o) = make_uint4(0, 0, 0, 0);
              if (TERMS == 3) *reinterpret_cast<uint4 *>(g + kWTile + o) = make_uint4(0, 0, 0, 0);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&full[st]);  // one arrival per warp (release)
            if (++st == NS) {
              st = 0;
              ++round;
            }
          }
        }
        ++issued_in_tile;
      }
      if (tile_end && ok) {
        // end-of-tile marker: a slot without data that tells the MMA thread to hand the accumulator
        // to the epilogue
        if (slot_free(st, round)) {
          if (tid == 0) {
            meta[st] = W_LAST_OF_TILE | (t == my_tiles - 1 ? W_LAST_OF_CTA : 0);
            mbar_arrive(&full[st]);  // stands in for the slab's transaction arrival
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(&full[st]);
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
    if (!ok) *sh_abort = 1;
  } else if (warp == kWMmaWarp) {
    // ==================================== MMA issue (one thread) ===============================
    if (lane == 0) {
      const unsigned idesc = wide_idesc(kWRows);
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
      const long long row0 = (blockIdx.x + t * gridDim.x) * kWRows;
      for (int mt = 0; mt < n_mt; ++mt) {
        const int plane0 = mt * kWPlanes + quad * 32;
        if (plane0 >= P.cout) break;
        const int plane = plane0 + lane;
        const bool plane_ok = plane < P.cout;
        const float b = (P.bias && plane_ok) ? P.bias[plane] : 0.f;
        const float sc = (P.bn_scale && plane_ok) ? P.bn_scale[plane] : 1.f;
        const float sh = (P.bn_scale && plane_ok) ? P.bn_shift[plane] : 0.f;
        const float leak = P.leak;
        for (int n0 = 0; n0 < kWRows; n0 += 32) {
          if (row0 + n0 >= P.n_out) break;
          float v[32];
          tmem_ld32(tmem_base + ((unsigned)(quad * 32) << 16) + (unsigned)((ab * n_mt + mt) * kWRows + n0), v);
          if (plane_ok) {
            float *dst = P.out + (row0 + n0) * P.ld_out + plane;
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (row0 + n0 + i < P.n_out) {
                float y = (v[i] + b) * sc + sh;
                y = y > 0.f ? y : y * leak;
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

size_t wide_stage_bytes(int terms, int cout, int rows) {
  const int parts = terms == 3 ? 2 : 1;
  const size_t w = (size_t)cout * kWSlice * 2 * parts;
  return ((w + 1023) & ~(size_t)1023) + (size_t)4 * (rows * 16 + 32) * parts;
}
// Rows per tile.  Measured alternatives that lost: 128-row tiles (N = 128 instructions are as efficient, but the
// per-group work of the producers doubles: 0.65 against 0.56 ms on 96 -> 96 planes at 154 k rows), 24 producer
// warps (0.45 against 0.44 ms) and two CTAs per SM with half the ring and one accumulator each (0.45 ms).
int wide_rows() { return 256; }
constexpr size_t kWideControlBytes = 4096;  // barriers, step flags, and the producers' row lists
constexpr size_t kWideSmemBudget = 226 * 1024;

}  // namespace

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
                      int K, int cin, int cout, int precision, int *flags, cudaStream_t stream) {
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

  WideParams P;
  P.in = in;
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
  P.n_tiles = ceil_div(n_out, rows);
  P.flags = flags;
  static int n_sm[64] = {0};
  int dev = 0;
  SCN_CUDA_CHECK(cudaGetDevice(&dev));
  SCN_REQUIRE(dev >= 0 && dev < 64, SCN_ERR_UNSUPPORTED, "device index %d unsupported", dev);
  if (!n_sm[dev]) {
    int sms = 0;
    SCN_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const int b = (int)kWideSmemBudget;
    SCN_CUDA_CHECK(cudaFuncSetAttribute(k_conv_wide<1, 256, 12>, cudaFuncAttributeMaxDynamicSharedMemorySize, b));
    SCN_CUDA_CHECK(cudaFuncSetAttribute(k_conv_wide<3, 256, 12>, cudaFuncAttributeMaxDynamicSharedMemorySize, b));
    n_sm[dev] = sms;
  }
  const unsigned grid = (unsigned)std::min<long long>(P.n_tiles, n_sm[dev]);
  // one CTA per SM by construction: it asks for the whole shared memory and owns all 512 TMEM columns
  if (terms == 3)
    SCN_LAUNCH((k_conv_wide<3, 256, 12>), grid, 17 * 32, budget, stream, P);
  else
    SCN_LAUNCH((k_conv_wide<1, 256, 12>), grid, 17 * 32, budget, stream, P);
  SCN_CUDA_CHECK(cudaGetLastError());
  SCN_TRY(weight_image_put(wi, stream));
  return SCN_OK;
}

}  // namespace scn
