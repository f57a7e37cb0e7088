// Persistent tensor-core sparse convolution for sm_100a: TMA row gather (tile::gather4),
// tcgen05.mma with double-buffered accumulators in TMEM.
//
// Same mathematics and orientation as conv_tc.cu (output stationary, D^T[planes x 256 rows] +=
// W_k^T * G_k^T, planes on the TMEM lanes), restructured so that nothing a tile needs is on
// the critical path of the tensor core:
//
//   * one CTA per SM walks tiles of 256 output rows (static round robin);
//   * gather: the copy pipe of the SM moves one 16-byte cp.async lane request per cycle, which
//     caps a cp.async gather at ~20 B/clk.  Here the TMA engine fetches the rows instead: one
//     `cp.async.bulk.tensor.2d...tile::gather4` brings four 128-byte row slices, named by four
//     row indices, into the 128-byte-swizzled K-major layout the MMA reads; a row index of -1
//     (no rule for this offset) is out of bounds for the tensor map and arrives as zeros.  One
//     warp issues 64 such copies per step -- two per lane -- with the indices it reads straight
//     from the dense rulebook (prefetched two offsets ahead), and skips offsets for which the
//     tile has no rule at all;
//   * the same warp issues the weight slab's bulk copy; both land on one transaction barrier;
//   * one thread issues the MMAs (4 x K=8 tf32, or 2 x K=16 bf16 per 32-plane slice, per 128
//     output planes) and commits to the stage's `empty` barrier;
//   * TF32X3 / BF16 need a pass over the gathered rows (low part / conversion): four transform
//     warps do it between the copy barrier and the MMA;
//   * epilogue warps drain one TMEM accumulator (tcgen05.ld -> +bias -> coalesced stores,
//     each row once) while the MMAs of the next tile fill the other.
//
// Every wait is bounded: on expiry the role raises the abort flag, everybody leaves their
// loops, tensor memory is freed and the host sees FLAG_TC_TIMEOUT through scn_md_poll_errors.
#include <cuda.h>
#include <stdlib.h>

#include <algorithm>

#include "metadata.cuh"
#include "tc_ptx.cuh"

namespace scn {

constexpr int kRows = 256;        // output rows per tile = MMA N
constexpr int kPlanes = 128;      // output planes per MMA = M
constexpr int kSlice = 32;        // input planes per step (128 bytes of fp32 per row)
constexpr int kGBytes = kRows * kSlice * 4;  // 32 KB of gathered fp32 rows per stage
constexpr int kMaxStages = 8;

// warps 0-7 gather (cp.async mode: all eight; TMA mode: warp 0 alone), 8-11 transform, 12-15
// epilogue (their warp id mod 4 selects the TMEM lane quadrant 0-3), 16 MMA
enum : int { WARP_PRODUCER = 0, N_PRODUCER_WARPS = 8, WARP_TRANSFORM0 = 8, WARP_EPILOGUE0 = 12, WARP_MMA = 16,
             N_WARPS = 17 };
enum : int { META_LAST_OF_TILE = 1, META_LAST_OF_CTA = 2 };

struct TmaParams {
  const float *in;  // cp.async gather only (the TMA gather goes through the tensor map)
  int ld_in;
  long long n_in;
  float *out;
  long long n_out;
  int ld_out;
  const unsigned char *wprep;
  const float *bias;
  const int *nbr;  // [K][n_out]
  int K, cin, cout;
  int n_stages;
  long long n_tiles;
  int *flags;
};

__device__ __forceinline__ void tma_gather4(unsigned dst, const CUtensorMap *map, int col, int r0, int r1, int r2,
                                            int r3, unsigned long long *bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cta.global.tile::gather4.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, "
      "%4, %5, %6}], [%7];" ::"r"(dst),
      "l"(map), "r"(col), "r"(r0), "r"(r1), "r"(r2), "r"(r3), "r"(smem_u32(bar))
      : "memory");
}
// K-major operand in the 128-byte swizzle: rows of 128 bytes, 8-row atoms of 1024 bytes.
__device__ __forceinline__ unsigned long long smem_desc_sw128(unsigned addr) {
  unsigned long long d = 0;
  d |= (unsigned long long)((addr >> 4) & 0x3FFF);
  d |= (unsigned long long)1 << 16;            // leading byte offset: unused for swizzled K-major
  d |= (unsigned long long)(1024 >> 4) << 32;  // stride between 8-row atoms
  d |= 1ull << 46;                             // descriptor version
  d |= 2ull << 61;                             // SWIZZLE_128B
  return d;
}
__host__ __device__ inline unsigned instr_desc_tma(bool bf16) {
  unsigned fmt = bf16 ? 1u : 2u;
  return (1u << 4) | (fmt << 7) | (fmt << 10) | ((unsigned)(kRows >> 3) << 17) | ((unsigned)(kPlanes >> 4) << 24);
}

template <int MODE, bool TMA_GATHER>
__global__ void __launch_bounds__(N_WARPS * 32, 1)
k_conv_tma(const __grid_constant__ CUtensorMap in_map, TmaParams P) {
  constexpr bool kBf16 = (MODE == TC_BF16 || MODE == TC_BF16X3);     // bf16 operands, made by the transform warps
  constexpr bool kSplit = (MODE == TC_TF32X3 || MODE == TC_BF16X3);  // two parts per operand, three products
  constexpr bool kB3 = (MODE == TC_BF16X3);
  constexpr bool kTransform = kBf16 || kSplit;
  constexpr int kEsize = kBf16 ? 2 : 4;
  constexpr unsigned kAuxBytes = kSplit ? kGBytes : (kBf16 ? kGBytes / 2 : 0);
  // TC_BF16X3 with the cp.async gather: the tensor core never reads the raw fp32 tile, only the two bf16 tiles
  // the transform warps make of it, so the producers copy the rows that have a rule and nothing else -- no zero
  // stores -- and leave a 256-bit mask of those rows with the stage; the transform warps write zeros for the
  // others without reading them.
  constexpr bool kMasked = kB3 && !TMA_GATHER;

  extern __shared__ __align__(1024) unsigned char smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int NS = P.n_stages;
  const int n_slices = P.cin / kSlice;
  const unsigned w_bytes = (unsigned)P.cout * kSlice * kEsize;
  const unsigned total_w = w_bytes * (kSplit ? 2 : 1);
  // stage: [W (| W_lo) | pad | G raw 32 KB | aux (low part / bf16 tile)].  G starts on a
  // 1024-byte boundary (swizzle atoms).  The weight slab comes first because an MMA always
  // reads 128 weight rows: with fewer output planes the rows past the slab are the gathered
  // rows behind it -- in bounds, and they only reach TMEM lanes that are never read back.
  const unsigned w_region = (total_w + 1023u) & ~1023u;
  const unsigned stage_bytes = w_region + kGBytes + kAuxBytes;
  const int n_mt = (P.cout + kPlanes - 1) / kPlanes;
  const int n_acc = n_mt == 1 ? 2 : 1;  // accumulator buffers in TMEM (512 columns in all)

  unsigned char *ctl = smem + (size_t)NS * stage_bytes;
  unsigned long long *full = reinterpret_cast<unsigned long long *>(ctl);  // [NS] copies landed
  unsigned long long *full_t = full + kMaxStages;                          // [NS] transform done
  unsigned long long *empty = full_t + kMaxStages;                         // [NS] MMAs done
  unsigned long long *acc_full = empty + kMaxStages;                       // [2]
  unsigned long long *acc_empty = acc_full + 2;                            // [2]
  int *meta = reinterpret_cast<int *>(acc_empty + 2);                      // [NS] step flags
  unsigned *sh_tmem = reinterpret_cast<unsigned *>(meta + kMaxStages);
  volatile int *sh_abort = reinterpret_cast<volatile int *>(sh_tmem + 1);

  if (tid == 0) {
    for (int s = 0; s < NS; ++s) {
      mbar_init(&full[s], TMA_GATHER ? 1 : N_PRODUCER_WARPS * 32 + 1);
      mbar_init(&full_t[s], 4);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);
    }
    *sh_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == WARP_MMA) tmem_alloc(sh_tmem, 512u);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem_base = *sh_tmem;
  const long long my_tiles =
      ((long long)blockIdx.x < P.n_tiles) ? (P.n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;

  if (!TMA_GATHER && warp < N_PRODUCER_WARPS) {
    // ============================ cp.async gather (eight warps) + weight slab ==================
    // The copy pipe retires cp.async at roughly one warp instruction per 27 cycles however few
    // of its lanes are active, so the gather must not spend instructions on rows that have no
    // rule (two thirds of a tile on surface data).  Per filter offset the 256 threads -- thread t
    // owns tile row t -- compact the rows that do have a rule (warp ballots + one prefix over
    // eight warp counts) into a list in shared memory; the copies then walk the list, eight
    // 16-byte chunks per row, 32 busy lanes per instruction.  The chunk goes where the 128-byte
    // swizzle puts it (position c ^ (row & 7) inside the row), the layout the MMA's descriptor
    // names.  Rows without a rule are zeroed with plain 128-bit stores (4 cycles per warp
    // instruction).  The copies signal the stage barrier themselves when they land.
    // The rulebook entry of (offset k, row t) is read two offsets ahead.
    int *list_row = reinterpret_cast<int *>(ctl + 512);   // [256] tile rows with a rule, then
    int *list_idx = list_row + kRows;                     // [256] their input rows
    int *list_miss = list_idx + kRows;                    // [256] tile rows without a rule
    int *warp_cnt = list_miss + kRows;                    // [8]
    unsigned *hit_mask = reinterpret_cast<unsigned *>(warp_cnt + N_PRODUCER_WARPS);  // [NS][8]
    int st = 0, round = 0;
    bool ok = true;
    auto producer_sync = [] { asm volatile("bar.sync 1, %0;" ::"n"(N_PRODUCER_WARPS * 32) : "memory"); };
    // barrier + OR over the producers: every producer thread gets the same answer, so they leave
    // the loop together (a warp that left alone would strand the others at the next barrier)
    auto producer_vote = [](bool x) -> bool {
      unsigned r;
      asm volatile(
          "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 p, %1, 0;\n\tbar.red.or.pred q, 1, %2, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
          : "=r"(r)
          : "r"((unsigned)x), "n"(N_PRODUCER_WARPS * 32)
          : "memory");
      return r != 0;
    };
    // one ring slot: wait until it is free, weight slab (or nothing for a marker), flags
    auto open_stage = [&](int k, int slice, int flags, bool marker) -> unsigned char * {
      if (round > 0) {
        int freed = 1;
        if (lane == 0) freed = mbar_wait(&empty[st], (unsigned)((round - 1) & 1)) ? 1 : 0;
        freed = __shfl_sync(0xffffffffu, freed, 0);
        if (!freed) {
          ok = false;
          return nullptr;
        }
      }
      unsigned char *stage = smem + (size_t)st * stage_bytes;
      if (tid == 0) {
        meta[st] = flags;
        if (marker) {
          mbar_arrive(&full[st]);
        } else {
          mbar_expect_tx(&full[st], total_w);
          bulk_copy_g2s(smem_u32(stage), P.wprep + ((size_t)k * n_slices + slice) * total_w, total_w, &full[st]);
        }
      }
      return stage;
    };
    auto close_stage = [&] {
      asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(&full[st])) : "memory");
      if (++st == NS) {
        st = 0;
        ++round;
      }
    };
    auto entry = [&](long long tile, int k) -> int {
      const long long r = tile * kRows + tid;
      return (tile < P.n_tiles && r < P.n_out) ? __ldg(P.nbr + (long long)k * P.n_out + r) : -1;
    };
    // flattened (tile, offset) walk with a two-deep prefetch of this thread's rulebook entry
    long long tile_a = blockIdx.x;  // position of v0
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
      // everybody is done with the previous offset's lists; stop together on a failure
      if (producer_vote(!ok || *sh_abort)) break;
      if (lane == 0) warp_cnt[warp] = __popc(hits);
      producer_sync();
      int base = 0, total = 0;
#pragma unroll
      for (int w = 0; w < N_PRODUCER_WARPS; ++w) {
        const int cw = warp_cnt[w];
        if (w < warp) base += cw;
        total += cw;
      }
      const bool tile_end = (k_a == P.K - 1);
      bool zero_step = tile_end && total == 0 && issued_in_tile == 0;  // a tile must get one step
      if (total > 0 || zero_step) {
        const unsigned lt = (1u << lane) - 1;
        if (hit) {
          const int pos = base + __popc(hits & lt);
          list_row[pos] = tid;
          list_idx[pos] = v0;
        } else {
          list_miss[32 * warp - base + __popc(~hits & lt)] = tid;
        }
        producer_sync();
        const int n_hit = total, n_miss = kRows - total;
        for (int slice = 0; slice < n_slices && ok; ++slice) {
          unsigned char *stage = open_stage(k_a, slice, 0, false);
          if (!stage) break;
          unsigned char *g = stage + w_region;
          const float *col = P.in + slice * kSlice + (tid & 7) * 4;
          const int c = tid & 7;
          for (int e = tid >> 3; e < n_hit; e += N_PRODUCER_WARPS * 4) {
            const int r = list_row[e];
            cp_async16(smem_u32(g) + (unsigned)r * 128 + ((unsigned)(c ^ (r & 7)) << 4),
                       col + (long long)list_idx[e] * P.ld_in, 16u);
          }
          if (kMasked) {
            if (lane == 0) {
              hit_mask[st * N_PRODUCER_WARPS + warp] = hits;
              __threadfence_block();  // ordered before this thread's arrival on the stage barrier
            }
          } else {
            for (int e = tid >> 3; e < n_miss; e += N_PRODUCER_WARPS * 4) {
              const int r = list_miss[e];
              *reinterpret_cast<uint4 *>(g + (unsigned)r * 128 + ((unsigned)(c ^ (r & 7)) << 4)) = make_uint4(0, 0, 0, 0);
            }
          }
          close_stage();
        }
        ++issued_in_tile;
      }
      if (tile_end && ok) {
        // end-of-tile marker: a slot without copies that tells the MMA thread to hand the
        // accumulator to the epilogue
        if (open_stage(0, 0, META_LAST_OF_TILE | (t == my_tiles - 1 ? META_LAST_OF_CTA : 0), true)) close_stage();
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
    cp_async_wait<0>();
  } else if (TMA_GATHER && warp == WARP_PRODUCER) {
    // =========================== rulebook read + TMA gather + weight slab ======================
    int st = 0, round = 0;
    bool ok = true;
    // Issues the n_slices steps of offset k whose row indices are in idx[8]: rows 4*lane..+3 and
    // 128 + 4*lane..+3 of the tile.
    auto issue = [&](const int *idx, int k, int last_flags) {
      for (int slice = 0; slice < n_slices && ok; ++slice) {
        if (round > 0) {
          int freed = 1;
          if (lane == 0) freed = mbar_wait(&empty[st], (unsigned)((round - 1) & 1)) ? 1 : 0;
          freed = __shfl_sync(0xffffffffu, freed, 0);
          if (!freed) {
            ok = false;
            break;
          }
        }
        unsigned char *stage = smem + (size_t)st * stage_bytes;
        if (lane == 0) {
          meta[st] = (slice == n_slices - 1) ? last_flags : 0;
          mbar_expect_tx(&full[st], (unsigned)kGBytes + total_w);
          bulk_copy_g2s(smem_u32(stage), P.wprep + ((size_t)k * n_slices + slice) * total_w, total_w, &full[st]);
        }
        __syncwarp();
        const unsigned g = smem_u32(stage) + w_region + lane * 512;
        tma_gather4(g, &in_map, slice * kSlice, idx[0], idx[1], idx[2], idx[3], &full[st]);
        tma_gather4(g + kGBytes / 2, &in_map, slice * kSlice, idx[4], idx[5], idx[6], idx[7], &full[st]);
        if (++st == NS) {
          st = 0;
          ++round;
        }
      }
    };
    auto load_idx = [&](long long row0, int k, int *v) {
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          long long r = row0 + h * 128 + 4 * lane + i;
          // rows at or beyond n_in are out of bounds for the tensor map and arrive as zeros
          v[h * 4 + i] = (k < P.K && r < P.n_out) ? __ldg(P.nbr + (long long)k * P.n_out + r) : -1;
        }
    };
    for (long long t = 0; t < my_tiles && ok && !*sh_abort; ++t) {
      const long long row0 = (blockIdx.x + t * gridDim.x) * kRows;
      const int tile_flags = META_LAST_OF_TILE | (t == my_tiles - 1 ? META_LAST_OF_CTA : 0);
      int cur[8], nx1[8], nx2[8], pend[8];
      int pend_k = -1;
      load_idx(row0, 0, cur);
      load_idx(row0, 1, nx1);
      for (int k = 0; k < P.K && ok; ++k) {
        load_idx(row0, k + 2, nx2);  // two offsets ahead: hides the rulebook read behind the steps
        bool any = false;
#pragma unroll
        for (int i = 0; i < 8; ++i) any |= (cur[i] >= 0);
        if (__any_sync(0xffffffffu, any)) {
          // the previous non-empty offset can go out now (it is not the tile's last)
          if (pend_k >= 0) issue(pend, pend_k, 0);
#pragma unroll
          for (int i = 0; i < 8; ++i) pend[i] = cur[i];
          pend_k = k;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          cur[i] = nx1[i];
          nx1[i] = nx2[i];
        }
      }
      if (pend_k < 0) {  // a tile without any rule still gets one (all-zero) step
#pragma unroll
        for (int i = 0; i < 8; ++i) pend[i] = -1;
        pend_k = 0;
      }
      if (ok) issue(pend, pend_k, tile_flags);
    }
    if (!ok) *sh_abort = 1;
  } else if (warp == WARP_MMA) {
    // ==================================== MMA issue (one thread) ===============================
    if (lane == 0) {
      const unsigned idesc = instr_desc_tma(kBf16);
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
          const unsigned ph = (unsigned)(round & 1);
          if (!mbar_wait(kTransform ? &full_t[st] : &full[st], ph)) {
            ok = false;
            break;
          }
          // rows written through the generic proxy (cp.async, plain stores, transform warps) were
          // acquired through the barrier; order them before the tensor core's async-proxy reads
          if (kTransform || !TMA_GATHER) fence_proxy_async_smem();
          tc_fence_after();
          const int flags = meta[st];
          if (!TMA_GATHER && (flags & META_LAST_OF_TILE)) {
            // marker slot of the cp.async producers: no data, just the end of the tile
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
          const unsigned aux_addr = g_addr + kGBytes;
          constexpr int n_mma = kBf16 ? 2 : 4;
#pragma unroll
          for (int jj = 0; jj < n_mma; ++jj) {
            // B operand: gathered rows.  tf32: the swizzled raw tile (32 bytes of K per MMA);
            // bf16: the converted tile in plain core-matrix layout (4 pieces of 16 bytes per row), in
            // the three-term form followed by the tile of what the rounding left over
            const unsigned long long dg = kBf16 ? smem_desc(aux_addr + jj * 256, 128, 512) : smem_desc_sw128(g_addr + jj * 32);
            const unsigned long long dg_lo =
                kB3 ? smem_desc(aux_addr + kGBytes / 2 + jj * 256, 128, 512) : smem_desc_sw128(aux_addr + jj * 32);
            const unsigned acc = (first && jj == 0) ? 0u : 1u;
            for (int mt = 0; mt < n_mt; ++mt) {
              const unsigned d = tmem_base + (unsigned)((ab * n_mt + mt) * kRows);
              // A operand: weight slab, plain core-matrix layout, 8 (fp32) / 4 (bf16) pieces per row
              const unsigned w_sbo = kBf16 ? 512u : 1024u;
              const unsigned w_mt = w_addr + (unsigned)mt * (kPlanes / 8) * w_sbo + jj * 256;
              const unsigned long long dw = smem_desc(w_mt, 128, w_sbo);
              tc_mma<kBf16>(d, dw, dg, idesc, acc);
              if (kSplit) {
                const unsigned long long dw_lo = smem_desc(w_mt + w_bytes, 128, w_sbo);
                tc_mma<kBf16>(d, dw, dg_lo, idesc, 1u);
                tc_mma<kBf16>(d, dw_lo, dg, idesc, 1u);
              }
            }
          }
          first = false;
          tc_commit(&empty[st]);
          if (flags & META_LAST_OF_TILE) tc_commit(&acc_full[ab]);
          if (++st == NS) {
            st = 0;
            ++round;
          }
          if (flags & META_LAST_OF_TILE) break;
        }
      }
      if (!ok) *sh_abort = 1;
    }
  } else if (warp >= WARP_TRANSFORM0 && warp < WARP_TRANSFORM0 + 4) {
    // =============================== transform warps (x3 / bf16) ==============================
    if (kTransform && my_tiles > 0) {
      const int t128 = tid - WARP_TRANSFORM0 * 32;
      int st = 0, round = 0;
      for (;;) {
        if (*sh_abort) break;
        int got = 1;
        if (lane == 0) got = mbar_wait(&full[st], (unsigned)(round & 1)) ? 1 : 0;
        got = __shfl_sync(0xffffffffu, got, 0);
        if (!got) {
          *sh_abort = 1;
          break;
        }
        unsigned char *g = smem + (size_t)st * stage_bytes + w_region;
        unsigned char *aux = g + kGBytes;
        const int flags = meta[st];
        const bool marker = !TMA_GATHER && (flags & META_LAST_OF_TILE);
        if (marker) {
          // end-of-tile marker slot: nothing to transform
        } else if (kSplit && !kB3) {
          // low part in the same (swizzled) position: g_lo = g - trunc_tf32(g)
#pragma unroll 4
          for (int i = 0; i < kGBytes / 16 / 128; ++i) {
            const int c = t128 + 128 * i;
            float4 a = *reinterpret_cast<const float4 *>(g + c * 16);
            float4 lo;
            lo.x = a.x - __uint_as_float(__float_as_uint(a.x) & 0xFFFFE000u);
            lo.y = a.y - __uint_as_float(__float_as_uint(a.y) & 0xFFFFE000u);
            lo.z = a.z - __uint_as_float(__float_as_uint(a.z) & 0xFFFFE000u);
            lo.w = a.w - __uint_as_float(__float_as_uint(a.w) & 0xFFFFE000u);
            *reinterpret_cast<float4 *>(aux + c * 16) = lo;
          }
        } else if (kB3) {
          // fp32 (swizzled rows of 128 bytes) -> two bf16 tiles in plain K-major core-matrix layout
          // (piece j = 8 planes of row r at (r/8)*512 + j*128 + (r%8)*16): the values rounded to bf16
          // and, 16 KB further on, what the rounding left over.  Rows without a rule become zeros.
          const unsigned *mask = reinterpret_cast<const unsigned *>(ctl + 512 + 3 * kRows * 4 + N_PRODUCER_WARPS * 4) +
                                 st * N_PRODUCER_WARPS;
#pragma unroll 4
          for (int i = 0; i < kRows * 4 / 128; ++i) {
            const int p = t128 + 128 * i;
            const int r = p >> 2, j = p & 3;
            uint4 hq = make_uint4(0, 0, 0, 0), mq = make_uint4(0, 0, 0, 0);
            if (!kMasked || ((mask[r >> 5] >> (r & 31)) & 1u)) {
              const unsigned char *row = g + r * 128;
              const float4 x = *reinterpret_cast<const float4 *>(row + (((2 * j) ^ (r & 7)) << 4));
              const float4 y = *reinterpret_cast<const float4 *>(row + (((2 * j + 1) ^ (r & 7)) << 4));
              split_bf16_pair(x.x, x.y, hq.x, mq.x);
              split_bf16_pair(x.z, x.w, hq.y, mq.y);
              split_bf16_pair(y.x, y.y, hq.z, mq.z);
              split_bf16_pair(y.z, y.w, hq.w, mq.w);
            }
            const unsigned off = (r >> 3) * 512 + j * 128 + (r & 7) * 16;
            *reinterpret_cast<uint4 *>(aux + off) = hq;
            *reinterpret_cast<uint4 *>(aux + kGBytes / 2 + off) = mq;
          }
        } else {
          // fp32 (swizzled rows of 128 bytes) -> bf16 tile in plain K-major core-matrix layout:
          // piece j (8 planes) of row r at (r/8)*512 + j*128 + (r%8)*16
#pragma unroll 4
          for (int i = 0; i < kRows * 4 / 128; ++i) {
            const int p = t128 + 128 * i;
            const int r = p >> 2, j = p & 3;
            const unsigned char *row = g + r * 128;
            float4 x = *reinterpret_cast<const float4 *>(row + (((2 * j) ^ (r & 7)) << 4));
            float4 y = *reinterpret_cast<const float4 *>(row + (((2 * j + 1) ^ (r & 7)) << 4));
            __nv_bfloat162 b0 = __floats2bfloat162_rn(x.x, x.y), b1 = __floats2bfloat162_rn(x.z, x.w);
            __nv_bfloat162 b2 = __floats2bfloat162_rn(y.x, y.y), b3 = __floats2bfloat162_rn(y.z, y.w);
            uint4 packed;
            packed.x = *reinterpret_cast<unsigned *>(&b0);
            packed.y = *reinterpret_cast<unsigned *>(&b1);
            packed.z = *reinterpret_cast<unsigned *>(&b2);
            packed.w = *reinterpret_cast<unsigned *>(&b3);
            *reinterpret_cast<uint4 *>(aux + (r >> 3) * 512 + j * 128 + (r & 7) * 16) = packed;
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&full_t[st]);
        if (++st == NS) {
          st = 0;
          ++round;
        }
        if (flags & META_LAST_OF_CTA) break;
      }
    }
  } else if (warp >= WARP_EPILOGUE0 && warp < WARP_EPILOGUE0 + 4) {
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
      const long long row0 = (blockIdx.x + t * gridDim.x) * kRows;
      for (int mt = 0; mt < n_mt; ++mt) {
        const int plane0 = mt * kPlanes + quad * 32;
        if (plane0 >= P.cout) break;
        const int plane = plane0 + lane;
        const bool plane_ok = plane < P.cout;
        const float b = (P.bias && plane_ok) ? P.bias[plane] : 0.f;
        for (int n0 = 0; n0 < kRows; n0 += 32) {
          if (row0 + n0 >= P.n_out) break;
          float v[32];
          tmem_ld32(tmem_base + ((unsigned)(quad * 32) << 16) + (unsigned)((ab * n_mt + mt) * kRows + n0), v);
          if (plane_ok) {
            float *dst = P.out + (row0 + n0) * P.ld_out + plane;
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (row0 + n0 + i < P.n_out) dst[(long long)i * P.ld_out] = v[i] + b;
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
  if (warp == WARP_MMA) tmem_dealloc(tmem_base, 512u);
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
static int tma_mode_of(int precision) {
  switch (precision) {
    case SCN_PRECISION_TF32: return TC_TF32;
    case SCN_PRECISION_BF16: return TC_BF16;
    case SCN_PRECISION_TF32X3: return split_mode_of_env();
    default: return -1;
  }
}

static size_t tma_stage_bytes(int mode, int cout) {
  const bool two_parts = mode == TC_TF32X3 || mode == TC_BF16X3;
  const bool bf16 = mode == TC_BF16 || mode == TC_BF16X3;
  size_t aux = two_parts ? kGBytes : (bf16 ? kGBytes / 2 : 0);
  size_t w = (size_t)cout * kSlice * (bf16 ? 2 : 4) * (two_parts ? 2 : 1);
  return ((w + 1023) & ~(size_t)1023) + kGBytes + aux;
}
constexpr size_t kTmaControlBytes = 4096;  // barriers, step flags, and the producers' row lists
constexpr size_t kTmaSmemBudget = 226 * 1024;

// SCN_TC_PERSISTENT=0 turns the persistent kernel off (the per-tile kernel of conv_tc.cu runs
// instead), SCN_TC_TMA_GATHER=1 selects the TMA gather4 producer instead of cp.async.
bool conv_tma_supported(int K, int cin, int cout, int groups, int precision, long long n_in) {
  int mode = tma_mode_of(precision);
  if (mode < 0 || groups != 1 || cin % kSlice != 0 || cout % 8 != 0 || cout < 8 || cout > 256 || n_in < 1) return false;
  (void)K;
  // Measured per layer of the U-Net: the persistent kernel wins where the tensor pipe is the
  // limit (three-pass mode); the single-pass modes are limited by the gather and run as fast in
  // the simpler per-tile kernel.  SCN_TC_PERSISTENT=1 / 0 forces it on / off for every mode.
  const char *e = getenv("SCN_TC_PERSISTENT");
  if (e && atoi(e) == 0) return false;
  if (!(e && atoi(e) != 0) && mode != TC_TF32X3 && mode != TC_BF16X3) return false;
  return (kTmaSmemBudget - kTmaControlBytes) / tma_stage_bytes(mode, cout) >= 2;
}

int conv_forward_tma(const float *in, long long n_in, float *out, long long n_out, const float *weight,
                     const float *bias, const int *table, int K, int cin, int cout, int precision, int *flags,
                     cudaStream_t stream) {
  if (n_out == 0) return SCN_OK;
  const int mode = tma_mode_of(precision);
  SCN_REQUIRE(mode >= 0, SCN_ERR_UNSUPPORTED, "tensor-core path: unsupported precision");
  SCN_REQUIRE((uintptr_t)in % 16 == 0, SCN_ERR_BAD_ARG, "tensor-core path needs a 16-byte aligned input matrix");
  SCN_REQUIRE(n_in < (1ll << 31) && n_out < (1ll << 31), SCN_ERR_UNSUPPORTED, "row count above 2^31");
  const size_t stage = tma_stage_bytes(mode, cout);
  const int stages = (int)std::min<size_t>(kMaxStages, (kTmaSmemBudget - kTmaControlBytes) / stage);
  SCN_REQUIRE(stages >= 2, SCN_ERR_UNSUPPORTED, "tensor-core path: stage does not fit shared memory");

  // tensor map of the input feature matrix [n_in rows][cin planes], box = 32 planes x 1 row
  // (gather4 fetches four such rows), 128-byte swizzle, zeros for rows outside the matrix
  CUtensorMap map;
  cuuint64_t gdim[2] = {(cuuint64_t)cin, (cuuint64_t)n_in};
  cuuint64_t gstride[1] = {(cuuint64_t)cin * sizeof(float)};
  cuuint32_t box[2] = {(cuuint32_t)kSlice, 1};
  cuuint32_t estr[2] = {1, 1};
  // The encoder is a driver entry point; it is looked up through the runtime so that the library
  // does not link against libcuda (and still loads on a machine without a driver).
  typedef CUresult (*EncodeTiled)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeTiled encode = nullptr;
  if (!encode) {
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    SCN_CUDA_CHECK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
    SCN_REQUIRE(fn && qres == cudaDriverEntryPointSuccess, SCN_ERR_CUDA, "cuTensorMapEncodeTiled is not available");
    encode = (EncodeTiled)fn;
  }
  CUresult cr = encode(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(in), gdim, gstride, box, estr,
                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  SCN_REQUIRE(cr == CUDA_SUCCESS, SCN_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)cr);

  const int esize = (mode == TC_BF16 || mode == TC_BF16X3) ? 2 : 4;
  const int parts = (mode == TC_TF32X3 || mode == TC_BF16X3) ? 2 : 1;
  WeightImage wi;
  bool build = true;
  SCN_TRY(weight_image_get(WIMG_TC, K, cin, cout, kSlice * 16 + mode, (size_t)K * cin * cout * esize * parts, stream, &wi,
                           &build));
  unsigned char *wprep = (unsigned char *)wi.ptr;
  if (build) SCN_TRY(prepare_weights(weight, wprep, K, cin, cout, kSlice, mode, stream));

  TmaParams P;
  P.in = in;
  P.ld_in = cin;
  P.n_in = n_in;
  P.out = out;
  P.n_out = n_out;
  P.ld_out = cout;
  P.wprep = wprep;
  P.bias = bias;
  P.nbr = table;
  P.K = K;
  P.cin = cin;
  P.cout = cout;
  P.n_stages = stages;
  P.n_tiles = ceil_div(n_out, kRows);
  P.flags = flags;
  static int n_sm[64] = {0};
  int dev = 0;
  SCN_CUDA_CHECK(cudaGetDevice(&dev));
  SCN_REQUIRE(dev >= 0 && dev < 64, SCN_ERR_UNSUPPORTED, "device index %d unsupported", dev);
  if (!n_sm[dev]) {
    int sms = 0;
    SCN_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const int b = (int)kTmaSmemBudget;
    SCN_CUDA_CHECK(cudaFuncSetAttribute(k_conv_tma<TC_TF32, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, b));
    SCN_CUDA_CHECK(cudaFuncSetAttribute(k_conv_tma<TC_BF16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, b));
    SCN_CUDA_CHECK(cudaFuncSetAttribute(k_conv_tma<TC_TF32X3, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, b));
    SCN_CUDA_CHECK(cudaFuncSetAttribute(k_conv_tma<TC_TF32, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, b));
    SCN_CUDA_CHECK(cudaFuncSetAttribute(k_conv_tma<TC_BF16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, b));
    SCN_CUDA_CHECK(cudaFuncSetAttribute(k_conv_tma<TC_TF32X3, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, b));
    SCN_CUDA_CHECK(cudaFuncSetAttribute(k_conv_tma<TC_BF16X3, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, b));
    SCN_CUDA_CHECK(cudaFuncSetAttribute(k_conv_tma<TC_BF16X3, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, b));
    n_sm[dev] = sms;  // only now: a failed attribute call is retried by the next call
  }
  const unsigned grid = (unsigned)std::min<long long>(P.n_tiles, n_sm[dev]);
  // Ask for the whole budget: one CTA per SM by construction (it also owns all 512 TMEM columns)
  const size_t smem = kTmaSmemBudget;
  const char *e = getenv("SCN_TC_TMA_GATHER");
  const bool tma_gather = e && atoi(e) != 0;
  if (tma_gather) {
    if (mode == TC_TF32)
      SCN_LAUNCH((k_conv_tma<TC_TF32, true>), grid, N_WARPS * 32, smem, stream, map, P);
    else if (mode == TC_BF16)
      SCN_LAUNCH((k_conv_tma<TC_BF16, true>), grid, N_WARPS * 32, smem, stream, map, P);
    else if (mode == TC_BF16X3)
      SCN_LAUNCH((k_conv_tma<TC_BF16X3, true>), grid, N_WARPS * 32, smem, stream, map, P);
    else
      SCN_LAUNCH((k_conv_tma<TC_TF32X3, true>), grid, N_WARPS * 32, smem, stream, map, P);
  } else {
    if (mode == TC_TF32)
      SCN_LAUNCH((k_conv_tma<TC_TF32, false>), grid, N_WARPS * 32, smem, stream, map, P);
    else if (mode == TC_BF16)
      SCN_LAUNCH((k_conv_tma<TC_BF16, false>), grid, N_WARPS * 32, smem, stream, map, P);
    else if (mode == TC_BF16X3)
      SCN_LAUNCH((k_conv_tma<TC_BF16X3, false>), grid, N_WARPS * 32, smem, stream, map, P);
    else
      SCN_LAUNCH((k_conv_tma<TC_TF32X3, false>), grid, N_WARPS * 32, smem, stream, map, P);
  }
  SCN_CUDA_CHECK(cudaGetLastError());
  SCN_TRY(weight_image_put(wi, stream));
  return SCN_OK;
}

}  // namespace scn
