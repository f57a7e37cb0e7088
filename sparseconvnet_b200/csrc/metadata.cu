// The Metadata object: GPU site hash per spatial scale and the rulebook builders.
//
// Replaces, with device kernels and no host round trip for the rules themselves,
//   Metadata<D>::inputLayer / inputLayerRules     (Metadata.cpp:413-425, IOLayersRules.h:18-121)
//   Metadata<D>::getSubmanifoldRuleBook           (Metadata.cpp:437-451,
//                                                  SubmanifoldConvolutionRules.h:11-87)
//   Metadata<D>::getRuleBook                      (Metadata.cpp:492-518, ConvolutionRules.h:11-105,
//                                                  RectangularRegions.h:94-119)
//   Metadata<D>::getSpatialLocations              (Metadata.cpp:149-170)
// of the reference.  Only counts (active sites, rules per offset) ever travel to the host.
#include <stdlib.h>

#include <algorithm>
#include <climits>

#include <atomic>
#include <mutex>

#include "metadata.cuh"

namespace scn {

static std::atomic<long long> g_rulebook_builds{0};  // rulebooks constructed (not served from a cache)

// ------------------------------------------------------------------------------------------
// key layout
// ------------------------------------------------------------------------------------------

static int make_layout(int dim, const int64_t *size, KeyLayout &L) {
  L = KeyLayout{};
  L.dim = dim;
  int sh = 0;
  for (int d = dim - 1; d >= 0; --d) {  // last dimension in the lowest bits
    SCN_REQUIRE(size[d] >= 1 && size[d] <= INT_MAX, SCN_ERR_BAD_ARG,
                "spatial size[%d]=%lld out of range", d, (long long)size[d]);
    int bits = std::max(1, bit_length((unsigned long long)size[d] - 1));
    L.shift[d] = sh;
    L.bits[d] = bits;
    L.size[d] = (int)size[d];
    sh += bits;
  }
  SCN_REQUIRE(sh <= 62, SCN_ERR_KEY_BITS, "spatial size needs %d key bits (max 62)", sh);
  L.batch_shift = sh;
  L.batch_bits = std::min(31, 63 - sh);
  return SCN_OK;
}

std::vector<int64_t> make_key(int dim, const int64_t *a, const int64_t *b, const int64_t *c) {
  std::vector<int64_t> k(a, a + dim);
  if (b) k.insert(k.end(), b, b + dim);
  if (c) k.insert(k.end(), c, c + dim);
  return k;
}

int md_touch(scn_metadata *md, cudaStream_t stream) {
  int dev = 0;
  SCN_CUDA_CHECK(cudaGetDevice(&dev));
  if (md->device < 0) md->device = dev;
  SCN_REQUIRE(md->device == dev, SCN_ERR_BAD_ARG, "metadata object lives on device %d, current device is %d",
              md->device, dev);
  md->last_stream = stream;
  return SCN_OK;
}

static int chain_finalize(scn_metadata *md, cudaStream_t stream, int *n_built);
static void chain_abandon(scn_metadata *md, cudaStream_t stream);

Grid *find_grid(scn_metadata *md, const int64_t *spatial_size) {
  auto it = md->grids.find(make_key(md->dim, spatial_size));
  if (it == md->grids.end() && md->pending) {
    // the grid may be one of a chain that was started on the side stream: take the chain over, then look again
    if (chain_finalize(md, md->last_stream, nullptr) != SCN_OK) return nullptr;
    it = md->grids.find(make_key(md->dim, spatial_size));
  }
  return it == md->grids.end() ? nullptr : &it->second;
}

static int alloc_table(HashTable &T, long long expected_sites, cudaStream_t stream) {
  unsigned long long slots = next_pow2((unsigned long long)std::max<long long>(64, 2 * expected_sites));
  SCN_REQUIRE(slots < (1ull << 31), SCN_ERR_UNSUPPORTED, "site table too large (%llu slots)", slots);
  T.n_buckets = slots / 2;
  SCN_TRY(device_alloc((void **)&T.slots, slots * sizeof(Slot), stream));
  // key = all ones (free), row = -1, aux = 0xFFFFFFFF
  SCN_CUDA_CHECK(cudaMemsetAsync(T.slots, 0xFF, slots * sizeof(Slot), stream));
  return SCN_OK;
}

static void free_grid(Grid &g, cudaStream_t stream) {
  device_free(g.row_keys, stream);
  device_free(g.table.slots, stream);
  g = Grid{};
}
static void free_rulebook(Rulebook &r, cudaStream_t stream) {
  count_ticket_release(r.ticket);
  device_free(r.nbr, stream);
  device_free(r.tnbr, stream);
  device_free(r.counts_dev, stream);
  r = Rulebook{};
}

static int ensure_scratch(scn_metadata *md, cudaStream_t stream) {
  if (!md->flags_dev) {
    SCN_TRY(device_alloc((void **)&md->flags_dev, sizeof(int), stream));
    SCN_CUDA_CHECK(cudaMemsetAsync(md->flags_dev, 0, sizeof(int), stream));
  }
  if (!md->scalars_dev) SCN_TRY(device_alloc((void **)&md->scalars_dev, 4 * sizeof(int), stream));
  return SCN_OK;
}

// ---- host mailboxes -------------------------------------------------------------------------------
// The few integers the host has to wait for (flag word, site counts) are written by a one-thread
// kernel into pinned host memory that is mapped into the device's address space, not copied by
// cudaMemcpy: a device-to-host copy queues on the copy engine behind whatever the application is
// copying at the time (a previous batch's 127 MB of results held every such read-back up for 2 ms,
// once per strided level of a U-Net forward).  Slots of 256 bytes from slabs that are never given back.
constexpr int kMailboxBytes = 256;  // 64 integers: flag word + the counts of a whole chain of levels
namespace {
struct MailboxPool {
  std::mutex mu;
  std::vector<int *> free_slots;
};
MailboxPool &mailbox_pool() {
  static MailboxPool *p = new MailboxPool();
  return *p;
}
}  // namespace

static int mailbox_acquire(int **slot) {
  MailboxPool &P = mailbox_pool();
  std::lock_guard<std::mutex> lock(P.mu);
  if (P.free_slots.empty()) {
    int *slab = nullptr;
    SCN_CUDA_CHECK(cudaHostAlloc((void **)&slab, 4096, cudaHostAllocMapped | cudaHostAllocPortable));
    for (int i = 0; i < 4096 / kMailboxBytes; ++i) P.free_slots.push_back(slab + i * (kMailboxBytes / 4));
  }
  *slot = P.free_slots.back();
  P.free_slots.pop_back();
  return SCN_OK;
}

static void mailbox_release(int *slot) {
  if (!slot) return;
  MailboxPool &P = mailbox_pool();
  std::lock_guard<std::mutex> lock(P.mu);
  P.free_slots.push_back(slot);
}

__global__ void k_post_scalars(int *flags_dev, const int *scalars_dev, volatile int *mailbox) {
  mailbox[0] = *flags_dev;
  *flags_dev = 0;
  if (scalars_dev)
    for (int i = 0; i < 4; ++i) mailbox[1 + i] = scalars_dev[i];
  __threadfence_system();
}

// Reads (and clears) the device flag word; waits for the stream.
static int fetch_flags(scn_metadata *md, cudaStream_t stream, int *flags, int *scalars4) {
  if (!md->mailbox) SCN_TRY(mailbox_acquire(&md->mailbox));
  int *mailbox_dev = nullptr;
  SCN_CUDA_CHECK(cudaHostGetDevicePointer((void **)&mailbox_dev, md->mailbox, 0));
  SCN_LAUNCH(k_post_scalars, 1, 1, 0, stream, md->flags_dev, scalars4 ? md->scalars_dev : nullptr, mailbox_dev);
  SCN_CUDA_CHECK(cudaGetLastError());
  note_host_wait();
  SCN_CUDA_CHECK(cudaStreamSynchronize(stream));
  const volatile int *host = md->mailbox;
  *flags = host[0];
  if (scalars4)
    for (int i = 0; i < 4; ++i) scalars4[i] = host[1 + i];
  return SCN_OK;
}

static int flags_to_status(int flags) {
  if (flags & FLAG_COORD_RANGE) {
    set_error("a coordinate or batch index lies outside the spatial size");
    return SCN_ERR_COORD_RANGE;
  }
  if (flags & FLAG_TABLE_FULL) {
    set_error("site hash probe limit reached");
    return SCN_ERR_TABLE_FULL;
  }
  if (flags & FLAG_TC_TIMEOUT) {
    set_error("a bounded wait inside the tensor-core convolution kernel expired");
    return SCN_ERR_CUDA;
  }
  if (flags & FLAG_BAD_ROW) {
    set_error("a rulebook entry points outside the feature matrix");
    return SCN_ERR_SIZE_MISMATCH;
  }
  return SCN_OK;
}

// ------------------------------------------------------------------------------------------
// input layer
// ------------------------------------------------------------------------------------------

// One thread per input row: range-check, pack, insert.  mode 0 keeps the largest row index
// per site (the reference's serial `mp[p] = i` leaves the last writer, IOLayersRules.h:41,55);
// the other modes record the first row that touched the site.
// bl_length > 0: coords are [batch, bl_length, dim] (BLInputLayer, IOLayersRules.h:134-288):
// the sample index is i / bl_length and a point whose first coordinate is negative is empty.
__global__ void k_insert_input(KeyLayout L, HashTable T, const long long *__restrict__ coords,
                               long long n, int ncols, int mode, long long bl_length,
                               unsigned long long *__restrict__ row_keys, int *__restrict__ slot_of,
                               int *flags, int *scalars) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const long long *c = coords + i * ncols;
  if (bl_length > 0 && c[0] < 0) {  // empty slot of the batch x length array: in no map, in no rule
    if (mode == 0) row_keys[i] = kEmptyKey;
    slot_of[i] = -1;
    return;
  }
  int x[kMaxDim];
  bool ok = true;
  for (int d = 0; d < L.dim; ++d) {
    long long v = c[d];
    ok &= (v >= 0 && v < L.size[d]);
    x[d] = (int)v;
  }
  long long bl = bl_length > 0 ? i / bl_length : ((ncols > L.dim) ? c[L.dim] : 0);
  ok &= (bl >= 0 && bl < (1ll << L.batch_bits));
  if (!ok) {
    atomicOr(flags, FLAG_COORD_RANGE);
    if (mode == 0) row_keys[i] = kEmptyKey;
    slot_of[i] = -1;
    return;
  }
  unsigned long long key = pack_key(L, x, (int)bl);
  long long s = hash_insert(T, key);
  if (s < 0) {
    atomicOr(flags, FLAG_TABLE_FULL);
    if (mode == 0) row_keys[i] = kEmptyKey;
    slot_of[i] = -1;
    return;
  }
  // largest batch index: one atomic per warp, and none once the word already holds the value
  {
    const unsigned peers = __activemask();
    const int warp_max = __reduce_max_sync(peers, (int)bl);
    if ((threadIdx.x & 31) == __ffs(peers) - 1 && warp_max > *(volatile int *)&scalars[1])
      atomicMax(&scalars[1], warp_max);
  }
  slot_of[i] = (int)s;
  if (mode == 0) {
    row_keys[i] = key;
    atomicMax(&T.slots[s].row, (int)i);
  } else {
    atomicMin(&T.slots[s].aux, (unsigned)i);
  }
}

// Input mode 0 with repeated coordinates: the site belongs to the last row that named it.
// Earlier rows keep their feature row but are in no map of the reference, so no rule ever
// touches them and getSpatialLocations leaves them zero; here their key is blanked.
__global__ void k_blank_overwritten(const Slot *__restrict__ slots, const int *__restrict__ slot_of,
                                    long long n, unsigned long long *__restrict__ row_keys) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  int s = slot_of[i];
  if (s >= 0 && slots[s].row != (int)i) row_keys[i] = kEmptyKey;
}

__global__ void k_flag_first(const Slot *__restrict__ slots, const int *__restrict__ slot_of,
                             long long n, int *__restrict__ flag) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  int s = slot_of[i];
  flag[i] = (s >= 0 && slots[s].aux == (unsigned)i) ? 1 : 0;
}

// The row that touched a site first gives the site its row number: its rank among such rows in input
// order, which is the numbering of the reference (one counter over the whole input,
// IOLayersRules.h:69-72,84-87; one per output grid, ConvolutionRules.h:24-30).  One thread per table
// SLOT, not per candidate: the table is read and written front to back, and what is reached at random
// (the rank of the slot's first toucher, the row -> key array) is a few MB that stay in L2.  The
// candidate-order form of this pass (a random read-modify-write of a slot per numbered site) was bound by
// the DRAM's random-access rate: 198 us against 142 us for the inserts themselves at 1.6 M sites.
// `capacity`: rows the output arrays were sized for; a site numbered beyond it (a chain level that
// shrank less than guessed) is not written and raises FLAG_TABLE_FULL in `level_flags`.
__global__ void k_number_slots(Slot *slots, long long n_slots, const int *__restrict__ rank,
                               long long capacity, int *level_flags,
                               unsigned long long *__restrict__ row_keys) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n_slots) return;
  const uint4 v = *reinterpret_cast<const uint4 *>(slots + idx);
  const unsigned long long key = ((unsigned long long)v.y << 32) | v.x;
  if (key == kEmptyKey || v.w == 0xFFFFFFFFu) return;
  const int r = rank[v.w];
  if (r >= capacity) {
    atomicOr(level_flags, FLAG_TABLE_FULL);
    return;
  }
  slots[idx].row = r;
  row_keys[r] = key;
}

__global__ void k_count_per_site(const Slot *__restrict__ slots, const int *__restrict__ slot_of,
                                 long long n, int *cnt) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  int s = slot_of[i];
  if (s >= 0) atomicAdd(&cnt[slots[s].row], 1);
}

__global__ void k_fill_per_site(const Slot *__restrict__ slots, const int *__restrict__ slot_of,
                                long long n, const int *__restrict__ start, int *cursor,
                                int *__restrict__ csr_rows) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  int s = slot_of[i];
  if (s < 0) return;
  int r = slots[s].row;
  int p = atomicAdd(&cursor[r], 1);
  csr_rows[start[r] + p] = (int)i;
}

// Puts the input rows of every site in ascending order (heap sort, in place, one thread per
// site; sites with duplicates hold a handful of rows).
__global__ void k_sort_segments(const int *__restrict__ start, long long n_sites, int *csr_rows) {
  long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= n_sites) return;
  int *a = csr_rows + start[r];
  int m = start[r + 1] - start[r];
  if (m < 2) return;
  if (m <= 16) {
    for (int i = 1; i < m; ++i) {
      int v = a[i], j = i - 1;
      while (j >= 0 && a[j] > v) {
        a[j + 1] = a[j];
        --j;
      }
      a[j + 1] = v;
    }
    return;
  }
  for (int root0 = m / 2 - 1; root0 >= 0; --root0) {
    int root = root0;
    for (;;) {
      int child = 2 * root + 1;
      if (child >= m) break;
      if (child + 1 < m && a[child] < a[child + 1]) ++child;
      if (a[root] >= a[child]) break;
      int t = a[root]; a[root] = a[child]; a[child] = t;
      root = child;
    }
  }
  for (int end = m - 1; end > 0; --end) {
    int t = a[0]; a[0] = a[end]; a[end] = t;
    int root = 0;
    for (;;) {
      int child = 2 * root + 1;
      if (child >= end) break;
      if (child + 1 < end && a[child] < a[child + 1]) ++child;
      if (a[root] >= a[child]) break;
      int u = a[root]; a[root] = a[child]; a[child] = u;
      root = child;
    }
  }
}

__global__ void k_init_scalars(int *scalars) {
  scalars[0] = 0;
  scalars[1] = -1;
  scalars[2] = 0;
  scalars[3] = 0;
}

static void clear_input_rules(scn_metadata *md, cudaStream_t stream) {
  device_free(md->input_csr_start, stream);
  device_free(md->input_csr_rows, stream);
  md->input_csr_start = md->input_csr_rows = nullptr;
  md->input_mode = -1;
  md->input_n_rows = md->input_n_active = 0;
}

static int md_clear(scn_metadata *md, cudaStream_t stream) {
  chain_abandon(md, stream);
  for (auto &g : md->grids) free_grid(g.second, stream);
  for (auto &r : md->sub_rules) free_rulebook(r.second, stream);
  for (auto &r : md->strided_rules) free_rulebook(r.second, stream);
  md->grids.clear();
  md->sub_rules.clear();
  md->strided_rules.clear();
  clear_input_rules(md, stream);
  return SCN_OK;
}

static int md_input_layer(scn_metadata *md, const int64_t *spatial_size, const int64_t *coords,
                          int coords_on_device, int64_t n, int ncols, int64_t batch_size, int mode,
                          int64_t bl_length, cudaStream_t stream, int64_t *n_active) {
  SCN_REQUIRE(md && spatial_size && n_active, SCN_ERR_BAD_ARG, "null argument");
  SCN_REQUIRE(mode >= 0 && mode <= 4, SCN_ERR_BAD_ARG, "input layer mode %d not in 0..4", mode);
  SCN_REQUIRE(ncols == md->dim || ncols == md->dim + 1, SCN_ERR_BAD_ARG,
              "coords must have %d or %d columns, got %d", md->dim, md->dim + 1, ncols);
  SCN_REQUIRE(n >= 0 && n < (1ll << 30), SCN_ERR_UNSUPPORTED, "row count %lld unsupported", (long long)n);
  SCN_REQUIRE(n == 0 || coords, SCN_ERR_BAD_ARG, "null coords");
  SCN_TRY(md_touch(md, stream));
  SCN_TRY(ensure_scratch(md, stream));

  // A new input replaces everything the object knew: grids of other scales and rulebooks built from
  // the old input would otherwise stay cached with the old row counts.  (The reference asserts that
  // the object is empty, IOLayersRules.h:22-24.)
  SCN_TRY(md_clear(md, stream));
  auto key = make_key(md->dim, spatial_size);

  Grid g;
  SCN_TRY(make_layout(md->dim, spatial_size, g.layout));
  SCN_TRY(alloc_table(g.table, n, stream));
  SCN_TRY(device_alloc((void **)&g.row_keys, sizeof(unsigned long long) * (size_t)std::max<int64_t>(n, 1), stream));

  const long long *coords_dev = (const long long *)coords;
  long long *staged = nullptr;
  if (!coords_on_device && n > 0) {
    size_t bytes = sizeof(long long) * (size_t)n * ncols;
    SCN_TRY(device_alloc((void **)&staged, bytes, stream));
    SCN_CUDA_CHECK(cudaMemcpyAsync(staged, coords, bytes, cudaMemcpyHostToDevice, stream));
    coords_dev = staged;
  }

  const int threads = 256;
  unsigned blocks = (unsigned)ceil_div(std::max<int64_t>(n, 1), threads);
  SCN_LAUNCH(k_init_scalars, 1, 1, 0, stream, md->scalars_dev);
  int *slot_of = nullptr, *flag = nullptr, *rank = nullptr, *cursor = nullptr;
  SCN_TRY(device_alloc((void **)&slot_of, sizeof(int) * (size_t)std::max<int64_t>(n, 1), stream));
  if (n > 0) {
    SCN_LAUNCH(k_insert_input, blocks, threads, 0, stream, g.layout, g.table, coords_dev, n, ncols, mode, (long long)bl_length, g.row_keys, slot_of, md->flags_dev, md->scalars_dev);
    if (mode == 0)
      SCN_LAUNCH(k_blank_overwritten, blocks, threads, 0, stream, g.table.slots, slot_of, n, g.row_keys);
    SCN_CUDA_CHECK(cudaGetLastError());
  }
  if (mode != 0 && n > 0) {
    SCN_TRY(device_alloc((void **)&flag, sizeof(int) * (size_t)n, stream));
    SCN_TRY(device_alloc((void **)&rank, sizeof(int) * (size_t)n, stream));
    SCN_LAUNCH(k_flag_first, blocks, threads, 0, stream, g.table.slots, slot_of, n, flag);
    SCN_TRY(exclusive_scan_i32(flag, rank, n, &md->scalars_dev[0], stream));
    const long long n_slots = 2 * (long long)g.table.n_buckets;
    SCN_LAUNCH(k_number_slots, (unsigned)ceil_div(n_slots, threads), threads, 0, stream, g.table.slots, n_slots, rank, (long long)n, md->flags_dev, g.row_keys);
    SCN_CUDA_CHECK(cudaGetLastError());
  }

  // stream-ordered: what only the kernels above read goes back before the host waits
  device_free(staged, stream);
  device_free(flag, stream);
  device_free(rank, stream);
  staged = nullptr;
  flag = rank = nullptr;
  int flags = 0, sc[4];
  SCN_TRY(fetch_flags(md, stream, &flags, sc));
  long long active = (mode == 0) ? n : (n > 0 ? sc[0] : 0);
  // Every point has a site of its own (no repeated coordinates, no empty slots): rows are numbered in
  // order of first occurrence, so row i is point i and the rule table is the identity -- the feature
  // pass is then the plain copy of mode 0 and no table is built.  Otherwise: CSR of the input rows of
  // every site, each site's rows ascending (the order the reference sums them in).
  const bool identity = mode != 0 && flags == 0 && active == n;
  if (mode != 0 && n > 0 && flags == 0 && active > 0 && !identity) {
    SCN_TRY(device_alloc((void **)&md->input_csr_start, sizeof(int) * (size_t)(n + 1), stream));
    SCN_TRY(device_alloc((void **)&md->input_csr_rows, sizeof(int) * (size_t)n, stream));
    SCN_TRY(device_alloc((void **)&cursor, sizeof(int) * (size_t)(n + 1), stream));
    SCN_CUDA_CHECK(cudaMemsetAsync(cursor, 0, sizeof(int) * (size_t)(n + 1), stream));
    SCN_LAUNCH(k_count_per_site, blocks, threads, 0, stream, g.table.slots, slot_of, n, cursor);
    SCN_TRY(exclusive_scan_i32(cursor, md->input_csr_start, n + 1, nullptr, stream));
    SCN_CUDA_CHECK(cudaMemsetAsync(cursor, 0, sizeof(int) * (size_t)(n + 1), stream));
    SCN_LAUNCH(k_fill_per_site, blocks, threads, 0, stream, g.table.slots, slot_of, n, md->input_csr_start, cursor, md->input_csr_rows);
    unsigned sblocks = (unsigned)ceil_div(active, threads);
    SCN_LAUNCH(k_sort_segments, sblocks, threads, 0, stream, md->input_csr_start, active, md->input_csr_rows);
    SCN_CUDA_CHECK(cudaGetLastError());
  }
  device_free(slot_of, stream);
  device_free(cursor, stream);
  int st = flags_to_status(flags);
  if (st != SCN_OK) {
    free_grid(g, stream);
    clear_input_rules(md, stream);
    return st;
  }
  g.n_active = active;
  g.may_have_blank_rows = (mode == 0);
  // batch size: IOLayersRules.h:25,35,52-53 -- one sample when there is no batch column,
  // otherwise max(requested, largest index + 1)
  if (bl_length > 0)
    g.batch_size = batch_size;
  else if (ncols == md->dim)
    g.batch_size = 1;
  else
    g.batch_size = std::max<long long>(batch_size, (long long)sc[1] + 1);
  md->input_mode = identity ? 0 : mode;  // what the feature passes do (a copy when the table is the identity)
  md->input_n_rows = n;
  md->input_n_active = active;
  md->grids[key] = g;
  *n_active = active;
  return SCN_OK;
}

// ------------------------------------------------------------------------------------------
// spatial locations
// ------------------------------------------------------------------------------------------

// Row r -> (x_0..x_{D-1}, batch).  A row with a blank key (an earlier duplicate under input
// mode 0) is reported as zeros, as the reference leaves it (Metadata.cpp:154-168 writes only
// rows reachable from the maps).
__global__ void k_spatial_locations(KeyLayout L, const unsigned long long *__restrict__ row_keys,
                                    long long n, long long *__restrict__ out) {
  long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= n) return;
  unsigned long long key = row_keys[r];
  long long *o = out + r * (L.dim + 1);
  bool live = (key != kEmptyKey);
  int x[kMaxDim], b = 0;
  if (live) unpack_key(L, key, x, b);
  for (int d = 0; d < L.dim; ++d) o[d] = live ? x[d] : 0;
  o[L.dim] = live ? b : 0;
}

// ------------------------------------------------------------------------------------------
// submanifold rulebook
// ------------------------------------------------------------------------------------------

struct FilterDesc {
  int f[kMaxDim];  // filter size
  int s[kMaxDim];  // stride (strided rules only)
  int out_size[kMaxDim];
  int tdim[kMaxDim];  // outputs an input can feed per dimension: ceil(f / s)
  int tmax;
};

// One thread per output site, looping over this block's range of filter offsets.  Offset k
// (row-major over the filter, last dimension fastest, RectangularRegions.h:30-38) looks at
// input = output + delta_k with delta = k_d - f_d / 2 (SubmanifoldConvolutionRules.h:15-19).
// The neighbour's key is the site's key plus a per-offset constant, so a probe is a bounds
// check, one 64-bit add and one 32-byte bucket read.
__global__ void __launch_bounds__(256)
k_submanifold_rules(KeyLayout L, HashTable T, const unsigned long long *__restrict__ row_keys,
                    long long n, int K, FilterDesc F, int k_chunk, int *__restrict__ nbr,
                    unsigned long long *counts, int mirrored) {
  extern __shared__ long long sh_raw[];
  long long *sh_keydelta = sh_raw;                         // [k_chunk]
  int *sh_count = (int *)(sh_keydelta + k_chunk);          // [k_chunk]
  signed char *sh_delta = (signed char *)(sh_count + k_chunk);  // [k_chunk][dim]
  // mirrored (all filter sizes odd): offset K-1-k is offset k seen from the neighbour, so only the
  // offsets up to the centre are looked up; a hit also fills the neighbour's entry at the mirrored
  // offset (pre-set to -1 by the caller), and the centre is the site itself.
  const int k_end = mirrored ? K / 2 + 1 : K;
  int k0 = blockIdx.y * k_chunk;
  int k1 = min(k_end, k0 + k_chunk);
  for (int kk = k0 + threadIdx.x; kk < k1; kk += blockDim.x) {
    int rem = kk;
    long long kd = 0;
    for (int d = L.dim - 1; d >= 0; --d) {
      int delta = rem % F.f[d] - F.f[d] / 2;
      rem /= F.f[d];
      sh_delta[(kk - k0) * L.dim + d] = (signed char)delta;
      kd += (long long)delta * (1ll << L.shift[d]);
    }
    sh_keydelta[kk - k0] = kd;
    sh_count[kk - k0] = 0;
  }
  __syncthreads();
  long long site = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  bool active = site < n;
  unsigned long long key = active ? row_keys[site] : kEmptyKey;
  active = active && (key != kEmptyKey);  // blank key: overwritten duplicate, in no map
  int x[kMaxDim], b = 0;
  if (active) unpack_key(L, key, x, b);
  for (int kk = k0; kk < k1; ++kk) {
    int row = -1;
    if (active) {
      bool ok = true;
      const signed char *dl = sh_delta + (kk - k0) * L.dim;
      for (int d = 0; d < L.dim; ++d) {
        int y = x[d] + dl[d];
        ok &= ((unsigned)y < (unsigned)L.size[d]);
      }
      if (mirrored && kk == K / 2)
        row = (int)site;
      else if (ok)
        row = hash_find_row(T, key + (unsigned long long)sh_keydelta[kk - k0]);
    }
    if (site < n) nbr[(long long)kk * n + site] = row;
    if (mirrored && kk < K / 2 && row >= 0) nbr[(long long)(K - 1 - kk) * n + row] = (int)site;
    unsigned hits = __ballot_sync(0xffffffffu, row >= 0);
    if ((threadIdx.x & 31) == 0 && hits) atomicAdd(&sh_count[kk - k0], __popc(hits));
  }
  __syncthreads();
  for (int kk = k0 + threadIdx.x; kk < k1; kk += blockDim.x)
    if (sh_count[kk - k0]) {
      atomicAdd(&counts[kk], (unsigned long long)sh_count[kk - k0]);
      if (mirrored && kk < K / 2) atomicAdd(&counts[K - 1 - kk], (unsigned long long)sh_count[kk - k0]);
    }
}

int get_submanifold_rulebook(scn_metadata *md, const int64_t *spatial_size,
                             const int64_t *filter_size, cudaStream_t stream, Rulebook **out) {
  SCN_TRY(md_touch(md, stream));
  auto key = make_key(md->dim, spatial_size, filter_size);
  Rulebook &rb = md->sub_rules[key];
  *out = &rb;
  if (rb.built) return SCN_OK;
  Grid *g = find_grid(md, spatial_size);
  if (!g) {
    md->sub_rules.erase(key);
    set_error("submanifold rulebook: no grid for that spatial size");
    return SCN_ERR_NO_GRID;
  }
  long long K = 1;
  FilterDesc F{};
  for (int d = 0; d < md->dim; ++d) {
    SCN_REQUIRE(filter_size[d] >= 1 && filter_size[d] <= 127, SCN_ERR_UNSUPPORTED,
                "filter size %lld unsupported", (long long)filter_size[d]);
    F.f[d] = (int)filter_size[d];
    K *= filter_size[d];
  }
  SCN_REQUIRE(K <= 4096, SCN_ERR_UNSUPPORTED, "filter volume %lld unsupported", K);
  long long n = g->n_active;
  SCN_REQUIRE(K * std::max<long long>(n, 1) < (1ll << 40), SCN_ERR_UNSUPPORTED, "rulebook too large");
  rb.n_offsets = (int)K;
  rb.n_in = rb.n_out = n;
  SCN_TRY(device_alloc((void **)&rb.nbr, sizeof(int) * (size_t)(K * std::max<long long>(n, 1)), stream));
  SCN_TRY(device_alloc((void **)&rb.counts_dev, sizeof(unsigned long long) * (size_t)K, stream));
  SCN_CUDA_CHECK(cudaMemsetAsync(rb.counts_dev, 0, sizeof(unsigned long long) * (size_t)K, stream));
  if (n > 0) {
    const int threads = 256;
    long long bx = ceil_div(n, threads);
    bool mirrored = K > 1 && !(getenv("SCN_RULES_MIRROR") && atoi(getenv("SCN_RULES_MIRROR")) == 0);
    for (int d = 0; d < md->dim; ++d) mirrored &= (filter_size[d] % 2 == 1);
    const long long k_end = mirrored ? K / 2 + 1 : K;  // offsets that are looked up
    if (mirrored)  // the mirrored half starts out empty
      SCN_CUDA_CHECK(cudaMemsetAsync(rb.nbr + k_end * n, 0xFF, sizeof(int) * (size_t)((K - k_end) * n), stream));
    // enough blocks to fill the machine even for few sites: split the offsets over grid.y
    long long want_y = std::max<long long>(1, std::min<long long>(k_end, ceil_div(148 * 16, bx)));
    int k_chunk = (int)ceil_div(k_end, want_y);
    int gy = (int)ceil_div(k_end, k_chunk);
    size_t smem = (size_t)k_chunk * (sizeof(long long) + sizeof(int) + md->dim);
    SCN_LAUNCH(k_submanifold_rules, dim3((unsigned)bx, (unsigned)gy), threads, smem, stream, g->layout, g->table, g->row_keys, n, (int)K, F, k_chunk, rb.nbr, rb.counts_dev, mirrored ? 1 : 0);
    SCN_CUDA_CHECK(cudaGetLastError());
  }
  rb.built = true;
  g_rulebook_builds.fetch_add(1);
  return SCN_OK;
}

// ------------------------------------------------------------------------------------------
// strided rulebook (Convolution / MaxPooling; Deconvolution reads it transposed)
// ------------------------------------------------------------------------------------------

// For input site x and candidate t in [0, tmax): the t-th output (row-major over the output
// region, last dimension fastest) that x feeds, and the filter offset it feeds it through.
// Output region per dimension: lb = max(0, (x - f + s) / s), ub = min(out - 1, x / s)
// (RectangularRegions.h:108-119); offset = sum (x_d - o_d * s_d) * prod_{j>d} f_j
// (RectangularRegions.h:30-38,94-105).
__device__ inline bool strided_target(const KeyLayout &L, const FilterDesc &F, const int *x, int t,
                                      int *o, int &k) {
  k = 0;
  int mult = 1;
  for (int d = L.dim - 1; d >= 0; --d) {
    int num = x[d] - F.f[d] + F.s[d];
    int lb = num > 0 ? num / F.s[d] : 0;
    int ub = min(F.out_size[d] - 1, x[d] / F.s[d]);
    int j = t % F.tdim[d];
    t /= F.tdim[d];
    int od = lb + j;
    if (od > ub) return false;
    o[d] = od;
    k += (x[d] - od * F.s[d]) * mult;
    mult *= F.f[d];
  }
  return true;
}

// The builders of a strided rulebook take the number of input sites either from the host (`n_in`,
// n_in_dev null) or, inside a chain of levels whose counts the host has not seen yet, from the device
// (*n_in_dev, with `n_in` the host's upper bound that sized the launch and the arrays): candidates
// between the real count and the bound are marked "no site" so that the scan over the bound counts
// only real ones.
__device__ __forceinline__ long long sites_here(const int *n_dev, long long bound) {
  if (!n_dev) return bound;
  long long n = *n_dev;
  return n < bound ? n : bound;
}

__global__ void k_strided_insert(KeyLayout Lin, KeyLayout Lout, FilterDesc F, HashTable Tout,
                                 const unsigned long long *__restrict__ in_keys, long long n_in,
                                 const int *__restrict__ n_in_dev, int *__restrict__ slot_of, int *flags) {
  long long id = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (id >= n_in * F.tmax) return;
  if (id >= sites_here(n_in_dev, n_in) * F.tmax) {
    slot_of[id] = -1;
    return;
  }
  long long i = id / F.tmax;
  int t = (int)(id % F.tmax);
  unsigned long long key = in_keys[i];
  unsigned long long okey = kEmptyKey;
  if (key != kEmptyKey) {
    int x[kMaxDim], o[kMaxDim], b, k;
    unpack_key(Lin, key, x, b);
    if (strided_target(Lin, F, x, t, o, k)) okey = pack_key(Lout, o, b);
  }
  // Candidates of one warp that name the same output site (neighbouring input rows usually do) insert
  // it once: the lowest lane of the group, which also holds the group's smallest id, does the insert
  // and hands the slot to the others.
  const unsigned peers = __match_any_sync(__activemask(), okey);
  const int leader = __ffs(peers) - 1;
  int s_out = -1;
  if (okey != kEmptyKey && (int)(threadIdx.x & 31) == leader) {
    long long s = hash_insert(Tout, okey);
    if (s < 0)
      atomicOr(flags, FLAG_TABLE_FULL);
    else {
      s_out = (int)s;
      atomicMin(&Tout.slots[s].aux, (unsigned)id);
    }
  }
  slot_of[id] = __shfl_sync(peers, s_out, leader);
}

__global__ void k_strided_fill(KeyLayout Lin, FilterDesc F, const Slot *__restrict__ slots,
                               const unsigned long long *__restrict__ in_keys,
                               const int *__restrict__ slot_of, long long n_in, long long n_out,
                               const int *__restrict__ n_out_dev, long long capacity,
                               int *__restrict__ nbr, unsigned long long *counts) {
  long long id = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (id >= n_in * F.tmax) return;
  int s = slot_of[id];
  if (s < 0) return;
  if (n_out_dev) {  // inside a chain: the level's row count is on the device only
    n_out = *n_out_dev;
    if (n_out > capacity) return;  // the level overflowed its arrays and will be rebuilt
  }
  long long i = id / F.tmax;
  int t = (int)(id % F.tmax);
  int x[kMaxDim], o[kMaxDim], b, k;
  unpack_key(Lin, in_keys[i], x, b);
  strided_target(Lin, F, x, t, o, k);
  // one read of the slot per group of lanes that share it
  const unsigned same = __match_any_sync(__activemask(), s);
  const int first = __ffs(same) - 1;
  int orow = ((int)(threadIdx.x & 31) == first) ? slots[s].row : 0;
  orow = __shfl_sync(same, orow, first);
  nbr[(long long)k * n_out + orow] = (int)i;
  // one counter update per distinct offset in the warp
  unsigned peers = __match_any_sync(__activemask(), k);
  if ((int)(threadIdx.x & 31) == __ffs(peers) - 1) atomicAdd(&counts[k], (unsigned long long)__popc(peers));
}

int get_strided_rulebook(scn_metadata *md, const int64_t *input_size, const int64_t *output_size,
                         const int64_t *filter_size, const int64_t *filter_stride,
                         cudaStream_t stream, Rulebook **out) {
  SCN_TRY(md_touch(md, stream));
  auto key = make_key(md->dim, input_size, filter_size, filter_stride);
  Rulebook &rb = md->strided_rules[key];
  *out = &rb;
  if (rb.built) return SCN_OK;
  if (md->pending) {  // it may be one of a chain that was started on the side stream
    SCN_TRY(chain_finalize(md, stream, nullptr));
    if (rb.built) return SCN_OK;
  }
  Grid *gin = find_grid(md, input_size);
  if (!gin) {
    md->strided_rules.erase(key);
    set_error("strided rulebook: no grid for the input spatial size");
    return SCN_ERR_NO_GRID;
  }
  SCN_TRY(ensure_scratch(md, stream));
  FilterDesc F{};
  long long K = 1;
  F.tmax = 1;
  for (int d = 0; d < md->dim; ++d) {
    SCN_REQUIRE(filter_size[d] >= 1 && filter_size[d] <= 127 && filter_stride[d] >= 1 &&
                    filter_stride[d] <= 127 && output_size[d] >= 1 && output_size[d] <= INT_MAX,
                SCN_ERR_UNSUPPORTED, "filter/stride/output size unsupported");
    F.f[d] = (int)filter_size[d];
    F.s[d] = (int)filter_stride[d];
    F.out_size[d] = (int)output_size[d];
    F.tdim[d] = (int)ceil_div(filter_size[d], filter_stride[d]);
    F.tmax *= F.tdim[d];
    K *= filter_size[d];
  }
  SCN_REQUIRE(K <= 4096 && F.tmax <= 4096, SCN_ERR_UNSUPPORTED, "filter volume unsupported");
  long long n_in = gin->n_active;
  long long n_ids = n_in * F.tmax;
  SCN_REQUIRE(n_ids < (1ll << 31), SCN_ERR_UNSUPPORTED, "too many (site, output) candidates");

  auto okey = make_key(md->dim, output_size);
  auto old = md->grids.find(okey);
  if (old != md->grids.end()) {
    free_grid(old->second, stream);
    md->grids.erase(old);
  }
  Grid gout;
  SCN_TRY(make_layout(md->dim, output_size, gout.layout));
  SCN_REQUIRE(gout.layout.batch_bits >= gin->layout.batch_bits ||
                  gin->batch_size <= (1ll << gout.layout.batch_bits),
              SCN_ERR_KEY_BITS, "batch index does not fit the output key");
  gout.batch_size = gin->batch_size;

  const int threads = 256;
  int *slot_of = nullptr, *flag = nullptr, *rank = nullptr;
  long long n_out = 0;
  if (n_ids > 0) {
    SCN_TRY(device_alloc((void **)&slot_of, sizeof(int) * (size_t)n_ids, stream));
    SCN_TRY(device_alloc((void **)&flag, sizeof(int) * (size_t)n_ids, stream));
    SCN_TRY(device_alloc((void **)&rank, sizeof(int) * (size_t)n_ids, stream));
    unsigned blocks = (unsigned)ceil_div(n_ids, threads);
    long long expect = n_in;
    for (int attempt = 0;; ++attempt) {
      SCN_TRY(alloc_table(gout.table, expect, stream));
      SCN_LAUNCH(k_strided_insert, blocks, threads, 0, stream, gin->layout, gout.layout, F, gout.table, gin->row_keys, n_in, nullptr, slot_of, md->flags_dev);
      SCN_LAUNCH(k_flag_first, blocks, threads, 0, stream, gout.table.slots, slot_of, n_ids, flag);
      SCN_TRY(exclusive_scan_i32(flag, rank, n_ids, &md->scalars_dev[0], stream));
      SCN_CUDA_CHECK(cudaGetLastError());
      int flags = 0, sc[4];
      SCN_TRY(fetch_flags(md, stream, &flags, sc));
      if ((flags & FLAG_TABLE_FULL) && attempt < 3) {  // more coarse sites than guessed: grow
        device_free(gout.table.slots, stream);
        gout.table = HashTable{};
        expect *= 4;
        continue;
      }
      int st = flags_to_status(flags);
      if (st != SCN_OK) {
        device_free(slot_of, stream);
        device_free(flag, stream);
        device_free(rank, stream);
        free_grid(gout, stream);
        md->strided_rules.erase(key);
        return st;
      }
      n_out = sc[0];
      break;
    }
  } else {
    SCN_TRY(alloc_table(gout.table, 0, stream));
  }
  gout.n_active = n_out;
  SCN_TRY(device_alloc((void **)&gout.row_keys, sizeof(unsigned long long) * (size_t)std::max<long long>(n_out, 1), stream));
  rb.n_offsets = (int)K;
  rb.n_in = n_in;
  rb.n_out = n_out;
  size_t nbr_bytes = sizeof(int) * (size_t)(K * std::max<long long>(n_out, 1));
  SCN_TRY(device_alloc((void **)&rb.nbr, nbr_bytes, stream));
  SCN_CUDA_CHECK(cudaMemsetAsync(rb.nbr, 0xFF, nbr_bytes, stream));
  SCN_TRY(device_alloc((void **)&rb.counts_dev, sizeof(unsigned long long) * (size_t)K, stream));
  SCN_CUDA_CHECK(cudaMemsetAsync(rb.counts_dev, 0, sizeof(unsigned long long) * (size_t)K, stream));
  if (n_ids > 0) {
    unsigned blocks = (unsigned)ceil_div(n_ids, threads);
    const long long n_slots = 2 * (long long)gout.table.n_buckets;
    SCN_LAUNCH(k_number_slots, (unsigned)ceil_div(n_slots, threads), threads, 0, stream, gout.table.slots, n_slots, rank, n_out, md->flags_dev, gout.row_keys);
    SCN_LAUNCH(k_strided_fill, blocks, threads, 0, stream, gin->layout, F, gout.table.slots, gin->row_keys, slot_of, n_in, n_out, nullptr, n_out, rb.nbr, rb.counts_dev);
    SCN_CUDA_CHECK(cudaGetLastError());
  }
  device_free(slot_of, stream);
  device_free(flag, stream);
  device_free(rank, stream);
  md->grids[okey] = gout;
  rb.built = true;
  g_rulebook_builds.fetch_add(1);
  return SCN_OK;
}

// ---- a chain of strided levels ---------------------------------------------------------------
// An encoder asks for the same (filter, stride) rulebook at every level (2/2 in a U-Net, 3/2 in a ResNet),
// each level's input being the last level's output.  Built one call at a time, every level ends with the host waiting for its row count
// (the next level's arrays and launches are sized by it), the GPU idling through each round trip.
// Here the whole chain is enqueued at once: level l reads its number of input sites from the device
// (`lev[l]`), its launches and arrays are sized by a bound the host knows, and one mailbox read at the
// end fetches every level's count.  With disjoint windows (filter == stride) a level has at most as
// many sites as its input; the arrays are sized for half of the input bound (surfaces and volumes
// shrink by 2.5x to 8x per level in 3-D); with overlapping windows they are sized for as many sites as
// the input has.  A level that needs more raises its own flag, after which that level and the deeper
// ones are enqueued again with the safe bound (one site per candidate).  Same kernels, same numbering
// (first touch in input-row order) as one call per level.
constexpr int kMaxChain = 16;

struct ChainLevel {
  std::vector<int64_t> in_size, out_size;
  FilterDesc F{};
  long long K = 1;
  Grid gout;
  Rulebook rb;
  long long bound_in = 0, cap_out = 0;
  int *slot_of = nullptr, *flag = nullptr, *rank = nullptr, *scan = nullptr;  // scratch of the level's build
};

__global__ void k_chain_init(int *lev, int n_ints, int n0) {
  for (int i = threadIdx.x; i < n_ints; i += blockDim.x) lev[i] = i == 0 ? n0 : 0;
}

__global__ void k_chain_post(const int *lev, int n_ints, volatile int *mailbox) {
  for (int i = threadIdx.x; i < n_ints; i += blockDim.x) mailbox[i] = lev[i];
  __threadfence_system();
}

static void chain_free_level(ChainLevel &lv, bool keep_result, cudaStream_t stream) {
  device_free(lv.slot_of, stream);
  device_free(lv.flag, stream);
  device_free(lv.rank, stream);
  device_free(lv.scan, stream);
  lv.slot_of = lv.flag = lv.rank = lv.scan = nullptr;
  if (!keep_result) {
    free_grid(lv.gout, stream);
    free_rulebook(lv.rb, stream);
  }
}

// Memory first, work second.  Everything the chain needs is allocated on `alloc_stream` (stream-ordered
// allocation: the blocks may be ones that earlier work of THAT stream is still using), and only then are the
// memsets and kernels enqueued on `stream`.  With two different streams the caller orders `stream` behind
// `alloc_stream` between the two calls and frees the scratch later, on a stream that is ordered behind `stream`.
static int chain_allocate(std::vector<ChainLevel> &plan, cudaStream_t alloc_stream) {
  for (auto &lv : plan) {
    const size_t n_ids = (size_t)std::max<long long>(lv.bound_in * lv.F.tmax, 1), cap = (size_t)std::max<long long>(lv.cap_out, 1);
    SCN_TRY(device_alloc((void **)&lv.slot_of, sizeof(int) * n_ids, alloc_stream));
    SCN_TRY(device_alloc((void **)&lv.flag, sizeof(int) * n_ids, alloc_stream));
    SCN_TRY(device_alloc((void **)&lv.rank, sizeof(int) * n_ids, alloc_stream));
    SCN_TRY(device_alloc((void **)&lv.scan, sizeof(int) * exclusive_scan_scratch_ints((long long)n_ids), alloc_stream));
    const unsigned long long slots = next_pow2((unsigned long long)std::max<long long>(64, 2 * lv.cap_out));
    SCN_REQUIRE(slots < (1ull << 31), SCN_ERR_UNSUPPORTED, "site table too large (%llu slots)", slots);
    lv.gout.table.n_buckets = slots / 2;
    SCN_TRY(device_alloc((void **)&lv.gout.table.slots, slots * sizeof(Slot), alloc_stream));
    SCN_TRY(device_alloc((void **)&lv.gout.row_keys, sizeof(unsigned long long) * cap, alloc_stream));
    SCN_TRY(device_alloc((void **)&lv.rb.nbr, sizeof(int) * (size_t)lv.K * cap, alloc_stream));
    SCN_TRY(device_alloc((void **)&lv.rb.counts_dev, sizeof(unsigned long long) * (size_t)lv.K, alloc_stream));
  }
  return SCN_OK;
}

static int chain_enqueue(scn_metadata *md, const Grid *gin, std::vector<ChainLevel> &plan, int *lev,
                         cudaStream_t stream) {
  const int L = (int)plan.size(), threads = 256;
  SCN_LAUNCH(k_chain_init, 1, 64, 0, stream, lev, 2 * L + 1, (int)gin->n_active);
  const unsigned long long *in_keys = gin->row_keys;
  KeyLayout Lin = gin->layout;
  for (int l = 0; l < L; ++l) {
    ChainLevel &lv = plan[l];
    const size_t cap = (size_t)std::max<long long>(lv.cap_out, 1);
    // key = all ones (free), row = -1, aux = 0xFFFFFFFF
    SCN_CUDA_CHECK(cudaMemsetAsync(lv.gout.table.slots, 0xFF, 2 * lv.gout.table.n_buckets * sizeof(Slot), stream));
    SCN_CUDA_CHECK(cudaMemsetAsync(lv.rb.nbr, 0xFF, sizeof(int) * (size_t)lv.K * cap, stream));
    SCN_CUDA_CHECK(cudaMemsetAsync(lv.rb.counts_dev, 0, sizeof(unsigned long long) * (size_t)lv.K, stream));
    if (lv.bound_in > 0) {
      const long long n_ids = lv.bound_in * lv.F.tmax;  // (site, output it may feed) candidates
      const unsigned blocks = (unsigned)ceil_div(n_ids, threads);
      int *n_in_dev = lev + l, *n_out_dev = lev + l + 1, *level_flags = lev + L + 1 + l;
      SCN_LAUNCH(k_strided_insert, blocks, threads, 0, stream, Lin, lv.gout.layout, lv.F, lv.gout.table, in_keys, lv.bound_in, n_in_dev, lv.slot_of, level_flags);
      SCN_LAUNCH(k_flag_first, blocks, threads, 0, stream, lv.gout.table.slots, lv.slot_of, n_ids, lv.flag);
      SCN_TRY(exclusive_scan_i32(lv.flag, lv.rank, n_ids, n_out_dev, stream, lv.scan));
      const long long n_slots = 2 * (long long)lv.gout.table.n_buckets;
      SCN_LAUNCH(k_number_slots, (unsigned)ceil_div(n_slots, threads), threads, 0, stream, lv.gout.table.slots, n_slots, lv.rank, lv.cap_out, level_flags, lv.gout.row_keys);
      SCN_LAUNCH(k_strided_fill, blocks, threads, 0, stream, Lin, lv.F, lv.gout.table.slots, in_keys, lv.slot_of, lv.bound_in, 0ll, n_out_dev, lv.cap_out, lv.rb.nbr, lv.rb.counts_dev);
      SCN_CUDA_CHECK(cudaGetLastError());
    }
    in_keys = lv.gout.row_keys;
    Lin = lv.gout.layout;
  }
  return SCN_OK;
}

// ---- plan / launch / collect: the three parts of a chain ------------------------------------------------------
// plan: sizes, layouts and bounds of the levels below `start` that can be chained (stops at the first level that
// is already there, does not divide, or does not fit the key)
static void chain_plan(scn_metadata *md, const Grid *gin, const std::vector<int64_t> &start, const int64_t *filter,
                       const int64_t *stride, int levels, bool safe, std::vector<ChainLevel> &plan) {
  const int dim = md->dim;
  std::vector<int64_t> cur = start;
  long long bound = gin->n_active;
  for (int l = 0; l < levels; ++l) {
    ChainLevel lv;
    lv.in_size = cur;
    lv.out_size.resize(dim);
    bool ok = true;
    lv.F.tmax = 1;
    long long out_volume = gin->batch_size;
    for (int d = 0; d < dim; ++d) {
      const int64_t f = filter[d], st = stride[d];
      if (cur[d] < f || (cur[d] - f) % st != 0) ok = false;
      lv.out_size[d] = ok ? (cur[d] - f) / st + 1 : 1;
      if (lv.out_size[d] > INT_MAX) ok = false;
      lv.F.f[d] = (int)f;
      lv.F.s[d] = (int)st;
      lv.F.out_size[d] = (int)lv.out_size[d];
      lv.F.tdim[d] = (int)ceil_div(f, st);
      lv.F.tmax *= lv.F.tdim[d];
      lv.K *= f;
      out_volume = out_volume > (1ll << 40) ? out_volume : out_volume * lv.out_size[d];
    }
    if (!ok || lv.K > 4096 || lv.F.tmax > 4096 || bound * lv.F.tmax >= (1ll << 31)) break;
    auto found = md->strided_rules.find(make_key(dim, cur.data(), filter, stride));
    if (found != md->strided_rules.end() && found->second.built) break;
    if (md->grids.count(make_key(dim, lv.out_size.data()))) break;
    if (make_layout(dim, lv.out_size.data(), lv.gout.layout) != SCN_OK) break;
    if (!(lv.gout.layout.batch_bits >= gin->layout.batch_bits || gin->batch_size <= (1ll << lv.gout.layout.batch_bits)))
      break;
    lv.bound_in = bound;
    // Sites of the level: at most one per candidate (and no more than the output volume).  Disjoint windows
    // (filter == stride) give at most one site per input site, and the arrays are first sized for half of that;
    // overlapping windows are first sized for as many sites as the input has.  A level that needs more raises its
    // flag and is built again from the safe bound.
    const long long most = std::min(bound * lv.F.tmax, std::max<long long>(out_volume, 1));
    if (safe)
      lv.cap_out = most;
    else if (lv.F.tmax == 1)
      lv.cap_out = std::max((bound + 1) / 2, std::min<long long>(bound, 4096));
    else
      lv.cap_out = std::min(most, std::max<long long>(bound, 4096));
    if (lv.cap_out >= (1ll << 30)) break;
    bound = lv.cap_out;
    cur = lv.out_size;
    plan.push_back(std::move(lv));
  }
}

// launch: every level's kernels and the post of all counts and flags into `mailbox` (pinned, mapped), on `stream`;
// the plan's arrays and `lev` (2 L + 1 ints) were allocated before
static int chain_launch(scn_metadata *md, const Grid *gin, std::vector<ChainLevel> &plan, int *lev, int *mailbox,
                        cudaStream_t stream) {
  const int L = (int)plan.size();
  int *mailbox_dev = nullptr;
  SCN_CUDA_CHECK(cudaHostGetDevicePointer((void **)&mailbox_dev, mailbox, 0));
  SCN_TRY(chain_enqueue(md, gin, plan, lev, stream));
  SCN_LAUNCH(k_chain_post, 1, 64, 0, stream, lev, 2 * L + 1, mailbox_dev);
  SCN_CUDA_CHECK(cudaGetLastError());
  return SCN_OK;
}

// collect (after the host has seen the mailbox): the levels up to the first that overflowed its arrays become
// grids and rulebooks of the object, the others are freed.  Returns the number of good levels.
static int chain_collect(scn_metadata *md, long long n_in, long long batch_size, std::vector<ChainLevel> &plan,
                         const int64_t *filter, const int64_t *stride, const volatile int *host, cudaStream_t stream,
                         int *n_built) {
  const int dim = md->dim, L = (int)plan.size();
  int good = 0;
  while (good < L && host[L + 1 + good] == 0 && host[good + 1] <= plan[good].cap_out) ++good;
  for (int l = 0; l < L; ++l) {
    ChainLevel &lv = plan[l];
    if (l < good) {
      const long long n_out = host[l + 1];
      lv.gout.n_active = n_out;
      lv.gout.batch_size = batch_size;
      lv.rb.n_offsets = (int)lv.K;
      lv.rb.n_in = n_in;
      lv.rb.n_out = n_out;
      lv.rb.built = true;
      chain_free_level(lv, true, stream);
      md->grids[make_key(dim, lv.out_size.data())] = lv.gout;
      md->strided_rules[make_key(dim, lv.in_size.data(), filter, stride)] = lv.rb;
      g_rulebook_builds.fetch_add(1);
      if (n_built) ++*n_built;
      n_in = n_out;
    } else {
      chain_free_level(lv, false, stream);
    }
  }
  return good;
}

static bool chain_applies(int dim, const int64_t *filter_size, const int64_t *filter_stride) {
  for (int d = 0; d < dim; ++d)
    if (filter_size[d] < 1 || filter_size[d] > 127 || filter_stride[d] < 1 || filter_stride[d] > 127) return false;
  return true;
}

static Grid *find_grid_now(scn_metadata *md, const int64_t *spatial_size) {  // no pending chain is waited for
  auto it = md->grids.find(make_key(md->dim, spatial_size));
  return it == md->grids.end() ? nullptr : &it->second;
}

// A chain that was started on the side stream and whose counts the host has not looked at yet.
struct PendingChain {
  std::vector<ChainLevel> plan;
  std::vector<int64_t> filter, stride;
  long long n_in = 0, batch_size = 0;
  cudaEvent_t done = nullptr;
  int *mailbox = nullptr;
  int *lev = nullptr;  // the chain's device counters, freed when the chain is taken over
};

static cudaStream_t g_side_stream[64] = {nullptr};
static std::mutex g_side_mu;

static int side_stream(cudaStream_t *out) {
  int dev = 0;
  SCN_CUDA_CHECK(cudaGetDevice(&dev));
  SCN_REQUIRE(dev >= 0 && dev < 64, SCN_ERR_UNSUPPORTED, "device index %d unsupported", dev);
  std::lock_guard<std::mutex> lock(g_side_mu);
  if (!g_side_stream[dev]) SCN_CUDA_CHECK(cudaStreamCreateWithFlags(&g_side_stream[dev], cudaStreamNonBlocking));
  *out = g_side_stream[dev];
  return SCN_OK;
}

static int build_strided_chain_from(scn_metadata *md, std::vector<int64_t> start, const int64_t *filter,
                                    const int64_t *stride, int levels, bool safe, cudaStream_t stream, int *n_built);

// The host looks at a started chain: waits for its event (usually long past), makes its levels the object's, and
// builds again, on `stream` and with the safe bounds, whatever overflowed.
static int chain_finalize(scn_metadata *md, cudaStream_t stream, int *n_built) {
  PendingChain *p = md->pending;
  if (!p) return SCN_OK;
  md->pending = nullptr;
  if (cudaEventQuery(p->done) != cudaSuccess) note_host_wait();
  int st = SCN_OK;
  if (cudaEventSynchronize(p->done) != cudaSuccess) {
    set_error("strided chain: CUDA error while waiting for the level counts");
    st = SCN_ERR_CUDA;
  }
  cudaEventDestroy(p->done);
  const int L = (int)p->plan.size();
  int good = L;
  std::vector<int64_t> rest;
  if (st == SCN_OK) {
    good = chain_collect(md, p->n_in, p->batch_size, p->plan, p->filter.data(), p->stride.data(), p->mailbox, stream,
                         n_built);
    if (good < L) rest = p->plan[good].in_size;
  } else {
    for (auto &lv : p->plan) chain_free_level(lv, false, stream);
  }
  device_free(p->lev, stream);
  mailbox_release(p->mailbox);
  std::vector<int64_t> filter = p->filter, stride = p->stride;
  delete p;
  if (st == SCN_OK && good < L)
    st = build_strided_chain_from(md, rest, filter.data(), stride.data(), L - good, true, stream, n_built);
  return st;
}

// Drops a started chain (the object is cleared or destroyed): its arrays go back once its kernels have run.
static void chain_abandon(scn_metadata *md, cudaStream_t stream) {
  PendingChain *p = md->pending;
  if (!p) return;
  md->pending = nullptr;
  cudaEventSynchronize(p->done);
  cudaEventDestroy(p->done);
  for (auto &lv : p->plan) chain_free_level(lv, false, stream);
  device_free(p->lev, stream);
  mailbox_release(p->mailbox);
  delete p;
}

static int build_strided_chain_from(scn_metadata *md, std::vector<int64_t> start, const int64_t *filter,
                                    const int64_t *stride, int levels, bool safe, cudaStream_t stream, int *n_built) {
  while (levels >= 2) {
    Grid *gin = find_grid_now(md, start.data());
    if (!gin || gin->n_active >= (1ll << 31)) return SCN_OK;
    std::vector<ChainLevel> plan;
    chain_plan(md, gin, start, filter, stride, levels, safe, plan);
    const int L = (int)plan.size();
    if (L < 2) return SCN_OK;
    if (!md->mailbox) SCN_TRY(mailbox_acquire(&md->mailbox));
    int *lev = nullptr;
    int st = device_alloc((void **)&lev, sizeof(int) * (2 * L + 1), stream);
    if (st == SCN_OK) st = chain_allocate(plan, stream);
    if (st == SCN_OK) st = chain_launch(md, gin, plan, lev, md->mailbox, stream);
    device_free(lev, stream);
    if (st == SCN_OK) {
      note_host_wait();
      if (cudaStreamSynchronize(stream) != cudaSuccess) {
        set_error("strided chain: CUDA error while waiting for the level counts");
        st = SCN_ERR_CUDA;
      }
    }
    if (st != SCN_OK) {
      for (auto &lv : plan) chain_free_level(lv, false, stream);
      return st;
    }
    const int good = chain_collect(md, gin->n_active, gin->batch_size, plan, filter, stride, md->mailbox, stream, n_built);
    if (good == L) return SCN_OK;
    // a level shrank less than guessed: that level and the deeper ones again, arrays sized by the input
    start = plan[good].in_size;
    levels = L - good;
    safe = true;
  }
  return SCN_OK;
}

// Builds up to `levels` consecutive rulebooks of (filter_size, filter_stride) starting at the grid of
// `input_size`, each level's output size (in - f) / s + 1.  Does nothing (SCN_OK) where the chain does
// not apply -- fewer than two levels to build, sizes that do not divide, no grid, rulebooks already there --
// because the per-level call that follows builds or reports whatever is left.  A chain that was started
// earlier on the side stream is taken over here.
int build_strided_chain(scn_metadata *md, const int64_t *input_size, const int64_t *filter_size,
                        const int64_t *filter_stride, int levels, cudaStream_t stream, int *n_built) {
  if (n_built) *n_built = 0;
  SCN_TRY(md_touch(md, stream));
  SCN_TRY(chain_finalize(md, stream, n_built));
  if (!chain_applies(md->dim, filter_size, filter_stride)) return SCN_OK;
  return build_strided_chain_from(md, std::vector<int64_t>(input_size, input_size + md->dim), filter_size, filter_stride,
                                  std::min(levels, kMaxChain), false, stream, n_built);
}

// The same chain, started without waiting for it: its kernels go to a side stream of the device behind what
// `stream` holds now (the input grid), so they run beside whatever the caller enqueues on `stream` next -- the
// first level's convolutions of a U-Net -- and the host does not wait here.  Whoever first asks for one of those
// levels (a grid that is not there yet, the rulebook of a level, scn_md_strided_chain) finds the chain finished,
// reads the counts and makes the levels the object's.  Nothing is started when a chain is already under way.
int start_strided_chain(scn_metadata *md, const int64_t *input_size, const int64_t *filter_size,
                        const int64_t *filter_stride, int levels, cudaStream_t stream) {
  SCN_TRY(md_touch(md, stream));
  if (md->pending || !chain_applies(md->dim, filter_size, filter_stride)) return SCN_OK;
  Grid *gin = find_grid_now(md, input_size);
  if (!gin || gin->n_active >= (1ll << 31)) return SCN_OK;
  PendingChain *p = new PendingChain();
  chain_plan(md, gin, std::vector<int64_t>(input_size, input_size + md->dim), filter_size, filter_stride,
             std::min(levels, kMaxChain), false, p->plan);
  if (p->plan.size() < 2) {
    delete p;
    return SCN_OK;
  }
  // The chain's memory comes from `stream` (blocks that earlier work of `stream` gave back can be used again at
  // once; taken on the side stream the pool would have to find blocks nobody can still be using, and grows when it
  // finds none: single steps of 18-22 ms among 13.6 ms ones).  The side stream starts behind that point of
  // `stream`; the scratch goes back when the chain is taken over.
  cudaStream_t side = nullptr;
  cudaEvent_t ready = nullptr;
  int st = side_stream(&side);
  if (st == SCN_OK) st = mailbox_acquire(&p->mailbox);
  if (st == SCN_OK) st = device_alloc((void **)&p->lev, sizeof(int) * (2 * p->plan.size() + 1), stream);
  if (st == SCN_OK) st = chain_allocate(p->plan, stream);
  if (st == SCN_OK && (cudaEventCreateWithFlags(&ready, cudaEventDisableTiming) != cudaSuccess ||
                       cudaEventCreateWithFlags(&p->done, cudaEventDisableTiming) != cudaSuccess ||
                       cudaEventRecord(ready, stream) != cudaSuccess || cudaStreamWaitEvent(side, ready, 0) != cudaSuccess)) {
    set_error("strided chain: could not order the side stream behind the caller's");
    st = SCN_ERR_CUDA;
  }
  bool launched = false;
  if (st == SCN_OK) {
    st = chain_launch(md, gin, p->plan, p->lev, p->mailbox, side);
    launched = true;  // (possibly in part)
  }
  if (st == SCN_OK && cudaEventRecord(p->done, side) != cudaSuccess) {
    set_error("strided chain: could not record the end of the chain");
    st = SCN_ERR_CUDA;
  }
  if (ready) cudaEventDestroy(ready);
  if (st != SCN_OK) {
    if (launched) cudaStreamSynchronize(side);  // what was enqueued must not outlive the arrays
    for (auto &lv : p->plan) chain_free_level(lv, false, stream);
    device_free(p->lev, stream);
    if (p->done) cudaEventDestroy(p->done);
    mailbox_release(p->mailbox);
    delete p;
    return st;
  }
  p->filter.assign(filter_size, filter_size + md->dim);
  p->stride.assign(filter_stride, filter_stride + md->dim);
  p->n_in = gin->n_active;
  p->batch_size = gin->batch_size;
  md->pending = p;
  return SCN_OK;
}

// ------------------------------------------------------------------------------------------
// rulebook views
// ------------------------------------------------------------------------------------------

// ---- rule counts: pinned chunks and events are pooled per device, never given back to the driver
namespace {
struct TicketPool {
  std::mutex mu;
  std::vector<unsigned long long *> chunks[64];  // kRMaxCounts values each
  std::vector<cudaEvent_t> events[64];
};
constexpr int kTicketValues = 256;  // filter volumes up to 256 offsets
TicketPool &ticket_pool() {
  static TicketPool *p = new TicketPool();  // leaked on purpose: tickets may be released at exit
  return *p;
}
}  // namespace

__global__ void k_post_counts(const unsigned long long *__restrict__ counts, volatile unsigned long long *host, int n) {
  for (int i = threadIdx.x; i < n; i += blockDim.x) host[i] = counts[i];
  __threadfence_system();
}

static int count_ticket_start(Rulebook &rb, cudaStream_t stream) {
  if (rb.ticket) return SCN_OK;
  SCN_REQUIRE(rb.n_offsets <= kTicketValues, SCN_ERR_UNSUPPORTED, "%d filter offsets", rb.n_offsets);
  int dev = 0;
  SCN_CUDA_CHECK(cudaGetDevice(&dev));
  SCN_REQUIRE(dev < 64, SCN_ERR_UNSUPPORTED, "device %d", dev);
  CountTicket *t = new CountTicket();
  t->n = rb.n_offsets;
  t->device = dev;
  {
    TicketPool &P = ticket_pool();
    std::lock_guard<std::mutex> lock(P.mu);
    if (!P.chunks[dev].empty()) {
      t->host = P.chunks[dev].back();
      P.chunks[dev].pop_back();
    }
    if (!P.events[dev].empty()) {
      t->event = P.events[dev].back();
      P.events[dev].pop_back();
    }
  }
  if (!t->host) {  // a slab of 256 chunks (512 KB of pinned memory) at a time
    unsigned long long *slab = nullptr;
    if (cudaHostAlloc((void **)&slab, sizeof(unsigned long long) * kTicketValues * 256,
                      cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) {
      cudaGetLastError();
      delete t;
      SCN_REQUIRE(false, SCN_ERR_CUDA, "pinned allocation failed");
    }
    t->host = slab;
    TicketPool &P = ticket_pool();
    std::lock_guard<std::mutex> lock(P.mu);
    for (int i = 1; i < 256; ++i) P.chunks[dev].push_back(slab + (size_t)i * kTicketValues);
  }
  if (!t->event && cudaEventCreateWithFlags(&t->event, cudaEventDisableTiming) != cudaSuccess) {
    cudaGetLastError();
    t->event = nullptr;
    count_ticket_release(t);
    SCN_REQUIRE(false, SCN_ERR_CUDA, "event creation failed");
  }
  // posted by a kernel into mapped host memory, not copied: a copy on this stream would hold the stream's next
  // kernels until the copy engine has finished whatever the application is copying (see the mailboxes above)
  unsigned long long *host_dev = nullptr;
  cudaError_t e = cudaHostGetDevicePointer((void **)&host_dev, t->host, 0);
  if (e == cudaSuccess) {
    SCN_LAUNCH(k_post_counts, 1, 256, 0, stream, rb.counts_dev, host_dev, rb.n_offsets);
    e = cudaGetLastError();
  }
  if (e == cudaSuccess) e = cudaEventRecord(t->event, stream);
  if (e != cudaSuccess) {
    // the rulebook gets the ticket only once its event has been recorded: a later wait on a
    // never-recorded event would return at once and sum whatever the chunk held
    cudaEventDestroy(t->event);  // possibly half-recorded: not returned to the pool
    t->event = nullptr;
    count_ticket_release(t);
    SCN_CUDA_CHECK(e);
  }
  rb.ticket = t;
  return SCN_OK;
}

void count_ticket_release(CountTicket *t) {
  if (!t || t->refs.fetch_sub(1) != 1) return;
  if (t->event) cudaEventSynchronize(t->event);  // the copy must not land in a chunk that was handed on
  TicketPool &P = ticket_pool();
  {
    std::lock_guard<std::mutex> lock(P.mu);
    if (t->host) P.chunks[t->device].push_back(t->host);
    if (t->event) P.events[t->device].push_back(t->event);
  }
  delete t;
}

int count_ticket_total(CountTicket *t, long long *total) {
  if (cudaEventQuery(t->event) != cudaSuccess) note_host_wait();  // an answer that already landed is no wait
  SCN_CUDA_CHECK(cudaEventSynchronize(t->event));
  long long s = 0;
  for (int k = 0; k < t->n; ++k) s += (long long)t->host[k];
  *total = s;
  return SCN_OK;
}

static void counts_from_ticket(Rulebook &rb) {
  rb.counts_host.assign(rb.ticket->host, rb.ticket->host + rb.n_offsets);
  long long t = 0;
  for (auto c : rb.counts_host) t += c;
  rb.total_rules = t;
}

// filter volumes beyond a ticket's chunk: plain copy and wait
static int rulebook_counts_blocking(Rulebook &rb, cudaStream_t stream) {
  std::vector<unsigned long long> h(rb.n_offsets);
  SCN_CUDA_CHECK(cudaMemcpyAsync(h.data(), rb.counts_dev, sizeof(unsigned long long) * rb.n_offsets,
                                 cudaMemcpyDeviceToHost, stream));
  note_host_wait();
  SCN_CUDA_CHECK(cudaStreamSynchronize(stream));
  rb.counts_host.assign(h.begin(), h.end());
  long long t = 0;
  for (auto c : rb.counts_host) t += c;
  rb.total_rules = t;
  return SCN_OK;
}

int rulebook_counts_async(Rulebook &rb, cudaStream_t stream) {
  if (rb.total_rules >= 0) return SCN_OK;
  if (rb.n_offsets > kTicketValues) return rulebook_counts_blocking(rb, stream);
  SCN_TRY(count_ticket_start(rb, stream));
  cudaError_t q = cudaEventQuery(rb.ticket->event);
  if (q == cudaSuccess) {
    counts_from_ticket(rb);
  } else if (q != cudaErrorNotReady) {
    SCN_CUDA_CHECK(q);
  }
  return SCN_OK;
}

int rulebook_counts(Rulebook &rb, cudaStream_t stream) {
  if (rb.total_rules >= 0) return SCN_OK;
  if (rb.n_offsets > kTicketValues) return rulebook_counts_blocking(rb, stream);
  SCN_TRY(count_ticket_start(rb, stream));
  note_host_wait();
  SCN_CUDA_CHECK(cudaEventSynchronize(rb.ticket->event));
  counts_from_ticket(rb);
  return SCN_OK;
}

__global__ void k_transpose_rules(const int *__restrict__ nbr, long long n_out, long long n_in, int K,
                                  int *__restrict__ tnbr) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)K * n_out) return;
  int i = nbr[idx];
  if (i < 0) return;
  long long k = idx / n_out, o = idx % n_out;
  tnbr[k * n_in + i] = (int)o;
}

int rulebook_transposed(Rulebook &rb, cudaStream_t stream) {
  if (rb.tnbr) return SCN_OK;
  size_t bytes = sizeof(int) * (size_t)(rb.n_offsets * std::max<long long>(rb.n_in, 1));
  SCN_TRY(device_alloc((void **)&rb.tnbr, bytes, stream));
  SCN_CUDA_CHECK(cudaMemsetAsync(rb.tnbr, 0xFF, bytes, stream));
  long long total = (long long)rb.n_offsets * rb.n_out;
  if (total > 0) {
    SCN_LAUNCH(k_transpose_rules, (unsigned)ceil_div(total, 256), 256, 0, stream, rb.nbr, rb.n_out, rb.n_in, rb.n_offsets, rb.tnbr);
    SCN_CUDA_CHECK(cudaGetLastError());
  }
  return SCN_OK;
}

__global__ void k_rule_flags(const int *__restrict__ nbr, long long total, int *__restrict__ flag) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx < total) flag[idx] = nbr[idx] >= 0;
}
__global__ void k_rule_compact(const int *__restrict__ nbr, const int *__restrict__ pos, long long total,
                               long long n_out, int *__restrict__ pairs) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  int i = nbr[idx];
  if (i < 0) return;
  long long p = pos[idx];
  pairs[2 * p] = i;
  pairs[2 * p + 1] = (int)(idx % n_out);
}

static int rulebook_export(Rulebook &rb, int64_t *n_offsets, int64_t *counts_host, int32_t *pairs_dev,
                           cudaStream_t stream) {
  SCN_TRY(rulebook_counts(rb, stream));
  if (n_offsets) *n_offsets = rb.n_offsets;
  if (counts_host)
    for (int k = 0; k < rb.n_offsets; ++k) counts_host[k] = rb.counts_host[k];
  if (!pairs_dev) return SCN_OK;
  long long total = (long long)rb.n_offsets * rb.n_out;
  if (total == 0) return SCN_OK;
  SCN_REQUIRE(total < (1ll << 31), SCN_ERR_UNSUPPORTED, "rulebook too large to export");
  int *flag = nullptr;
  SCN_TRY(device_alloc((void **)&flag, sizeof(int) * (size_t)total, stream));
  unsigned blocks = (unsigned)ceil_div(total, 256);
  SCN_LAUNCH(k_rule_flags, blocks, 256, 0, stream, rb.nbr, total, flag);
  SCN_TRY(exclusive_scan_i32(flag, flag, total, nullptr, stream));
  SCN_LAUNCH(k_rule_compact, blocks, 256, 0, stream, rb.nbr, flag, total, rb.n_out, pairs_dev);
  SCN_CUDA_CHECK(cudaGetLastError());
  SCN_TRY(device_free(flag, stream));
  return SCN_OK;
}

}  // namespace scn

// ------------------------------------------------------------------------------------------
// C ABI
// ------------------------------------------------------------------------------------------

using namespace scn;

extern "C" {

long long scn_rulebook_build_count(void) { return g_rulebook_builds.load(); }

int scn_md_create(int dimension, scn_metadata **md) {
  SCN_REQUIRE(md, SCN_ERR_BAD_ARG, "null output pointer");
  SCN_REQUIRE(dimension >= 1 && dimension <= SCN_MAX_DIMENSION, SCN_ERR_BAD_ARG,
              "dimension %d not in 1..%d", dimension, SCN_MAX_DIMENSION);
  *md = new scn_metadata();
  (*md)->dim = dimension;
  return SCN_OK;
}

int scn_md_clear(scn_metadata *md, void *stream) {
  SCN_REQUIRE(md, SCN_ERR_BAD_ARG, "null metadata");
  return md_clear(md, (cudaStream_t)stream);
}

static int md_destroy_on(scn_metadata *md, cudaStream_t stream) {
  if (!md) return SCN_OK;
  // free on the device that owns the tables, whatever device is current
  int current = -1;
  const bool switch_device = md->device >= 0 && cudaGetDevice(&current) == cudaSuccess && current != md->device;
  if (switch_device) cudaSetDevice(md->device);
  mailbox_release(md->mailbox);
  md->mailbox = nullptr;
  count_ticket_release(md->last_ticket);
  md->last_ticket = nullptr;
  md_clear(md, stream);
  device_free(md->flags_dev, stream);
  device_free(md->scalars_dev, stream);
  delete md;
  if (switch_device) cudaSetDevice(current);
  return SCN_OK;
}

int scn_md_destroy(scn_metadata *md) {
  // stream-ordered frees behind the last work enqueued on the object: kernels of that stream that
  // still read the tables finish before the memory can be handed out again
  return md_destroy_on(md, md ? md->last_stream : nullptr);
}

int scn_md_destroy_on_stream(scn_metadata *md, void *stream) { return md_destroy_on(md, (cudaStream_t)stream); }

int scn_md_input_layer(scn_metadata *md, const int64_t *spatial_size, const int64_t *coords,
                       int coords_on_device, int64_t n_rows, int n_cols, int64_t batch_size,
                       int mode, void *stream, int64_t *n_active) {
  return md_input_layer(md, spatial_size, coords, coords_on_device, n_rows, n_cols, batch_size, mode, 0,
                        (cudaStream_t)stream, n_active);
}

int scn_md_bl_input_layer(scn_metadata *md, const int64_t *spatial_size, const int64_t *coords,
                          int coords_on_device, int64_t batch_size, int64_t length, int mode, void *stream,
                          int64_t *n_active) {
  SCN_REQUIRE(md, SCN_ERR_BAD_ARG, "null metadata");
  SCN_REQUIRE(batch_size >= 0 && length >= 0, SCN_ERR_BAD_ARG, "negative batch size or length");
  SCN_REQUIRE(mode >= 0 && mode <= 4, SCN_ERR_BAD_ARG, "input layer mode %d not in 0..4", mode);
  // blRules keeps the LAST point of a site in mode 1 and the FIRST in mode 2 (IOLayersRules.h:172-199),
  // inputLayerRules the other way round (IOLayersRules.h:95-106): stored in the latter's terms.
  const int stored_mode = mode == 1 ? 2 : mode == 2 ? 1 : mode;
  // an empty batch x length array still needs a non-zero stride for the sample index
  SCN_TRY(md_input_layer(md, spatial_size, coords, coords_on_device, batch_size * length, md->dim, batch_size,
                         stored_mode, std::max<int64_t>(length, 1), (cudaStream_t)stream, n_active));
  return SCN_OK;
}

int scn_md_poll_errors(scn_metadata *md, void *stream) {
  SCN_REQUIRE(md, SCN_ERR_BAD_ARG, "null metadata");
  if (!md->flags_dev) return SCN_OK;
  SCN_TRY(md_touch(md, (cudaStream_t)stream));
  int flags = 0;
  SCN_TRY(fetch_flags(md, (cudaStream_t)stream, &flags, nullptr));
  return flags_to_status(flags);
}

int scn_md_n_active(scn_metadata *md, const int64_t *spatial_size, int64_t *n_active) {
  SCN_REQUIRE(md && spatial_size && n_active, SCN_ERR_BAD_ARG, "null argument");
  Grid *g = find_grid(md, spatial_size);
  // the reference's unordered_map lookup default-constructs a zero for an unknown size
  *n_active = g ? g->n_active : 0;
  return SCN_OK;
}

int scn_md_batch_size(scn_metadata *md, const int64_t *spatial_size, int64_t *batch_size) {
  SCN_REQUIRE(md && spatial_size && batch_size, SCN_ERR_BAD_ARG, "null argument");
  Grid *g = find_grid(md, spatial_size);
  *batch_size = g ? g->batch_size : 0;
  return SCN_OK;
}

int scn_md_spatial_locations(scn_metadata *md, const int64_t *spatial_size, int64_t *out_dev,
                             void *stream) {
  SCN_REQUIRE(md && spatial_size, SCN_ERR_BAD_ARG, "null argument");
  Grid *g = find_grid(md, spatial_size);
  SCN_REQUIRE(g, SCN_ERR_NO_GRID, "no grid for that spatial size");
  if (g->n_active == 0) return SCN_OK;
  SCN_REQUIRE(out_dev, SCN_ERR_BAD_ARG, "null output");
  SCN_TRY(md_touch(md, (cudaStream_t)stream));
  SCN_LAUNCH(k_spatial_locations, (unsigned)ceil_div(g->n_active, 256), 256, 0, (cudaStream_t)stream, g->layout, g->row_keys, g->n_active, (long long *)out_dev);
  SCN_CUDA_CHECK(cudaGetLastError());
  return SCN_OK;
}

int scn_md_submanifold_rulebook(scn_metadata *md, const int64_t *spatial_size,
                                const int64_t *filter_size, void *stream, int64_t *n_rules) {
  SCN_REQUIRE(md && spatial_size && filter_size, SCN_ERR_BAD_ARG, "null argument");
  Rulebook *rb = nullptr;
  SCN_TRY(get_submanifold_rulebook(md, spatial_size, filter_size, (cudaStream_t)stream, &rb));
  if (n_rules) {
    SCN_TRY(rulebook_counts(*rb, (cudaStream_t)stream));
    *n_rules = rb->total_rules;
  }
  return SCN_OK;
}

int scn_md_strided_chain(scn_metadata *md, const int64_t *input_size, const int64_t *filter_size,
                         const int64_t *filter_stride, int levels, void *stream, int *n_built) {
  SCN_REQUIRE(md && input_size && filter_size && filter_stride, SCN_ERR_BAD_ARG, "null argument");
  return build_strided_chain(md, input_size, filter_size, filter_stride, levels, (cudaStream_t)stream, n_built);
}

int scn_md_strided_chain_start(scn_metadata *md, const int64_t *input_size, const int64_t *filter_size,
                               const int64_t *filter_stride, int levels, void *stream) {
  SCN_REQUIRE(md && input_size && filter_size && filter_stride, SCN_ERR_BAD_ARG, "null argument");
  return start_strided_chain(md, input_size, filter_size, filter_stride, levels, (cudaStream_t)stream);
}

int scn_md_strided_rulebook(scn_metadata *md, const int64_t *input_size, const int64_t *output_size,
                            const int64_t *filter_size, const int64_t *filter_stride, void *stream,
                            int64_t *n_active_out, int64_t *n_rules) {
  SCN_REQUIRE(md && input_size && output_size && filter_size && filter_stride, SCN_ERR_BAD_ARG,
              "null argument");
  Rulebook *rb = nullptr;
  SCN_TRY(get_strided_rulebook(md, input_size, output_size, filter_size, filter_stride,
                               (cudaStream_t)stream, &rb));
  if (n_active_out) *n_active_out = rb->n_out;
  if (n_rules) {
    SCN_TRY(rulebook_counts(*rb, (cudaStream_t)stream));
    *n_rules = rb->total_rules;
  }
  return SCN_OK;
}

int scn_md_rulebook_export(scn_metadata *md, int kind, const int64_t *sizes_a, const int64_t *sizes_b,
                           const int64_t *sizes_c, int64_t *n_offsets, int64_t *counts_host,
                           int32_t *pairs_dev, void *stream) {
  SCN_REQUIRE(md && sizes_a && sizes_b, SCN_ERR_BAD_ARG, "null argument");
  Rulebook *rb = nullptr;
  if (kind == SCN_RULES_SUBMANIFOLD) {
    auto it = md->sub_rules.find(make_key(md->dim, sizes_a, sizes_b));
    if (it != md->sub_rules.end()) rb = &it->second;
  } else if (kind == SCN_RULES_STRIDED) {
    SCN_REQUIRE(sizes_c, SCN_ERR_BAD_ARG, "null stride");
    auto it = md->strided_rules.find(make_key(md->dim, sizes_a, sizes_b, sizes_c));
    if (it != md->strided_rules.end()) rb = &it->second;
  } else {
    SCN_REQUIRE(false, SCN_ERR_BAD_ARG, "unknown rulebook kind %d", kind);
  }
  SCN_REQUIRE(rb && rb->built, SCN_ERR_NO_GRID, "that rulebook has not been built");
  return rulebook_export(*rb, n_offsets, counts_host, pairs_dev, (cudaStream_t)stream);
}
}
