// Status strings, stream-ordered allocation and the device-wide prefix sum used by the
// rulebook builders.
#include <stdarg.h>

#include <atomic>
#include <mutex>

#include "common.cuh"

namespace scn {

static thread_local char g_last_error[512] = "";
static std::atomic<long long> g_launches{0};

void note_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
static std::atomic<long long> g_host_waits{0};
void note_host_wait() { g_host_waits.fetch_add(1, std::memory_order_relaxed); }

void set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
}

// The library's scratch memory (site tables, rulebooks, prepared weight images, partial sums) comes
// from a memory pool of its own per device, not from the device's default pool: its release
// threshold is raised so that freed blocks are reused instead of going back to the driver at every
// synchronisation, and that setting must not leak to other users of cudaMallocAsync in the process.
// scn_trim_memory gives idle blocks back.
static cudaMemPool_t g_pool[64] = {nullptr};
static std::mutex g_pool_mu;

static int device_pool(cudaMemPool_t *pool) {
  int dev = 0;
  SCN_CUDA_CHECK(cudaGetDevice(&dev));
  SCN_REQUIRE(dev >= 0 && dev < 64, SCN_ERR_UNSUPPORTED, "device index %d unsupported", dev);
  std::lock_guard<std::mutex> lock(g_pool_mu);
  if (!g_pool[dev]) {
    cudaMemPoolProps props = {};
    props.allocType = cudaMemAllocationTypePinned;
    props.handleTypes = cudaMemHandleTypeNone;
    props.location.type = cudaMemLocationTypeDevice;
    props.location.id = dev;
    cudaMemPool_t p = nullptr;
    SCN_CUDA_CHECK(cudaMemPoolCreate(&p, &props));
    unsigned long long keep = ~0ull;
    SCN_CUDA_CHECK(cudaMemPoolSetAttribute(p, cudaMemPoolAttrReleaseThreshold, &keep));
    g_pool[dev] = p;
  }
  *pool = g_pool[dev];
  return SCN_OK;
}

int device_alloc(void **p, size_t bytes, cudaStream_t stream) {
  cudaMemPool_t pool = nullptr;
  SCN_TRY(device_pool(&pool));
  *p = nullptr;
  if (bytes == 0) bytes = 16;
  SCN_CUDA_CHECK(cudaMallocFromPoolAsync(p, bytes, pool, stream));
  return SCN_OK;
}

int device_free(void *p, cudaStream_t stream) {
  if (p) SCN_CUDA_CHECK(cudaFreeAsync(p, stream));
  return SCN_OK;
}

// ---- exclusive scan -----------------------------------------------------------------------
// Three passes over tiles of 4096 values: per-tile sums, a recursive scan of those sums, and
// a per-tile scan seeded with the tile's base.  All int32; callers keep totals below 2^31.

constexpr int kScanThreads = 1024;
constexpr int kScanItems = 4;
constexpr int kScanTile = kScanThreads * kScanItems;

__device__ inline int block_exclusive_scan(int v, int &block_total) {
  __shared__ int warp_sums[32];
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int w = warp_sums[lane];
    int wi = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int t = __shfl_up_sync(0xffffffffu, wi, o);
      if (lane >= o) wi += t;
    }
    warp_sums[lane] = wi - w;  // exclusive offset of each warp
    if (lane == 31) block_total = wi;
  }
  __syncthreads();
  int base = warp_sums[warp];
  return base + incl - v;
}

__global__ void __launch_bounds__(kScanThreads) k_scan_tile_sums(const int *in, int *tile_sums,
                                                                 long long n) {
  __shared__ int total;
  long long base = (long long)blockIdx.x * kScanTile + (long long)threadIdx.x * kScanItems;
  int s = 0;
#pragma unroll
  for (int i = 0; i < kScanItems; ++i)
    if (base + i < n) s += in[base + i];
  block_exclusive_scan(s, total);
  if (threadIdx.x == 0) tile_sums[blockIdx.x] = total;
}

__global__ void __launch_bounds__(kScanThreads) k_scan_tiles(const int *in, int *out,
                                                             const int *tile_base, long long n,
                                                             int *total_dev) {
  __shared__ int total;
  long long base = (long long)blockIdx.x * kScanTile + (long long)threadIdx.x * kScanItems;
  int v[kScanItems];
  int s = 0;
#pragma unroll
  for (int i = 0; i < kScanItems; ++i) {
    v[i] = (base + i < n) ? in[base + i] : 0;
    s += v[i];
  }
  int excl = block_exclusive_scan(s, total) + (tile_base ? tile_base[blockIdx.x] : 0);
#pragma unroll
  for (int i = 0; i < kScanItems; ++i) {
    if (base + i < n) out[base + i] = excl;
    excl += v[i];
  }
  if (total_dev && blockIdx.x == gridDim.x - 1 && threadIdx.x == 0)
    *total_dev = total + (tile_base ? tile_base[blockIdx.x] : 0);
}

__global__ void k_set_zero(int *p) { *p = 0; }

size_t exclusive_scan_scratch_ints(long long n) {
  size_t total = 0;
  for (long long tiles = ceil_div(std::max<long long>(n, 1), kScanTile); tiles > 1; tiles = ceil_div(tiles, kScanTile))
    total += (size_t)tiles;
  return total + 1;
}

// `scratch` (optional): exclusive_scan_scratch_ints(n) ints the caller owns, so that nothing is allocated here
int exclusive_scan_i32(const int *in, int *out, long long n, int *total_dev, cudaStream_t stream, int *scratch) {
  if (n <= 0) {
    if (total_dev) SCN_LAUNCH(k_set_zero, 1, 1, 0, stream, total_dev);
    return SCN_OK;
  }
  long long tiles = ceil_div(n, kScanTile);
  if (tiles == 1) {
    SCN_LAUNCH(k_scan_tiles, 1, kScanThreads, 0, stream, in, out, nullptr, n, total_dev);
    SCN_CUDA_CHECK(cudaGetLastError());
    return SCN_OK;
  }
  int *sums = scratch;
  if (!sums) SCN_TRY(device_alloc((void **)&sums, sizeof(int) * (size_t)tiles, stream));
  SCN_LAUNCH(k_scan_tile_sums, (unsigned)tiles, kScanThreads, 0, stream, in, sums, n);
  SCN_CUDA_CHECK(cudaGetLastError());
  SCN_TRY(exclusive_scan_i32(sums, sums, tiles, nullptr, stream, scratch ? scratch + tiles : nullptr));
  SCN_LAUNCH(k_scan_tiles, (unsigned)tiles, kScanThreads, 0, stream, in, out, sums, n, total_dev);
  SCN_CUDA_CHECK(cudaGetLastError());
  if (!scratch) SCN_TRY(device_free(sums, stream));
  return SCN_OK;
}

}  // namespace scn

extern "C" {

int scn_abi_version(void) { return SCN_ABI_VERSION; }

long long scn_launch_count(void) { return scn::g_launches.load(std::memory_order_relaxed); }
long long scn_host_wait_count(void) { return scn::g_host_waits.load(std::memory_order_relaxed); }

int scn_memory_usage(uint64_t *reserved_bytes, uint64_t *used_bytes) {
  using namespace scn;
  SCN_REQUIRE(reserved_bytes && used_bytes, SCN_ERR_BAD_ARG, "null argument");
  *reserved_bytes = *used_bytes = 0;
  int dev = 0;
  SCN_CUDA_CHECK(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lock(g_pool_mu);
  if (dev >= 0 && dev < 64 && g_pool[dev]) {
    unsigned long long r = 0, u = 0;
    SCN_CUDA_CHECK(cudaMemPoolGetAttribute(g_pool[dev], cudaMemPoolAttrReservedMemCurrent, &r));
    SCN_CUDA_CHECK(cudaMemPoolGetAttribute(g_pool[dev], cudaMemPoolAttrUsedMemCurrent, &u));
    *reserved_bytes = r;
    *used_bytes = u;
  }
  return SCN_OK;
}

int scn_trim_memory(uint64_t keep_bytes) {
  using namespace scn;
  int dev = 0;
  SCN_CUDA_CHECK(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lock(g_pool_mu);
  if (dev >= 0 && dev < 64 && g_pool[dev]) SCN_CUDA_CHECK(cudaMemPoolTrimTo(g_pool[dev], (size_t)keep_bytes));
  return SCN_OK;
}

const char *scn_last_error(void) { return scn::g_last_error; }

const char *scn_status_string(int status) {
  switch (status) {
    case SCN_OK: return "ok";
    case SCN_ERR_BAD_ARG: return "bad argument";
    case SCN_ERR_CUDA: return "CUDA runtime error";
    case SCN_ERR_COORD_RANGE: return "coordinate or batch index out of range";
    case SCN_ERR_KEY_BITS: return "spatial size x batch does not fit a 63-bit site key";
    case SCN_ERR_NO_GRID: return "no grid for that spatial size";
    case SCN_ERR_TABLE_FULL: return "site hash probe limit reached";
    case SCN_ERR_UNSUPPORTED: return "unsupported shape";
    case SCN_ERR_SIZE_MISMATCH: return "size mismatch";
    default: return "unknown status";
  }
}
}
