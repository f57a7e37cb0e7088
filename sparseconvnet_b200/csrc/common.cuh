// Shared definitions of the sm_100a sparse-convolution library: status handling, the packed
// site key, and the open-addressing site hash used by every rulebook kernel.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <string>

#include "../../include/scn_b200.h"

namespace scn {

// ---- status -----------------------------------------------------------------------------

void set_error(const char *fmt, ...);

#define SCN_CUDA_CHECK(expr)                                                                   \
  do {                                                                                         \
    cudaError_t _e = (expr);                                                                   \
    if (_e != cudaSuccess) {                                                                   \
      scn::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__,         \
                     __LINE__);                                                                \
      return SCN_ERR_CUDA;                                                                     \
    }                                                                                          \
  } while (0)

#define SCN_TRY(expr)                                                                          \
  do {                                                                                         \
    int _s = (expr);                                                                           \
    if (_s != SCN_OK) return _s;                                                               \
  } while (0)

#define SCN_REQUIRE(cond, code, ...)                                                           \
  do {                                                                                         \
    if (!(cond)) {                                                                             \
      scn::set_error(__VA_ARGS__);                                                             \
      return (code);                                                                           \
    }                                                                                          \
  } while (0)

// Every kernel launch of the library goes through this macro so that the number of launches
// can be read back (scn_launch_count), e.g. to state how many kernels a timed region ran.
void note_launch();
// Every place where the library makes the calling thread wait for the GPU (a stream or event
// synchronisation) notes it; scn_host_wait_count reads the total.
void note_host_wait();
#define SCN_LAUNCH(kernel, grid, block, smem, stream, ...)                                      \
  do {                                                                                         \
    scn::note_launch();                                                                        \
    kernel<<<(grid), (block), (smem), (stream)>>>(__VA_ARGS__);                                \
  } while (0)

// Kernels report problems by OR-ing a bit into a device word; the host reads it at the next
// point where it waits for the stream anyway.  Nothing on the device traps.
enum DeviceFlag : int {
  FLAG_COORD_RANGE = 1,
  FLAG_TABLE_FULL = 2,
  FLAG_BAD_ROW = 4,
  FLAG_TC_TIMEOUT = 8,
};

// ---- packed site key ----------------------------------------------------------------------
//
// A site (batch index, x_0 .. x_{D-1}) is packed into one 64-bit word: coordinate d occupies
// bits [shift[d], shift[d] + bits[d]), the batch index the bits above batch_shift.  Because
// every coordinate is range-checked against its field before packing, the key of a neighbour
// is the site's key plus a precomputed signed delta.  The all-ones word is the empty marker.

constexpr int kMaxDim = SCN_MAX_DIMENSION;
constexpr unsigned long long kEmptyKey = 0xFFFFFFFFFFFFFFFFull;

struct KeyLayout {
  int dim;
  int shift[kMaxDim];
  int bits[kMaxDim];
  int size[kMaxDim];  // spatial size per dimension
  int batch_shift;
  int batch_bits;
};

__host__ __device__ inline unsigned long long pack_key(const KeyLayout &L, const int *x, int b) {
  unsigned long long k = (unsigned long long)(unsigned)b << L.batch_shift;
  for (int d = 0; d < L.dim; ++d) k |= (unsigned long long)(unsigned)x[d] << L.shift[d];
  return k;
}
__host__ __device__ inline void unpack_key(const KeyLayout &L, unsigned long long k, int *x,
                                           int &b) {
  for (int d = 0; d < L.dim; ++d) x[d] = (int)((k >> L.shift[d]) & ((1ull << L.bits[d]) - 1));
  b = (int)(k >> L.batch_shift);
}

// ---- site hash ----------------------------------------------------------------------------
//
// Open addressing over 32-byte buckets of two 16-byte slots, so one probe is one aligned
// 32-byte sector: both slots of a bucket arrive with two 128-bit loads of the same sector.
// Inserts claim the first free slot of the home bucket, then walk to the next bucket.
// Nothing is ever deleted, so a lookup can stop at the first bucket with a free slot.

struct __align__(16) Slot {
  unsigned long long key;  // kEmptyKey when free
  int row;                 // feature-row index of the site (-1 until numbered)
  unsigned aux;            // build-time scratch: smallest id that touched the site
};

struct HashTable {
  Slot *slots;            // 2 * n_buckets slots
  unsigned long long n_buckets;  // power of two
};

__host__ __device__ inline unsigned long long mix64(unsigned long long k) {
  k ^= k >> 33;
  k *= 0xff51afd7ed558ccdull;
  k ^= k >> 33;
  k *= 0xc4ceb9fe1a85ec53ull;
  k ^= k >> 33;
  return k;
}

#ifdef __CUDACC__
// Returns the slot index holding `key` (inserting it if absent) or -1 if the bounded walk
// gave up.
__device__ inline long long hash_insert(const HashTable &T, unsigned long long key) {
  unsigned long long mask = T.n_buckets - 1;
  unsigned long long b = mix64(key) & mask;
  unsigned long long limit = T.n_buckets < 4096 ? T.n_buckets : 4096;
  for (unsigned long long p = 0; p < limit; ++p) {
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      unsigned long long idx = 2 * b + s;
      unsigned long long prev = atomicCAS(&T.slots[idx].key, kEmptyKey, key);
      if (prev == kEmptyKey || prev == key) return (long long)idx;
    }
    b = (b + 1) & mask;
  }
  return -1;
}

// Returns the slot index of `key` or -1 when absent.  Read-only tables only.
__device__ inline long long hash_find_slot(const HashTable &T, unsigned long long key) {
  unsigned long long mask = T.n_buckets - 1;
  unsigned long long b = mix64(key) & mask;
  unsigned long long limit = T.n_buckets < 4096 ? T.n_buckets : 4096;
  for (unsigned long long p = 0; p < limit; ++p) {
    const uint4 *q = reinterpret_cast<const uint4 *>(T.slots + 2 * b);
    uint4 s0 = __ldg(q);
    uint4 s1 = __ldg(q + 1);
    unsigned long long k0 = ((unsigned long long)s0.y << 32) | s0.x;
    unsigned long long k1 = ((unsigned long long)s1.y << 32) | s1.x;
    if (k0 == key) return (long long)(2 * b);
    if (k1 == key) return (long long)(2 * b + 1);
    if (k0 == kEmptyKey || k1 == kEmptyKey) return -1;
    b = (b + 1) & mask;
  }
  return -1;
}

// Returns the feature row of `key` or -1 when absent.
__device__ inline int hash_find_row(const HashTable &T, unsigned long long key) {
  unsigned long long mask = T.n_buckets - 1;
  unsigned long long b = mix64(key) & mask;
  unsigned long long limit = T.n_buckets < 4096 ? T.n_buckets : 4096;
  for (unsigned long long p = 0; p < limit; ++p) {
    const uint4 *q = reinterpret_cast<const uint4 *>(T.slots + 2 * b);
    uint4 s0 = __ldg(q);
    uint4 s1 = __ldg(q + 1);
    unsigned long long k0 = ((unsigned long long)s0.y << 32) | s0.x;
    unsigned long long k1 = ((unsigned long long)s1.y << 32) | s1.x;
    if (k0 == key) return (int)s0.z;
    if (k1 == key) return (int)s1.z;
    if (k0 == kEmptyKey || k1 == kEmptyKey) return -1;
    b = (b + 1) & mask;
  }
  return -1;
}
#endif  // __CUDACC__

// ---- small host helpers -------------------------------------------------------------------

inline unsigned long long next_pow2(unsigned long long v) {
  unsigned long long p = 1;
  while (p < v) p <<= 1;
  return p;
}
inline int bit_length(unsigned long long v) {
  int n = 0;
  while (v) {
    ++n;
    v >>= 1;
  }
  return n;
}
inline long long ceil_div(long long a, long long b) { return (a + b - 1) / b; }

// Stream-ordered device allocation (cudaMallocAsync on the current device's default pool,
// whose release threshold is raised once so freed blocks are reused instead of returned).
int device_alloc(void **p, size_t bytes, cudaStream_t stream);
int device_free(void *p, cudaStream_t stream);

// Exclusive prefix sum of n int32 values (out may alias in).  total_dev (may be null)
// receives the sum of all inputs as int32.
int exclusive_scan_i32(const int *in, int *out, long long n, int *total_dev, cudaStream_t stream,
                       int *scratch = nullptr);
size_t exclusive_scan_scratch_ints(long long n);  // ints of caller-owned scratch that make the scan allocation-free

}  // namespace scn
