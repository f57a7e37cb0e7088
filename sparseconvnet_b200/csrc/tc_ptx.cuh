// Inline-PTX wrappers shared by the tensor-core convolution kernels: mbarriers with bounded
// waits, cp.async, bulk (TMA) copies, tcgen05 allocation / MMA / commit / load, and the
// shared-memory matrix descriptors.
#pragma once

#include <cuda_bf16.h>

#include "common.cuh"

namespace scn {

constexpr unsigned kWaitLimit = 1u << 20;  // polls before a bounded wait gives up

// TC_TF32X3 and TC_BF16X3 are the two forms of the fp32-class mode: x = hi + lo with hi the tf32
// truncation (three tf32 products, or one tf32 and two bf16 ones), or x = h + m with h = bf16(x),
// m = bf16(x - h) and the three bf16 products h h, m h, h m (what is left out is 2^-17 of a product).
enum TcMode : int { TC_TF32 = 0, TC_BF16 = 1, TC_TF32X3 = 2, TC_BF16X3 = 3 };

// Which form SCN_PRECISION_TF32X3 runs in a kernel whose default is `dflt`: SCN_X3_FORM=tf32 / bf16
// forces one form everywhere (for measurements and the parity tests of both).
int split_mode_of_env(int dflt = TC_BF16X3);

// W [K][Cin][Cout] fp32 -> per (offset, slice of kc input planes) the shared-memory image of the
// weight operand (conv_tc.cu)
int prepare_weights(const float *w, unsigned char *out, int K, int cin, int cout, int kc, int mode,
                    cudaStream_t stream);

// Prepared weight images (the operand layouts the kernels read) are small and depend only on the
// weights, so a caller whose weights do not change between calls can have them kept: while the calling
// thread has a non-zero weight token set (scn_set_weight_token), an image is looked up under
// (device, token, layout, shape) and built only when it is not there; with token 0 it is scratch of the
// call.  `needs_build` says whether the caller has to launch its preparation kernel.
enum WeightImageKind : int { WIMG_ROWS = 1, WIMG_ROWS_B3, WIMG_ROWS_THIN, WIMG_TC };
struct WeightImage {
  void *ptr = nullptr;
  bool cached = false;
};
int weight_image_get(int kind, int K, int cin, int cout, int extra, size_t bytes, cudaStream_t stream,
                     WeightImage *img, bool *needs_build);
int weight_image_put(WeightImage &img, cudaStream_t stream);  // frees a scratch image, keeps a cached one

// ---------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ unsigned smem_u32(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned long long *bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
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
// 32 lanes x 32 consecutive 32-bit columns.
__device__ __forceinline__ void tmem_ld32(unsigned taddr, float *v) {
  unsigned r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// Two floats as a bf16 pair rounded to nearest (`a` in the low half) and the pair of what the
// rounding left over, again as bf16: the two parts of the three-term bf16 split.
__device__ __forceinline__ void split_bf16_pair(float a, float b, unsigned &h, unsigned &m) {
  __nv_bfloat162 hv = __floats2bfloat162_rn(a, b);
  h = *reinterpret_cast<unsigned *>(&hv);
  __nv_bfloat162 mv = __floats2bfloat162_rn(a - __uint_as_float(h << 16), b - __uint_as_float(h & 0xFFFF0000u));
  m = *reinterpret_cast<unsigned *>(&mv);
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
}  // namespace scn
