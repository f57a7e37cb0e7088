// Self-calibration of the tensor path: how many SM cycles one tcgen05.mma of a given shape costs
// when many of them are issued back to back.  The kernel choice in conv_api.cu (dense 256-row
// tiles against per-group issue) rests on how that cost falls with N, so the figure is measured
// by the library itself instead of being assumed.
//
// One CTA per requested SM; thread 0 issues `n_mma` instructions round-robin onto disjoint TMEM
// column ranges (no instruction waits for the accumulator of the previous one), one commit at the
// end, one bounded wait.  The operands are zero-filled shared memory (or TMEM columns for the A
// operand): the tensor pipe's timing does not depend on the values.
#include "tc_ptx.cuh"

namespace scn {
namespace {

template <bool BF16>
__device__ __forceinline__ void tc_mma_a_tmem(unsigned d_tmem, unsigned a_tmem, unsigned long long b_desc,
                                              unsigned idesc, unsigned accumulate) {
  if (BF16)
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  else
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// acc_cols: TMEM columns per accumulator range (>= N, power of two); n_acc ranges (power of two).
template <bool BF16, bool A_TMEM>
__global__ void __launch_bounds__(128) k_tc_probe(int M, int N, int n_acc, int n_mma, long long *out, int *err) {
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ unsigned long long bar;
  __shared__ unsigned tmem;
  // 16 KB A image + 32 KB B image, zero filled
  for (int i = threadIdx.x; i < 48 * 1024 / 16; i += blockDim.x) reinterpret_cast<uint4 *>(smem)[i] = make_uint4(0, 0, 0, 0);
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (threadIdx.x < 32) tmem_alloc(&tmem, 512);
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned base = tmem;
  if (threadIdx.x == 0) {
    const unsigned fmt = BF16 ? 1u : 2u;
    const unsigned idesc =
        (1u << 4) | (fmt << 7) | (fmt << 10) | ((unsigned)(N >> 3) << 17) | ((unsigned)(M >> 4) << 24);
    const unsigned a_addr = smem_u32(smem), b_addr = a_addr + 16384;
    // K-major, no swizzle, 8 x 16-byte core matrices; one instruction reads two core matrices along K
    unsigned long long da[4], db[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      da[j] = smem_desc(a_addr + j * 256, 128, 1024);
      db[j] = smem_desc(b_addr + j * 256, 128, 1024);
    }
    // accumulators from column 0; the A operand, when it lives in TMEM, in the last 32 columns
    const unsigned a_tmem = base + 480;
    const int acc_mask = n_acc - 1;
    const long long t0 = clock64();
#pragma unroll 4
    for (int i = 0; i < n_mma; ++i) {
      const unsigned d = base + (unsigned)((i & acc_mask) * N);
      const unsigned accumulate = i >= n_acc ? 1u : 0u;
      if (A_TMEM)
        tc_mma_a_tmem<BF16>(d, a_tmem + (i & 3) * 8, db[i & 3], idesc, accumulate);
      else
        tc_mma<BF16>(d, da[i & 3], db[i & 3], idesc, accumulate);
    }
    tc_commit(&bar);
    const long long t1 = clock64();
    const bool ok = mbar_wait(&bar, 0);
    const long long t2 = clock64();
    out[2 * blockIdx.x] = t1 - t0;
    out[2 * blockIdx.x + 1] = t2 - t0;
    if (!ok) atomicOr(err, FLAG_TC_TIMEOUT);
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) tmem_dealloc(base, 512);
}

}  // namespace
}  // namespace scn

using namespace scn;

extern "C" int scn_tc_probe_mma(int m, int n, int kind_bf16, int a_in_tmem, int n_mma, int n_ctas, void *stream_,
                                double *cycles_issue, double *cycles_total, double *event_ms) {
  cudaStream_t stream = (cudaStream_t)stream_;
  SCN_REQUIRE(m == 64 || m == 128, SCN_ERR_BAD_ARG, "M must be 64 or 128, got %d", m);
  SCN_REQUIRE(n >= (m == 128 ? 16 : 8) && n <= 256 && n % (m == 128 ? 16 : 8) == 0, SCN_ERR_BAD_ARG,
              "N = %d is not a legal width for M = %d", n, m);
  SCN_REQUIRE(n_mma >= 1 && n_mma <= (1 << 20) && n_ctas >= 1 && n_ctas <= 1024, SCN_ERR_BAD_ARG,
              "bad instruction or CTA count");
  SCN_REQUIRE(cycles_issue && cycles_total && event_ms, SCN_ERR_BAD_ARG, "null result pointer");
  SCN_REQUIRE(!a_in_tmem || m == 128, SCN_ERR_BAD_ARG, "the A-in-TMEM form is probed for M = 128 only");
  int n_acc = 1;  // as many disjoint accumulator ranges as fit 448 columns, at most 8
  while (n_acc < 8 && 2 * n_acc * n <= 448) n_acc *= 2;
  long long *out = nullptr;
  int *err = nullptr;
  SCN_CUDA_CHECK(cudaMalloc((void **)&out, sizeof(long long) * 2 * n_ctas + sizeof(int)));
  err = (int *)(out + 2 * n_ctas);
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  int status = SCN_OK;
  std::string msg;
  auto fail = [&](cudaError_t e, const char *what) {
    if (e != cudaSuccess && status == SCN_OK) {
      status = SCN_ERR_CUDA;
      msg = std::string(what) + ": " + cudaGetErrorString(e);
    }
  };
  fail(cudaMemsetAsync(out, 0, sizeof(long long) * 2 * n_ctas + sizeof(int), stream), "memset");
  fail(cudaEventCreate(&e0), "event");
  fail(cudaEventCreate(&e1), "event");
  const int smem = 48 * 1024 + 1024;
  auto launch = [&]() {
    note_launch();
    if (kind_bf16 && a_in_tmem)
      k_tc_probe<true, true><<<n_ctas, 128, smem, stream>>>(m, n, n_acc, n_mma, out, err);
    else if (kind_bf16)
      k_tc_probe<true, false><<<n_ctas, 128, smem, stream>>>(m, n, n_acc, n_mma, out, err);
    else if (a_in_tmem)
      k_tc_probe<false, true><<<n_ctas, 128, smem, stream>>>(m, n, n_acc, n_mma, out, err);
    else
      k_tc_probe<false, false><<<n_ctas, 128, smem, stream>>>(m, n, n_acc, n_mma, out, err);
  };
  if (status == SCN_OK) {
    fail(cudaFuncSetAttribute(k_tc_probe<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem), "attr");
    fail(cudaFuncSetAttribute(k_tc_probe<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem), "attr");
    fail(cudaFuncSetAttribute(k_tc_probe<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem), "attr");
    fail(cudaFuncSetAttribute(k_tc_probe<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem), "attr");
  }
  if (status == SCN_OK) {
    launch();  // warm-up
    fail(cudaEventRecord(e0, stream), "record");
    launch();
    fail(cudaEventRecord(e1, stream), "record");
    fail(cudaGetLastError(), "launch");
    fail(cudaEventSynchronize(e1), "synchronize");
  }
  if (status == SCN_OK) {
    std::string host(sizeof(long long) * 2 * n_ctas + sizeof(int), '\0');
    fail(cudaMemcpy(&host[0], out, host.size(), cudaMemcpyDeviceToHost), "copy");
    float ms = 0.f;
    fail(cudaEventElapsedTime(&ms, e0, e1), "elapsed");
    if (status == SCN_OK) {
      const long long *c = (const long long *)host.data();
      double si = 0, st = 0;
      for (int i = 0; i < n_ctas; ++i) {
        si += (double)c[2 * i];
        st += (double)c[2 * i + 1];
      }
      *cycles_issue = si / n_ctas / n_mma;
      *cycles_total = st / n_ctas / n_mma;
      *event_ms = ms;
      int e = *(const int *)(host.data() + sizeof(long long) * 2 * n_ctas);
      if (e) {
        status = SCN_ERR_CUDA;
        msg = "a bounded wait of the probe ran out";
      }
    }
  }
  if (e0) cudaEventDestroy(e0);
  if (e1) cudaEventDestroy(e1);
  cudaFree(out);
  if (status != SCN_OK) set_error("tensor-path probe: %s", msg.c_str());
  return status;
}
