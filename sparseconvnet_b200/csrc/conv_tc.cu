// Tensor-core (tcgen05 / TMEM) convolution path.
#include "metadata.cuh"

namespace scn {

bool conv_tc_supported(int cin, int cout, int groups, int precision) {
  (void)cin; (void)cout; (void)groups; (void)precision;
  return false;
}

int conv_forward_tc(const float *, long long, float *, long long, const float *, const float *,
                    const int *, int, int, int, int, int *, cudaStream_t) {
  set_error("tensor-core convolution path not available");
  return SCN_ERR_UNSUPPORTED;
}

}  // namespace scn
