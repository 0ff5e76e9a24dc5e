// tt.dot path: placeholder until the tcgen05 kernel lands.
#include "tsb_common.cuh"
using namespace tsb;
extern "C" int tsb_gemm(const void *a, const void *b, void *c, int32_t dtype, int64_t M, int64_t N, int64_t K,
             int64_t stride_am, int64_t stride_ak, int64_t stride_bk, int64_t stride_bn,
             int64_t stride_cm, int64_t stride_cn, int32_t block_m, int32_t block_n,
             int32_t block_k, const int32_t *tile_of_pid, int64_t n_programs, int64_t pid_lo,
             int64_t pid_hi, int32_t *status, void *stream) {
  return fail(TSB_ERR_UNSUPPORTED, "tsb_gemm: not built yet");
}
