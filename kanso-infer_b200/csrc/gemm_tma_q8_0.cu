// The TMA-staged batched GEMM kernel for Q8_0 weights (see gemm_tma.cu for the design and
// gemm_tma_kernel.cuh for the code): this file only instantiates and launches it.
#include "gemm_tma_kernel.cuh"

namespace kanso {

int32_t tm_launch_q8_0(kanso_cuda_ctx* ctx, dim3 grid, size_t smem, const CUtensorMap& tmap,
                       const TmArgs& a) {
  return tm_launch<TM_FMT_Q8_0>(ctx, grid, smem, tmap, a);
}

}  // namespace kanso
