// The TMA-staged batched GEMM kernel for Q4_K weights (see gemm_tma.cu for the design and
// gemm_tma_kernel.cuh for the code): this file only instantiates and launches it.
#include "gemm_tma_kernel.cuh"

namespace kanso {

int32_t tm_launch_q4_k(kanso_cuda_ctx* ctx, dim3 grid, size_t smem, const CUtensorMap& tmap,
                       const TmArgs& a) {
  return tm_launch<TM_FMT_Q4_K>(ctx, grid, smem, tmap, a);
}

}  // namespace kanso
