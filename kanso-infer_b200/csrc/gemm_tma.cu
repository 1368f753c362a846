// Batched quantized GEMM with TMA-staged weight tiles (cp.async.bulk.tensor) feeding
// tcgen05 / TMEM: LinearWeight::forward for continuous-batching and chunked-prefill rows
// (src/weights.rs:43-45; callers src/model.rs:390-421,1418-1740), up to 512 activation rows in
// ONE pass over the weights.
//
//   y[M,N] = x[M,K] @ W[N,K]^T,  W in GGUF Q8_0 / Q4_K blocks, x and y f32.
//
// The contraction runs over the BYTE STREAM of a weight row, not over k. A CTA owns 128 weight
// rows; one elected thread pulls boxes of 128 rows x 128 bytes of the block matrix
// [N][row_bytes] into a ring of shared-memory slots with 2-D tensor-map copies (128-byte
// swizzle, so that 16-byte reads with one lane per row are free of bank conflicts; rows and
// bytes past the matrix are zero-filled by the copy engine). A box does not line up with the
// 34-byte (Q8_0) or 144-byte (Q4_K) blocks and it does not have to: the sum over k may be taken
// in any order as long as both operands agree, so every 16-byte chunk of the stream becomes MMA
// k-positions in the order its bytes lie in memory, and a small pack kernel lays the
// activations out in that same order (zero at the positions of scale bytes and headers):
//   * Q8_0: one chunk = 16 positions = one k-step; a position that holds a byte of a block's
//     f16 scale is multiplied by a zero on the activation side. No realignment of the 2-byte-
//     aligned int8 runs is ever done.
//   * Q4_K: one nibble chunk = 16 low nibbles + 16 high nibbles = two k-steps (sub-blocks 2g
//     and 2g+1 of the chunk's 64-weight group); header chunks produce nothing and are skipped
//     by the MMA issuer.
// 16 producer warps (thread = weight row x 32 stream bytes) read the raw chunks, dequantise with
// packed f16 arithmetic (Q8_0: exact int8 -> f16 by byte permute, one rounding in d*q; Q4_K:
// d*sc*(q-8) - (dmin*m - 8*d*sc) with both factors rounded once to f16) and store 16-byte
// core-matrix rows of the A tile (K-major, no swizzle). Where a block's scale or header falls
// inside a thread's bytes repeats with a short period (17 positions for Q8_0, 9 for Q4_K), so the
// dequantising code exists once per position, with every selection resolved at compile time, and
// a switch picks the body. One warp issues tcgen05.mma
// (kind::f16, M = 128 weight rows, N = up to 256 activation rows per instruction, f32
// accumulation in up to 512 TMEM columns); one warp streams the packed activations through a
// ring of bulk copies. All hand-offs are mbarriers with bounded waits: a wait that runs out sets
// the status word, the CTA drains its own copies, frees its TMEM and returns.
//
// Numerics: both operands are rounded once to f16 (as the f16 tensor path prescribes); the
// products are exact and accumulate in f32. The error of a K = 4096 product is about 1e-4 of
// the output scale against the 1e-3 bound. The decode step's chain of matmuls keeps the
// three-product kernel in gemm_tc.cu.
#include "gemm_tma_kernel.cuh"

namespace kanso {

template <int FMT>
__global__ void tm_pack_kernel(const float* __restrict__ x, __half* __restrict__ bp, int M, int Mt,
                               int K, int units_total, const TmZero zero) {
  pdl_launch_dependents();
  pdl_wait();  // x (and the readers of the buffer cleared here) belong to earlier kernels
  const int64_t gtid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  for (int64_t j = gtid; j < zero.n; j += nthreads) zero.p[j] = 0.f;
  const int64_t total = (int64_t)units_total * 2 * Mt;
  for (int64_t i = gtid; i < total; i += nthreads) {
    const int m = (int)(i % Mt);
    const int uk = (int)(i / Mt);  // unit * 2 + k-chunk
    const int u = uk >> 1, kc8 = uk & 1;
    __align__(16) __half v[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      int k;
      if (FMT == TM_FMT_Q8_0)
        k = tm_k_of_q8_0(u, 8 * kc8 + e);
      else
        k = tm_k_of_q4_k(u >> 1, u & 1, 8 * kc8 + e);
      const float f = (m < M && k >= 0 && k < K) ? x[(int64_t)m * K + k] : 0.f;
      v[e] = __float2half_rn(f);
    }
    *reinterpret_cast<uint4*>(bp + i * 8) = *reinterpret_cast<const uint4*>(v);
  }
}

// cuTensorMapEncodeTiled, looked up once through the runtime (no link-time dependency on the
// driver library).
typedef CUresult (*TmEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                               const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                               const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static TmEncodeFn tm_encoder() {
  static std::once_flag once;
  static TmEncodeFn fn = nullptr;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<TmEncodeFn>(p);
    else
      cudaGetLastError();
  });
  return fn;
}

// The tensor map of a block matrix [N][row_bytes] read in boxes of 128 rows x 128 bytes with
// the 128-byte swizzle (shared with the int8 GEMM). KANSO_ERR_UNSUPPORTED: no encoder.
int32_t tma_encode_weight_map(const void* w, int64_t row_bytes, int64_t N, CUtensorMap* map) {
  TmEncodeFn encode = tm_encoder();
  if (!encode) return KANSO_ERR_UNSUPPORTED;
  const cuuint64_t gdim[2] = {(cuuint64_t)row_bytes, (cuuint64_t)N};
  const cuuint64_t gstride[1] = {(cuuint64_t)row_bytes};
  const cuuint32_t box[2] = {TM_BOX_W, TM_TILE_N};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult cr = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(w), gdim,
                             gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return cr == CUDA_SUCCESS ? KANSO_OK : KANSO_ERR_DEVICE;
}

// y[M,N] = x[M,K] @ W^T for 9..512 activation rows (Q8_0: 2..512). Sets *handled = false (and launches
// nothing) when the shape is outside this kernel's range: rows of the block matrix must start
// on 16-byte boundaries (every Q4_K matrix; Q8_0 when K % 256 == 0).
int32_t tma_matmul(kanso_cuda_ctx* ctx, int32_t dtype, const void* w, const float* x, float* y,
                   int64_t M, int64_t N, int64_t K, bool* handled) {
  *handled = false;
  if (dtype != KANSO_DTYPE_Q8_0 && dtype != KANSO_DTYPE_Q4_K) return KANSO_OK;
  const int blk = dtype == KANSO_DTYPE_Q8_0 ? 32 : 256;
  const int bb = dtype == KANSO_DTYPE_Q8_0 ? Q8_BYTES : Q4K_BYTES;
  const int64_t min_m = dtype == KANSO_DTYPE_Q8_0 ? 2 : 9;  // below: the GEMV kernels are faster
  if (M < min_m || M > TM_MAX_M || N < 1 || K < blk || K % blk != 0 || !w || !x || !y)
    return KANSO_OK;
  const int64_t row_bytes = K / blk * bb;
  if (row_bytes % 16 != 0 || !aligned16(w) || row_bytes > (1 << 28) || N > (1 << 30))
    return KANSO_OK;
  TmEncodeFn encode = tm_encoder();
  if (!encode) return KANSO_OK;

  const int Mt = (int)((M + 15) / 16 * 16);
  const int boxes_total = (int)((row_bytes + TM_BOX_W - 1) / TM_BOX_W);
  const int upc = dtype == KANSO_DTYPE_Q8_0 ? 1 : 2;
  const int units_total = boxes_total * 8 * upc;
  const int tiles_n = (int)((N + TM_TILE_N - 1) / TM_TILE_N);
  // Split the stream while the grid stays within about one wave of CTAs (one CTA per SM) and
  // every CTA keeps at least four boxes; the partial sums of a split are added with atomics
  // onto a y that the pack kernel clears.
  int ksplit = 1;
  while (tiles_n * ksplit * 2 <= ctx->sm_count + ctx->sm_count / 4 &&
         boxes_total / (ksplit * 2) >= 4)
    ksplit *= 2;
  // activation units per ring slot: a whole stage (8 k-steps) when that stays at or below
  // 16 KB, else the largest power-of-two share of it that does
  int ub = 1;
  while (ub * 2 <= 8 && ub * 2 * 32 * Mt <= 16384) ub *= 2;

  CUtensorMap tmap;
  const cuuint64_t gdim[2] = {(cuuint64_t)row_bytes, (cuuint64_t)N};
  const cuuint64_t gstride[1] = {(cuuint64_t)row_bytes};
  const cuuint32_t box[2] = {TM_BOX_W, TM_TILE_N};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult cr = encode(&tmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(w), gdim,
                             gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (cr != CUDA_SUCCESS)
    return fail(ctx, KANSO_ERR_DEVICE, "gemm_tma: cuTensorMapEncodeTiled failed (%d)", (int)cr);

  const size_t bp_bytes = (size_t)units_total * 32 * Mt;
  uint8_t* scratch = (uint8_t*)ctx_scratch(ctx, bp_bytes + 256);
  if (!scratch) return KANSO_ERR_DEVICE;
  *handled = true;

  TmZero zero = {nullptr, 0};
  if (ksplit > 1) {
    zero.p = y;
    zero.n = M * N;
  }
  const int64_t pack_items = (int64_t)units_total * 2 * Mt;
  int64_t pack_blocks = (pack_items + 255) / 256;
  if (pack_blocks > 8 * ctx->sm_count) pack_blocks = 8 * ctx->sm_count;
  cudaError_t le;
  if (dtype == KANSO_DTYPE_Q8_0)
    le = launch_dependent(ctx, tm_pack_kernel<TM_FMT_Q8_0>, dim3((unsigned)pack_blocks), dim3(256),
                          0, x, reinterpret_cast<__half*>(scratch), (int)M, Mt, (int)K,
                          units_total, zero);
  else
    le = launch_dependent(ctx, tm_pack_kernel<TM_FMT_Q4_K>, dim3((unsigned)pack_blocks), dim3(256),
                          0, x, reinterpret_cast<__half*>(scratch), (int)M, Mt, (int)K,
                          units_total, zero);
  if (le != cudaSuccess) return cuda_fail(ctx, le, "gemm_tma pack launch");
  int32_t st = after_launch(ctx, "gemm_tma pack activations");
  if (st) return st;

  TmArgs a;
  a.y = y;
  a.bp = scratch;
  a.N = N;
  a.M = (int)M;
  a.Mt = Mt;
  a.row_bytes = (int)row_bytes;
  a.boxes_total = boxes_total;
  a.ksplit = ksplit;
  a.ub = ub;
  a.status = ctx->dev_status;
  const size_t smem = (size_t)TM_RAW_SLOTS * TM_BOX + (size_t)TM_A_STAGES * TM_A_STAGE +
                      (size_t)TM_B_SLOTS * ub * 32 * Mt + 256;
  if (smem > (size_t)ctx->smem_optin)
    return fail(ctx, KANSO_ERR_UNSUPPORTED, "gemm_tma: %zu bytes of shared memory needed", smem);
  const dim3 grid(tiles_n, ksplit);
  return dtype == KANSO_DTYPE_Q8_0 ? tm_launch_q8_0(ctx, grid, smem, tmap, a)
                                   : tm_launch_q4_k(ctx, grid, smem, tmap, a);
}

}  // namespace kanso
