// GPTQ solve, part 2: the blockwise column sweep.
//
// Rows of W are independent, so they are spread over warps: one warp owns one row of the
// current 128-column block, lane l holding columns l, l+32, l+64, l+96 in registers.  The
// 128x128 diagonal block of U sits in shared memory.  Column by column the owning lane's
// value is broadcast by shuffle, every lane computes the same quantised value, and each
// lane applies the rank-1 correction to the columns it holds.  The quantisation error of the
// block goes to a [N,128] scratch panel and the update of all later columns is one fp32
// tile GEMM  W[:, after] -= Err * U[block, after].
//
// Rounding follows the reference's sequence of separate float32 operations (product, then
// subtraction; true divisions), so that the propagated errors agree.
#include "common.cuh"
#include "sgemm.cuh"

namespace b200q {
namespace sweep {

constexpr int kMaxBlock = 128;
constexpr int kWarps = 8;

struct Params {
  float* W; int64_t ldw; int64_t N; int64_t K;
  const float* U; int64_t ldu;
  const void* scale; const void* zp; const int32_t* col_group; const float* gscale;
  int strategy, group_size, block_h, zp_kind;
  int64_t groups_per_row;
  QRange qr;
  float* err; int64_t lde;   // [N, bs]
  float* losses;
  int i1, bs;                // block start and width (<= 128)
  int first;                 // first block: losses are overwritten
};

// SB: scale tensor is bf16 (and no global scale) -> dequantised value rounded to bf16.
template <int SDT, bool GLOBAL>
__global__ void __launch_bounds__(kWarps * 32) sweep_block_kernel(Params p) {
  constexpr bool SB = Elem<SDT>::is_bf16 && !GLOBAL;
  extern __shared__ float sU[];  // [bs][kMaxBlock + 1] row i, local col c; identity when U is null
  constexpr int LD = kMaxBlock + 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bs = p.bs;
  for (int idx = threadIdx.x; idx < bs * kMaxBlock; idx += blockDim.x) {
    int r = idx / kMaxBlock, c = idx - r * kMaxBlock;
    float v = 0.0f;
    if (c < bs) v = p.U ? p.U[(int64_t)(p.i1 + r) * p.ldu + (p.i1 + c)] : (r == c ? 1.0f : 0.0f);
    sU[r * LD + c] = v;
  }
  __syncthreads();
  const float g = GLOBAL ? *p.gscale : 1.0f;
  const bool has_zp = p.zp != nullptr;

  for (int64_t row = (int64_t)blockIdx.x * kWarps + warp; row < p.N; row += (int64_t)gridDim.x * kWarps) {
    float w[4], qv[4], ev[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int c = lane + 32 * j;
      w[j] = (c < bs) ? p.W[row * p.ldw + p.i1 + c] : 0.0f;
      qv[j] = 0.0f; ev[j] = 0.0f;
    }
    float loss = 0.0f;
    int64_t cur_pi = -1;
    float s = 1.0f, z = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int lim = min(32, bs - 32 * j);
      for (int l = 0; l < lim; ++l) {
        const int i = 32 * j + l;
        const float wi = __shfl_sync(0xffffffffu, w[j], l);
        // parameters of this column for this row
        int64_t pi;
        const int col = p.i1 + i;
        switch (p.strategy) {
          case B200Q_TENSOR: pi = 0; break;
          case B200Q_CHANNEL: pi = row; break;
          case B200Q_BLOCK: pi = (row / p.block_h) * p.groups_per_row + (p.col_group ? p.col_group[col] : col / p.group_size); break;
          default: pi = row * p.groups_per_row + (p.col_group ? p.col_group[col] : col / p.group_size); break;
        }
        if (pi != cur_pi) {
          cur_pi = pi;
          s = Elem<SDT>::load((const typename Elem<SDT>::type*)p.scale + pi);
          if (GLOBAL) s = __fdiv_rn(s, g);
          if (has_zp) z = load_zp(p.zp, p.zp_kind, pi);
        }
        const float d = sU[i * LD + i];
        // w is float32, so the quantise arithmetic is float32; only the dequantised value takes
        // the scale's dtype
        float q = quant_code<false>(wi, s, z, p.qr);
        q = dequant_code<SB>(q, s, z);
        const float diff = __fsub_rn(wi, q);
        loss += __fdiv_rn(__fmul_rn(diff, diff), __fmul_rn(d, d));
        const float e = __fdiv_rn(diff, d);
        if (lane == l) { qv[j] = q; ev[j] = e; }
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          const int c = lane + 32 * jj;
          if (jj >= j && c >= i && c < bs) w[jj] = __fsub_rn(w[jj], __fmul_rn(e, sU[i * LD + c]));
        }
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int c = lane + 32 * j;
      if (c < bs) {
        p.W[row * p.ldw + p.i1 + c] = qv[j];
        p.err[row * p.lde + c] = ev[j];
      }
    }
    if (lane == 0) {
      const float half = loss * 0.5f;
      p.losses[row] = p.first ? half : p.losses[row] + half;
    }
  }
}

}  // namespace sweep
}  // namespace b200q

using namespace b200q;

extern "C" {

size_t b200q_gptq_sweep_workspace_bytes(int64_t N, int64_t K, int blocksize) {
  (void)K;
  if (N <= 0 || blocksize <= 0) return 0;
  int bs = blocksize < sweep::kMaxBlock ? blocksize : sweep::kMaxBlock;
  return (size_t)N * (size_t)((bs + 3) / 4 * 4) * sizeof(float);
}

int b200q_gptq_sweep(float* Wf, int64_t N, int64_t K, int64_t ldf, const float* U, int64_t ldu, const void* scale,
                     int sdtype, const void* zp, const int32_t* col_group, const float* gscale,
                     const b200q_qargs* qa, int blocksize, float* losses, void* workspace, void* stream) {
  using namespace b200q::sweep;
  if (!Wf || !scale || !qa || !losses || !workspace || N <= 0 || K <= 0 || ldf < K) return B200Q_ERR_ARG;
  if (U && ldu < K) return B200Q_ERR_ARG;
  if (blocksize <= 0 || blocksize > kMaxBlock) return B200Q_ERR_UNSUPPORTED;
  Params p;
  int rc = make_qrange(qa, &p.qr); if (rc) return rc;
  ParamMap pm;
  rc = make_param_map(qa, N, K, col_group, &pm); if (rc) return rc;
  p.W = Wf; p.ldw = ldf; p.N = N; p.K = K; p.U = U; p.ldu = ldu;
  p.scale = scale; p.zp = zp; p.col_group = col_group; p.gscale = gscale;
  p.strategy = qa->strategy;
  p.group_size = (qa->strategy == B200Q_BLOCK) ? qa->block_w : qa->group_size;
  p.block_h = qa->block_h > 0 ? qa->block_h : 1;
  p.zp_kind = qa->zp_kind;
  p.groups_per_row = pm.groups_per_row;
  p.err = (float*)workspace;
  p.lde = (blocksize + 3) / 4 * 4;
  p.losses = losses;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t smem = (size_t)kMaxBlock * (kMaxBlock + 1) * sizeof(float);
  void (*kern)(Params) = nullptr;
  if (sdtype == B200Q_BF16) kern = gscale ? sweep_block_kernel<B200Q_BF16, true> : sweep_block_kernel<B200Q_BF16, false>;
  else if (sdtype == B200Q_F32) kern = gscale ? sweep_block_kernel<B200Q_F32, true> : sweep_block_kernel<B200Q_F32, false>;
  else return B200Q_ERR_UNSUPPORTED;
  B200Q_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const int grid = grid_for((N + kWarps - 1) / kWarps, 3);
  for (int64_t i1 = 0; i1 < K; i1 += blocksize) {
    const int bs = (int)((K - i1) < blocksize ? (K - i1) : blocksize);
    p.i1 = (int)i1; p.bs = bs; p.first = (i1 == 0);
    kern<<<grid, kWarps * 32, smem, st>>>(p);
    B200Q_LAUNCH_CHECK();
    const int64_t i2 = i1 + bs;
    if (i2 < K && U) {
      // W[:, i2:] -= Err[N, bs] * U[i1:i2, i2:]
      B200Q_TRY(sgemm::launch(sgemm::kNN, p.err, p.lde, U + i1 * ldu + i2, ldu, Wf + i2, ldf, (int)N,
                              (int)(K - i2), bs, -1.0f, 1.0f, sgemm::kAllTiles, st));
    }
  }
  return B200Q_OK;
}

}  // extern "C"
