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
#include "tgemm_tf32.cuh"

namespace b200q {
namespace sweep {

constexpr int kMaxBlock = 128;
constexpr int kWarps = 16;

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
  __shared__ float s_rd[kMaxBlock];   // 1 / U[i][i]
  __shared__ int s_grp[kMaxBlock];    // parameter column (group / block column) of each column
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bs = p.bs;
  for (int idx = threadIdx.x; idx < bs * kMaxBlock; idx += blockDim.x) {
    int r = idx / kMaxBlock, c = idx - r * kMaxBlock;
    float v = 0.0f;
    if (c < bs) v = p.U ? p.U[(int64_t)(p.i1 + r) * p.ldu + (p.i1 + c)] : (r == c ? 1.0f : 0.0f);
    sU[r * LD + c] = v;
  }
  for (int i = threadIdx.x; i < bs; i += blockDim.x) {
    const float d = p.U ? p.U[(int64_t)(p.i1 + i) * p.ldu + (p.i1 + i)] : 1.0f;
    s_rd[i] = __frcp_rn(d);
    const int col = p.i1 + i;
    s_grp[i] = (p.strategy == B200Q_TENSOR || p.strategy == B200Q_CHANNEL)
                   ? 0 : (p.col_group ? p.col_group[col] : col / p.group_size);
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
    // base index of this row's parameters; the column's group is added per column
    int64_t pbase;
    switch (p.strategy) {
      case B200Q_TENSOR: pbase = 0; break;
      case B200Q_CHANNEL: pbase = row; break;
      case B200Q_BLOCK: pbase = (row / p.block_h) * p.groups_per_row; break;
      default: pbase = row * p.groups_per_row; break;
    }
    float loss = 0.0f;
    int64_t cur_pi = -1;
    float s = 1.0f, z = 0.0f, rs = 1.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int lim = min(32, bs - 32 * j);
      for (int l = 0; l < lim; ++l) {
        const int i = 32 * j + l;
        const float wi = __shfl_sync(0xffffffffu, w[j], l);
        const int64_t pi = pbase + s_grp[i];
        if (pi != cur_pi) {
          cur_pi = pi;
          s = Elem<SDT>::load((const typename Elem<SDT>::type*)p.scale + pi);
          if (GLOBAL) s = __fdiv_rn(s, g);
          rs = __frcp_rn(s);
          if (has_zp) z = load_zp(p.zp, p.zp_kind, pi);
        }
        // w is float32, so the quantise arithmetic is float32 (quant_code_fast gives the same code
        // as the true division); only the dequantised value takes the scale's dtype
        float q = quant_code_fast<false>(wi, s, rs, z, p.qr);
        q = dequant_code<SB>(q, s, z);
        const float diff = __fsub_rn(wi, q);
        const float rd = s_rd[i];
        // loss and error use the reciprocal of the pivot (an ulp from the reference's divisions)
        const float t = __fmul_rn(diff, rd);
        loss = fmaf(t, t, loss);
        const float e = t;
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
  if (N <= 0 || K <= 0 || blocksize <= 0) return 0;
  // error panel [N][128] + hi/lo copies of it + hi/lo copies of a 128-row panel of U
  const size_t np = (size_t)((N + 127) / 128 * 128), kp = (size_t)((K + 127) / 128 * 128);
  return (np * 128 * 3 + 2 * 128 * kp) * sizeof(float) + 64;
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
  p.lde = 128;
  const size_t np128 = (size_t)((N + 127) / 128 * 128) * 128, kp128 = (size_t)((K + 127) / 128 * 128) * 128;
  float* sa_hi = p.err + np128;
  float* sa_lo = sa_hi + np128;
  float* sb_hi = sa_lo + np128;
  float* sb_lo = sb_hi + kp128;
  int* gemm_status = nullptr;
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
      // W[:, i2:] -= Err[N, bs] * U[i1:i2, i2:]   (3xTF32 on the tensor cores)
      const int rest = (int)(K - i2);
      rc = tgemm::split(p.err, p.lde, (int)N, bs, sa_hi, sa_lo, st); if (rc) return rc;
      rc = tgemm::split_transposed(U + i1 * ldu + i2, ldu, bs, rest, sb_hi, sb_lo, st); if (rc) return rc;
      rc = tgemm::launch(tgemm::kNT, tgemm::Split{sa_hi, sa_lo, tgemm::split_ld(bs)},
                         tgemm::Split{sb_hi, sb_lo, tgemm::split_ld(bs)}, Wf + i2, ldf, (int)N, rest, bs, -1.0f,
                         1.0f, tgemm::kAllTiles, gemm_status, st);
      if (rc) return rc;
    }
  }
  return B200Q_OK;
}

}  // extern "C"
