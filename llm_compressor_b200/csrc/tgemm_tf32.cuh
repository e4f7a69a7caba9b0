// Interface of the float32-accurate tensor-core GEMM (implementation: tgemm_tf32.cu).
#pragma once

#include "common.cuh"

#include <cuda_runtime.h>

namespace b200q {
namespace tgemm {

enum Trans { kNN = 0, kNT = 1 };
// kSkipBlockTiles (argument kb): C spans all columns of a matrix whose row 0 is the first row below
// block row kb; tiles in column blocks < kb are all computed, column block kb is skipped, and
// column blocks > kb only on and below the diagonal of the matrix (tile (tm, kb + 1 + j), j <= tm).
// kSkipBlockFirst / kSkipBlockRest split the kSkipBlockTiles set in two: First = row block 0 and
// column block kb + 1 (what the next step of a right-looking factorisation reads), Rest = the
// other tiles (which can run beside that next step).
enum TileMask { kAllTiles = 0, kLowerTiles = 1, kSkipBlockTiles = 2, kSkipBlockFirst = 3, kSkipBlockRest = 4 };

struct Split {       // a split operand: hi / lo arrays with a common leading dimension
  const float* hi;
  const float* lo;
  int64_t ld;
};

inline int64_t split_ld(int64_t cols) { return (cols + 31) / 32 * 32; }

// One half of an operand split: x rounded to nearest even on 10 mantissa bits, as a float32 word
// whose low 13 mantissa bits are zero.  hi = tf32_rn(x), lo = tf32_rn(x - hi).
__device__ __forceinline__ float tf32_rn(float x) {
  uint32_t b = __float_as_uint(x);
  b = (b + 0xFFFu + ((b >> 13) & 1u)) & 0xFFFFE000u;
  return __uint_as_float(b);
}

// src [rows][cols] -> hi/lo [rows][split_ld(cols)]
int split(const float* src, int64_t ld_src, int rows, int cols, float* hi, float* lo, cudaStream_t st);
// src [rows][cols] -> hi/lo [cols][split_ld(rows)]
int split_transposed(const float* src, int64_t ld_src, int rows, int cols, float* hi, float* lo, cudaStream_t st);
// C[M,N] = beta*C + alpha * A[M,Kd] * B[N,Kd]^T with A, B given as hi/lo splits whose buffers hold
// whole 128-row tiles (rows beyond M / N may hold anything).
int launch(int trans, Split A, Split B, float* C, int64_t ldc, int M, int N, int Kd, float alpha, float beta,
           int mask, int* status, cudaStream_t st, int mask_arg = 0, int max_ctas = 0);
// CTAs a bulk update leaves free for the look-ahead work that runs beside it
int side_reserve();

// A helper stream of the calling host thread (same priority as `like`), with two events, for the
// look-ahead of the blocked solves: the bulk of a rank-128 update runs there while the caller's
// stream goes on with the next block.  Created once per device and caller stream; null on failure.
struct SideStream {
  cudaStream_t stream = nullptr;
  cudaEvent_t ready = nullptr;   // recorded on the caller's stream: operands of the bulk update exist
  cudaEvent_t done = nullptr;    // recorded on the helper: bulk update finished
};
SideStream* side_stream(cudaStream_t like);

}  // namespace tgemm
}  // namespace b200q
