// GPTQ solve, part 1: act-order permutation, dead columns + dampening, and the factor
// U (upper) with U^T U = (H + damp I)^-1, all on device in fp32.
//
// Factorisation.  Let J be the index reversal.  If J H J = L L^T (ordinary lower Cholesky)
// then H = V V^T with V = J L J upper triangular, hence H^-1 = V^-T V^-1 and the wanted
// factor is U = V^-1 = J L^-1 J (upper, positive diagonal, so it equals the upper Cholesky
// factor of H^-1).  That is one Cholesky and one triangular inverse (2/3 K^3 flops) instead
// of Cholesky, Cholesky-inverse and a second Cholesky (4/3 K^3).
//   1. A = J H J                                   (reverse copy into the workspace)
//   2. one pass over the 128-column blocks does the right-looking Cholesky of A and the
//      forward substitution for X = L^-1 together (see b200q_gptq_factor): the diagonal block is
//      factored and inverted in registers by one CTA, and all rows below it take their updates,
//      of the substitution's accumulators left of the block and of the Schur complement right
//      of it, from one rank-128 tensor-core GEMM launch
//   3. U = J X J written over H, strictly lower part zeroed
// A pivot <= 0 (or NaN) sets *status; the host then takes the reference's identity fallback.
#include "common.cuh"
#include "tgemm_tf32.cuh"

namespace b200q {
namespace solve {

constexpr int NB = 128;

// ---------------------------------------------------------------------------------------
// act-order: stable descending rank by counting.  The comparison runs on an integer key that
// orders every float the way torch.sort does (NaN above +inf, -0 equal to +0), so the ranks are
// a permutation of 0..K-1 whatever the diagonal holds.
__device__ __forceinline__ uint32_t order_key(float d) {
  if (d != d) return 0xFFFFFFFFu;
  const uint32_t b = __float_as_uint(d + 0.0f);   // -0 + 0 = +0
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__global__ void __launch_bounds__(256) perm_kernel(const float* __restrict__ H, int64_t K, int64_t ldh,
                                                   int32_t* __restrict__ perm) {
  __shared__ uint32_t sd[1024];
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const uint32_t ki = (i < K) ? order_key(H[i * ldh + i]) : 0u;
  int rank = 0;
  for (int64_t j0 = 0; j0 < K; j0 += 1024) {
    for (int t = threadIdx.x; t < 1024; t += blockDim.x) {
      int64_t j = j0 + t;
      sd[t] = (j < K) ? order_key(H[j * ldh + j]) : 0u;
    }
    __syncthreads();
    if (i < K) {
      const int lim = (int)min((int64_t)1024, K - j0);
      for (int t = 0; t < lim; ++t) {
        const uint32_t kj = sd[t];
        rank += (kj > ki) || (kj == ki && (j0 + t) < i);
      }
    }
    __syncthreads();
  }
  if (i < K) perm[rank] = (int32_t)i;
}

// column index taken from a caller-supplied permutation, kept inside the matrix
__device__ __forceinline__ int64_t perm_at(const int32_t* __restrict__ perm, int64_t c, int64_t K) {
  const int64_t v = (int64_t)perm[c];
  return v < 0 ? 0 : (v >= K ? K - 1 : v);
}

template <int DT>
__global__ void gather_cols_kernel(const void* __restrict__ W, int64_t N, int64_t K, int64_t ldw,
                                   const int32_t* __restrict__ perm, float* __restrict__ out, int64_t ldo) {
  using E = Elem<DT>;
  const int64_t total = N * K;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    int64_t r = i / K, c = i - r * K;
    int64_t src = perm ? perm_at(perm, c, K) : c;
    out[r * ldo + c] = E::load((const typename E::type*)W + r * ldw + src);
  }
}

// Batched forms for many weights of one shape (device arrays of pointers, blockIdx.y = problem):
// the gather also zeroes the columns whose Hessian diagonal entry (after the permutation) is zero.
template <int DT>
__global__ void gather_cols_batched_kernel(const void* const* __restrict__ W, int64_t N, int64_t K, int64_t ldw,
                                           const int32_t* const* __restrict__ perm,
                                           const float* const* __restrict__ diag, float* const* __restrict__ out,
                                           int64_t ldo) {
  using E = Elem<DT>;
  const int j = blockIdx.y;
  const typename E::type* w = (const typename E::type*)W[j];
  const int32_t* pm = perm ? perm[j] : nullptr;
  const float* dg = diag ? diag[j] : nullptr;
  float* o = out[j];
  const int64_t total = N * K;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / K, c = i - r * K;
    const int64_t src = pm ? perm_at(pm, c, K) : c;
    const bool dead = dg && dg[c] == 0.0f;
    o[r * ldo + c] = dead ? 0.0f : E::load(w + r * ldw + src);
  }
}

template <int DT>
__global__ void scatter_cols_batched_kernel(const float* const* __restrict__ Wf, int64_t N, int64_t K, int64_t ldf,
                                            const int32_t* const* __restrict__ perm, void* const* __restrict__ out,
                                            int64_t ldo) {
  using E = Elem<DT>;
  const int j = blockIdx.y;
  const float* wf = Wf[j];
  const int32_t* pm = perm ? perm[j] : nullptr;
  typename E::type* o = (typename E::type*)out[j];
  const int64_t total = N * K;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / K, c = i - r * K;
    const int64_t dst = pm ? perm_at(pm, c, K) : c;
    E::store(o + r * ldo + dst, wf[r * ldf + c]);
  }
}

__global__ void permute_hessian_kernel(const float* __restrict__ H, int64_t K, int64_t ldh,
                                       const int32_t* __restrict__ perm, float* __restrict__ out,
                                       int64_t ldo) {
  const int64_t total = K * K;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    int64_t r = i / K, c = i - r * K;
    out[r * ldo + c] = H[perm_at(perm, r, K) * ldh + perm_at(perm, c, K)];
  }
}

template <int DT>
__global__ void scatter_cols_kernel(const float* __restrict__ Wf, int64_t N, int64_t K, int64_t ldf,
                                    const int32_t* __restrict__ perm, void* __restrict__ out, int64_t ldo) {
  using E = Elem<DT>;
  const int64_t total = N * K;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    int64_t r = i / K, c = i - r * K;
    int64_t dst = perm ? perm_at(perm, c, K) : c;
    E::store((typename E::type*)out + r * ldo + dst, Wf[r * ldf + c]);
  }
}

// ---------------------------------------------------------------------------------------
// dead columns and dampening
__global__ void zero_dead_columns_kernel(const float* __restrict__ H, int64_t K, int64_t diag_stride,
                                         float* __restrict__ W, int64_t N, int64_t ldf) {
  // one warp per column; only dead columns touch W
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t c = warp; c < K; c += nwarps) {
    if (H[c * diag_stride] == 0.0f)
      for (int64_t r = lane; r < N; r += 32) W[r * ldf + c] = 0.0f;
  }
}
__global__ void __launch_bounds__(1024) damp_kernel(float* __restrict__ H, int64_t K, int64_t ldh,
                                                    float percdamp) {
  __shared__ float s_part[32];
  __shared__ float s_damp;
  float sum = 0.0f;
  for (int64_t i = threadIdx.x; i < K; i += blockDim.x) {
    float d = H[i * ldh + i];
    if (d == 0.0f) { d = 1.0f; H[i * ldh + i] = 1.0f; }
    sum += d;
  }
  sum = warp_sum(sum);
  if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = sum;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = (threadIdx.x < (blockDim.x >> 5)) ? s_part[threadIdx.x] : 0.0f;
    v = warp_sum(v);
    if (threadIdx.x == 0) s_damp = percdamp * (v / (float)K);
  }
  __syncthreads();
  const float damp = s_damp;
  for (int64_t i = threadIdx.x; i < K; i += blockDim.x) H[i * ldh + i] += damp;
}

// ---------------------------------------------------------------------------------------
// index reversal copies
__global__ void reverse_in_kernel(const float* __restrict__ H, int64_t K, int64_t ldh,
                                  float* __restrict__ A, int64_t lda) {
  const int64_t total = K * K;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    int64_t r = i / K, c = i - r * K;
    A[r * lda + c] = H[(K - 1 - r) * ldh + (K - 1 - c)];
  }
}
__global__ void reverse_out_kernel(const float* __restrict__ A, int64_t K, int64_t lda,
                                   float* __restrict__ U, int64_t ldu) {
  const int64_t total = K * K;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    int64_t r = i / K, c = i - r * K;
    U[r * ldu + c] = (c >= r) ? A[(K - 1 - r) * lda + (K - 1 - c)] : 0.0f;
  }
}

// ---------------------------------------------------------------------------------------
// Diagonal block: Cholesky L of the n x n (n <= 128) block at A[k0,k0]; L^-1 is written both to
// Dinv (128 x 128, zero above the diagonal) and over the block itself (L is not needed again).
//
// The block lives in registers: 256 threads as a 16 x 16 grid, thread (ty,tx) holding the 64
// elements (ty + 16a, tx + 16b).  The cyclic layout keeps every thread busy while the active
// part shrinks.  Right-looking elimination, one barrier per column: the owners of column j
// publish it (unscaled) to shared memory, the owners of row j publish that row of the inverse
// under construction, and every thread then applies the rank-1 update to the rows below j that
// it holds.  Column c of the block is dead once step c has exported it, and column c of the
// inverse is born at step c, so the same register holds first A[i][c] and then Linv[i][c]:
//     c > j:  A[i][c]    -= l_i * l_c            (l = column j / pivot root)
//     c = j:  Linv[i][j]  = -l_i / root          (Linv[j][j] = 1 / root)
//     c < j:  Linv[i][c] -= l_i * Linv[j][c]     (row j of the inverse, scaled by 1 / root)
// The column-block index of j is a compile-time constant inside the unrolled outer loop, which
// keeps every register index static and drops finished register rows at compile time.
constexpr int kDiagThreads = 256;
constexpr int kDiagLD = NB + 1;  // stride of the published columns
constexpr int kDiagSmemFloats = NB * kDiagLD + 2 * NB + NB;

template <int JA>
__device__ __forceinline__ void chol_diag_steps(float (&v)[8][8], float* __restrict__ Lt, float* __restrict__ rowbuf,
                                                float* __restrict__ rinvs, int n, int k0, int* __restrict__ status,
                                                int tx, int ty) {
  for (int jr = 0; jr < 16; ++jr) {
    const int j = JA * 16 + jr;
    if (j >= n) break;   // uniform
    float* col = Lt + j * kDiagLD;
    float* row = rowbuf + (j & 1) * NB;
    if (tx == jr) {
#pragma unroll
      for (int a = JA; a < 8; ++a) {
        const int i = ty + 16 * a;
        if (i >= j) col[i] = v[a][JA];
      }
    }
    if (ty == jr) {
#pragma unroll
      for (int b = 0; b <= JA; ++b) {
        const int c = tx + 16 * b;
        if (c < j) row[c] = v[JA][b];
      }
    }
    __syncthreads();
    float piv = col[j];
    if (!(piv > 0.0f)) {  // also true for NaN
      if (threadIdx.x == 0 && atomicCAS(status, 0, B200Q_NOT_POSITIVE_DEFINITE) == 0) status[1] = k0 + j + 1;
      piv = 1.0f;
    }
    const float rinv = __fdiv_rn(1.0f, sqrtf(piv));
    if (threadIdx.x == 0) rinvs[j] = rinv;
    // multipliers of the columns this thread holds
    float m[8];
#pragma unroll
    for (int b = 0; b < 8; ++b) {
      const int c = tx + 16 * b;
      float x;
      if (b > JA) x = col[c];
      else if (b < JA) x = row[c];
      else x = (tx > jr) ? col[c] : ((tx < jr) ? row[c] : 0.0f);
      m[b] = x * rinv;
    }
#pragma unroll
    for (int a = JA; a < 8; ++a) {
      const int i = ty + 16 * a;
      if (a == JA && ty <= jr) {
        if (ty == jr) {
          // row j of the inverse takes its final value
#pragma unroll
          for (int b = 0; b <= JA; ++b) {
            const int c = tx + 16 * b;
            if (c < j) v[a][b] = m[b];
            else if (c == j) v[a][b] = rinv;
          }
        }
        continue;
      }
      const float li = col[i] * rinv;
#pragma unroll
      for (int b = 0; b < 8; ++b) v[a][b] = fmaf(-li, m[b], v[a][b]);
      if (tx == jr) v[a][JA] = -li * rinv;
    }
  }
}

__global__ void __launch_bounds__(kDiagThreads, 1) chol_diag_kernel(float* __restrict__ A, int64_t lda, int k0, int n,
                                                                    float* __restrict__ Dinv, int* __restrict__ status) {
  extern __shared__ float sm[];
  float* Lt = sm;                      // [NB][kDiagLD]: Lt[j][i] = column j as published at step j
  float* rowbuf = Lt + NB * kDiagLD;   // [2][NB]
  float* rinvs = rowbuf + 2 * NB;      // [NB] 1 / L[j][j]
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  float v[8][8];
#pragma unroll
  for (int a = 0; a < 8; ++a)
#pragma unroll
    for (int b = 0; b < 8; ++b) {
      const int i = ty + 16 * a, c = tx + 16 * b;
      float x = (i == c) ? 1.0f : 0.0f;   // identity padding beyond n
      if (i < n && c < n) x = (c <= i) ? A[(int64_t)(k0 + i) * lda + (k0 + c)] : 0.0f;
      v[a][b] = x;
    }
  chol_diag_steps<0>(v, Lt, rowbuf, rinvs, n, k0, status, tx, ty);
  chol_diag_steps<1>(v, Lt, rowbuf, rinvs, n, k0, status, tx, ty);
  chol_diag_steps<2>(v, Lt, rowbuf, rinvs, n, k0, status, tx, ty);
  chol_diag_steps<3>(v, Lt, rowbuf, rinvs, n, k0, status, tx, ty);
  chol_diag_steps<4>(v, Lt, rowbuf, rinvs, n, k0, status, tx, ty);
  chol_diag_steps<5>(v, Lt, rowbuf, rinvs, n, k0, status, tx, ty);
  chol_diag_steps<6>(v, Lt, rowbuf, rinvs, n, k0, status, tx, ty);
  chol_diag_steps<7>(v, Lt, rowbuf, rinvs, n, k0, status, tx, ty);
  __syncthreads();
  // inverse: registers -> Dinv
#pragma unroll
  for (int a = 0; a < 8; ++a)
#pragma unroll
    for (int b = 0; b < 8; ++b) {
      const int i = ty + 16 * a, c = tx + 16 * b;
      Dinv[i * NB + c] = (c <= i && i < n) ? v[a][b] : 0.0f;
    }
  // the diagonal block of A takes the inverse as well: L_kk itself is not needed again
  for (int a = 0; a < 8; ++a)
    for (int b = 0; b < 8; ++b) {
      const int i = ty + 16 * a, c = tx + 16 * b;
      if (i < n && c < n) A[(int64_t)(k0 + i) * lda + (k0 + c)] = (c <= i) ? v[a][b] : 0.0f;
    }
}

// ---------------------------------------------------------------------------------------
// Whole factorisation of one SMALL Hessian per CTA, many Hessians per launch.
//
// The same one-pass block algorithm as b200q_gptq_factor - A = J H J (index reversal), a
// right-looking Cholesky A = L L^T carried out together with the forward substitution for
// X = L^-1, U = J X J - but with every step of a problem inside one CTA: the diagonal blocks go
// through chol_diag_steps, the 128 x 128 tile products run on the CTA's FMA units from slices
// staged in shared memory.  A layer with hundreds of small Hessians (the experts of a
// mixture-of-experts layer) then costs one launch instead of dozens per Hessian.
//
// Storage: A (K x K, this problem's scratch) holds, on and below the diagonal, first the
// remaining part of J H J, then per block column k the panel L[i,k], and finally X; block row k
// left of the diagonal holds S'[k,j] = -sum_m L[k,m] X[m,j] until step k turns it into
// X[k,j] = X[k,k] S'[k,j].
constexpr int kTP = NB + 4;   // stride of a staged operand slice: 16-byte aligned rows, conflict-free transposing stores

struct FactorBatch {
  float* const* H;     // per problem: the matrix, K x K, leading dimension ldh (in: H, out: U)
  float* const* A;     // per problem: K * K floats of scratch
  int* status;         // [count][4], zeroed by the caller
  int64_t K, ldh;
};

// C[rows x cols] = beta * C + alpha * P[rows x kk] * Q, all operands with their own leading
// dimension, rows / cols / kk <= 128.  QT = false: Q = Qm^T with Qm [cols x kk]; QT = true:
// Q = Qm [kk x cols].  Operands may live in global or shared memory and may have been written
// earlier by this CTA (no read-only loads).  All 256 threads; thread (ty, tx) owns rows
// {ty*4 .. +3, 64 + ty*4 .. +3} and columns {tx*4 .. +3, 64 + tx*4 .. +3}.
template <bool QT>
__device__ void tile_product(float* C, int64_t ldc, const float* P, int64_t ldp, const float* Qm, int64_t ldq,
                             int rows, int cols, int kk, float alpha, float beta, float* sP, float* sQ) {
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.0f;
  for (int k0 = 0; k0 < kk; k0 += 32) {
    // slices [32 k][128] of P^T and of Q; a lane per row so that the transposing stores spread over the banks
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int r = tid & 127, k = 4 * ((tid >> 7) + 2 * it);
      float x[4] = {0.f, 0.f, 0.f, 0.f};
      if (r < rows) {
        const float* src = P + (int64_t)r * ldp + k0 + k;
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (k0 + k + e < kk) x[e] = src[e];
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) sP[(k + e) * kTP + r] = x[e];
      if (!QT) {
        float y[4] = {0.f, 0.f, 0.f, 0.f};
        if (r < cols) {
          const float* src = Qm + (int64_t)r * ldq + k0 + k;
#pragma unroll
          for (int e = 0; e < 4; ++e)
            if (k0 + k + e < kk) y[e] = src[e];
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) sQ[(k + e) * kTP + r] = y[e];
      }
    }
    if (QT) {
#pragma unroll
      for (int it = 0; it < 4; ++it) {
        const int idx = tid + kDiagThreads * it;     // 32 k x 32 column quads
        const int k = idx >> 5, c = (idx & 31) << 2;
        float4 y = make_float4(0.f, 0.f, 0.f, 0.f);
        if (k0 + k < kk) {
          const float* src = Qm + (int64_t)(k0 + k) * ldq + c;
          if (c < cols) y.x = src[0];
          if (c + 1 < cols) y.y = src[1];
          if (c + 2 < cols) y.z = src[2];
          if (c + 3 < cols) y.w = src[3];
        }
        *reinterpret_cast<float4*>(sQ + k * kTP + c) = y;
      }
    }
    __syncthreads();
#pragma unroll 4
    for (int k = 0; k < 32; ++k) {
      const float4 a0 = *reinterpret_cast<const float4*>(sP + k * kTP + ty * 4);
      const float4 a1 = *reinterpret_cast<const float4*>(sP + k * kTP + 64 + ty * 4);
      const float4 b0 = *reinterpret_cast<const float4*>(sQ + k * kTP + tx * 4);
      const float4 b1 = *reinterpret_cast<const float4*>(sQ + k * kTP + 64 + tx * 4);
      const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float q[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], q[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = (i < 4) ? ty * 4 + i : 64 + ty * 4 + (i - 4);
    if (r >= rows) continue;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int c = (j < 4) ? tx * 4 + j : 64 + tx * 4 + (j - 4);
      if (c >= cols) continue;
      float* d = C + (int64_t)r * ldc + c;
      const float prod = alpha * acc[i][j];
      *d = (beta == 0.0f) ? prod : fmaf(beta, *d, prod);
    }
  }
  __syncthreads();
}

constexpr size_t kFactorSmallSmem = ((size_t)kDiagSmemFloats + 2 * 32 * kTP) * sizeof(float);

__global__ void __launch_bounds__(kDiagThreads, 1) factor_small_kernel(FactorBatch fb) {
  extern __shared__ float sm[];
  float* Lt = sm;                      // diagonal-block scratch; between diagonal blocks a 128 x 129 staging tile
  float* rowbuf = Lt + NB * kDiagLD;
  float* rinvs = rowbuf + 2 * NB;
  float* sP = sm + kDiagSmemFloats;
  float* sQ = sP + 32 * kTP;
  const int job = blockIdx.x;
  float* H = fb.H[job];
  float* A = fb.A[job];
  int* status = fb.status + 4 * job;
  const int64_t K = fb.K, ld = fb.K;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  for (int64_t i = tid; i < K * K; i += kDiagThreads) {
    const int64_t r = i / K, c = i - r * K;
    A[i] = H[(K - 1 - r) * fb.ldh + (K - 1 - c)];
  }
  __syncthreads();
  const int nb = (int)((K + NB - 1) / NB);
  for (int k = 0; k < nb; ++k) {
    const int k0 = k * NB;
    const int n = (int)((K - k0) < NB ? (K - k0) : NB);
    const int rem = (int)(K - k0 - n);
    float* Xkk = A + (int64_t)k0 * ld + k0;
    {
      float v[8][8];
#pragma unroll
      for (int a = 0; a < 8; ++a)
#pragma unroll
        for (int b = 0; b < 8; ++b) {
          const int i = ty + 16 * a, c = tx + 16 * b;
          float x = (i == c) ? 1.0f : 0.0f;
          if (i < n && c < n) x = (c <= i) ? Xkk[(int64_t)i * ld + c] : 0.0f;
          v[a][b] = x;
        }
      chol_diag_steps<0>(v, Lt, rowbuf, rinvs, n, k0, status, tx, ty);
      chol_diag_steps<1>(v, Lt, rowbuf, rinvs, n, k0, status, tx, ty);
      chol_diag_steps<2>(v, Lt, rowbuf, rinvs, n, k0, status, tx, ty);
      chol_diag_steps<3>(v, Lt, rowbuf, rinvs, n, k0, status, tx, ty);
      chol_diag_steps<4>(v, Lt, rowbuf, rinvs, n, k0, status, tx, ty);
      chol_diag_steps<5>(v, Lt, rowbuf, rinvs, n, k0, status, tx, ty);
      chol_diag_steps<6>(v, Lt, rowbuf, rinvs, n, k0, status, tx, ty);
      chol_diag_steps<7>(v, Lt, rowbuf, rinvs, n, k0, status, tx, ty);
      __syncthreads();
#pragma unroll
      for (int a = 0; a < 8; ++a)
#pragma unroll
        for (int b = 0; b < 8; ++b) {
          const int i = ty + 16 * a, c = tx + 16 * b;
          if (i < n && c < n) Xkk[(int64_t)i * ld + c] = (c <= i) ? v[a][b] : 0.0f;
        }
    }
    __syncthreads();
    float* tmp = Lt;   // [128][kDiagLD]
    // X[k, j] = X[k,k] * S'[k, j] for the block columns left of the diagonal
    for (int j = 0; j < k; ++j) {
      float* Skj = A + (int64_t)k0 * ld + j * NB;
      for (int idx = tid; idx < NB * NB; idx += kDiagThreads) {
        const int r = idx >> 7, c = idx & 127;
        if (r < n) tmp[r * kDiagLD + c] = Skj[(int64_t)r * ld + c];
      }
      __syncthreads();
      tile_product<true>(Skj, ld, Xkk, ld, tmp, kDiagLD, n, NB, n, 1.0f, 0.0f, sP, sQ);
    }
    if (rem <= 0) break;
    const int nrem = (rem + NB - 1) / NB;
    // panel: L[i,k] = A[i,k] * X[k,k]^T
    for (int i = 0; i < nrem; ++i) {
      const int ri = (rem - i * NB) < NB ? (rem - i * NB) : NB;
      float* Pi = A + (int64_t)(k0 + n + i * NB) * ld + k0;
      for (int idx = tid; idx < NB * NB; idx += kDiagThreads) {
        const int r = idx >> 7, c = idx & 127;
        if (r < ri && c < n) tmp[r * kDiagLD + c] = Pi[(int64_t)r * ld + c];
      }
      __syncthreads();
      tile_product<false>(Pi, ld, tmp, kDiagLD, Xkk, ld, ri, n, n, 1.0f, 0.0f, sP, sQ);
    }
    // trailing updates:  S'[i,j] -= L[i,k] X[k,j] (j < k),  A[i,j] -= L[i,k] L[j,k]^T (k < j <= i)
    for (int i = 0; i < nrem; ++i) {
      const int ri = (rem - i * NB) < NB ? (rem - i * NB) : NB;
      const float* Pi = A + (int64_t)(k0 + n + i * NB) * ld + k0;
      float* rowi = A + (int64_t)(k0 + n + i * NB) * ld;
      for (int j = 0; j < k; ++j)
        tile_product<true>(rowi + j * NB, ld, Pi, ld, A + (int64_t)k0 * ld + j * NB, ld, ri, NB, n, -1.0f, 1.0f, sP, sQ);
      for (int j = 0; j <= i; ++j) {
        const int rj = (rem - j * NB) < NB ? (rem - j * NB) : NB;
        const float* Pj = A + (int64_t)(k0 + n + j * NB) * ld + k0;
        tile_product<false>(rowi + (k0 + n + j * NB), ld, Pi, ld, Pj, ld, ri, rj, n, -1.0f, 1.0f, sP, sQ);
      }
    }
    // S'[i,k] = -L[i,k] * X[k,k], in place of the panel
    for (int i = 0; i < nrem; ++i) {
      const int ri = (rem - i * NB) < NB ? (rem - i * NB) : NB;
      float* Pi = A + (int64_t)(k0 + n + i * NB) * ld + k0;
      for (int idx = tid; idx < NB * NB; idx += kDiagThreads) {
        const int r = idx >> 7, c = idx & 127;
        if (r < ri && c < n) tmp[r * kDiagLD + c] = Pi[(int64_t)r * ld + c];
      }
      __syncthreads();
      tile_product<true>(Pi, ld, tmp, kDiagLD, Xkk, ld, ri, n, n, -1.0f, 0.0f, sP, sQ);
    }
  }
  __syncthreads();
  for (int64_t i = tid; i < K * K; i += kDiagThreads) {
    const int64_t r = i / K, c = i - r * K;
    H[r * fb.ldh + c] = (c >= r) ? A[(K - 1 - r) * ld + (K - 1 - c)] : 0.0f;
  }
}

static inline int64_t round_up(int64_t v, int64_t m) { return (v + m - 1) / m * m; }

}  // namespace solve
}  // namespace b200q

using namespace b200q;
using namespace b200q::solve;

extern "C" {

int b200q_actorder_perm(const float* H, int64_t K, int64_t ldh, int32_t* perm, void* stream) {
  if (!H || !perm || K <= 0 || ldh < K) return B200Q_ERR_ARG;
  perm_kernel<<<(int)((K + 255) / 256), 256, 0, (cudaStream_t)stream>>>(H, K, ldh, perm);
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_gather_columns_f32(const void* W, int wdtype, int64_t N, int64_t K, int64_t ldw, const int32_t* perm,
                             float* Wf, int64_t ldf, void* stream) {
  if (!W || !Wf || N <= 0 || K <= 0 || ldw < K || ldf < K) return B200Q_ERR_ARG;
  int grid = grid_for((N * K + 255) / 256, 8);
  cudaStream_t st = (cudaStream_t)stream;
  if (wdtype == B200Q_BF16) gather_cols_kernel<B200Q_BF16><<<grid, 256, 0, st>>>(W, N, K, ldw, perm, Wf, ldf);
  else if (wdtype == B200Q_F32) gather_cols_kernel<B200Q_F32><<<grid, 256, 0, st>>>(W, N, K, ldw, perm, Wf, ldf);
  else return B200Q_ERR_UNSUPPORTED;
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_permute_hessian(const float* H, int64_t K, int64_t ldh, const int32_t* perm, float* Hp, int64_t ldp,
                          void* stream) {
  if (!H || !perm || !Hp || K <= 0 || ldh < K || ldp < K || H == Hp) return B200Q_ERR_ARG;
  permute_hessian_kernel<<<grid_for((K * K + 255) / 256, 8), 256, 0, (cudaStream_t)stream>>>(H, K, ldh, perm, Hp, ldp);
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_scatter_columns_cast(const float* Wf, int64_t N, int64_t K, int64_t ldf, const int32_t* perm, void* out,
                               int odtype, int64_t ldo, void* stream) {
  if (!Wf || !out || N <= 0 || K <= 0 || ldf < K || ldo < K) return B200Q_ERR_ARG;
  int grid = grid_for((N * K + 255) / 256, 8);
  cudaStream_t st = (cudaStream_t)stream;
  if (odtype == B200Q_BF16) scatter_cols_kernel<B200Q_BF16><<<grid, 256, 0, st>>>(Wf, N, K, ldf, perm, out, ldo);
  else if (odtype == B200Q_F32) scatter_cols_kernel<B200Q_F32><<<grid, 256, 0, st>>>(Wf, N, K, ldf, perm, out, ldo);
  else return B200Q_ERR_UNSUPPORTED;
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_gather_columns_f32_batched(const void* const* W, int wdtype, const int32_t* const* perm,
                                     const float* const* dead_diag, float* const* Wf, int count, int64_t N,
                                     int64_t K, int64_t ldw, int64_t ldf, void* stream) {
  if (!W || !Wf || count <= 0 || count > 65535 || N <= 0 || K <= 0 || ldw < K || ldf < K) return B200Q_ERR_ARG;
  int gx = grid_for((N * K + 255) / 256, 8);
  const int cap = 8 * kNumSMs / count + 1;          // enough blocks over all problems to fill the machine
  if (gx > cap) gx = cap;
  dim3 grid((unsigned)gx, (unsigned)count, 1);
  cudaStream_t st = (cudaStream_t)stream;
  if (wdtype == B200Q_BF16) gather_cols_batched_kernel<B200Q_BF16><<<grid, 256, 0, st>>>(W, N, K, ldw, perm, dead_diag, Wf, ldf);
  else if (wdtype == B200Q_F32) gather_cols_batched_kernel<B200Q_F32><<<grid, 256, 0, st>>>(W, N, K, ldw, perm, dead_diag, Wf, ldf);
  else return B200Q_ERR_UNSUPPORTED;
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_scatter_columns_cast_batched(const float* const* Wf, const int32_t* const* perm, void* const* out,
                                       int odtype, int count, int64_t N, int64_t K, int64_t ldf, int64_t ldo,
                                       void* stream) {
  if (!Wf || !out || count <= 0 || count > 65535 || N <= 0 || K <= 0 || ldf < K || ldo < K) return B200Q_ERR_ARG;
  int gx = grid_for((N * K + 255) / 256, 8);
  const int cap = 8 * kNumSMs / count + 1;
  if (gx > cap) gx = cap;
  dim3 grid((unsigned)gx, (unsigned)count, 1);
  cudaStream_t st = (cudaStream_t)stream;
  if (odtype == B200Q_BF16) scatter_cols_batched_kernel<B200Q_BF16><<<grid, 256, 0, st>>>(Wf, N, K, ldf, perm, out, ldo);
  else if (odtype == B200Q_F32) scatter_cols_batched_kernel<B200Q_F32><<<grid, 256, 0, st>>>(Wf, N, K, ldf, perm, out, ldo);
  else return B200Q_ERR_UNSUPPORTED;
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_gptq_prepare(float* H, int64_t K, int64_t ldh, float* Wf, int64_t N, int64_t ldf, float percdamp,
                       void* stream) {
  if (!H || K <= 0 || ldh < K) return B200Q_ERR_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  if (Wf && N > 0) {
    zero_dead_columns_kernel<<<grid_for((K * 32 + 255) / 256, 4), 256, 0, st>>>(H, K, ldh + 1, Wf, N, ldf);
    B200Q_LAUNCH_CHECK();
  }
  damp_kernel<<<1, 1024, 0, st>>>(H, K, ldh, percdamp);
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_gptq_zero_dead_columns(const float* diag, int64_t diag_stride, int64_t K, float* Wf, int64_t N,
                                 int64_t ldf, void* stream) {
  if (!diag || !Wf || K <= 0 || N <= 0 || ldf < K || diag_stride <= 0) return B200Q_ERR_ARG;
  zero_dead_columns_kernel<<<grid_for((K * 32 + 255) / 256, 4), 256, 0, (cudaStream_t)stream>>>(diag, K, diag_stride,
                                                                                                Wf, N, ldf);
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

size_t b200q_gptq_factor_workspace_bytes(int64_t K) {
  if (K <= 0) return 0;
  int64_t lda = round_up(K, 32);
  int64_t nb = (K + NB - 1) / NB;
  // reversed matrix + inverse diagonal blocks + hi/lo copies of the two GEMM operands
  // (split buffers are whole 128-row tiles: the GEMM's TMA boxes read full tiles)
  return (size_t)(K * lda + nb * NB * NB + 6 * (nb * NB) * NB + 4 * NB * NB) * sizeof(float);
}

int b200q_gptq_factor(float* H, int64_t K, int64_t ldh, void* workspace, int* status, void* stream) {
  if (!H || !workspace || !status || K <= 0 || ldh < K || K > (1 << 24)) return B200Q_ERR_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t lda = round_up(K, 32);
  const int nb = (int)((K + NB - 1) / NB);
  float* A = (float*)workspace;
  float* Dinv = A + K * lda;                      // nb blocks of 128 x 128
  const int64_t cap = (int64_t)nb * NB * NB;      // floats per split buffer: [roundup(K,128)][128]
  float* sa_hi = Dinv + cap;                      // panel before its update: [rem][128]
  float* sa_lo = sa_hi + cap;
  float* sb_base = sa_lo + cap;                   // operand rows by absolute column: [roundup(K,128)][128],
                                                  // hi and lo, two copies used by alternate steps
  float* d_hi = sb_base + 4 * cap;                // Linv_kk and its transpose, split
  float* d_lo = d_hi + NB * NB;
  float* dt_hi = d_lo + NB * NB;
  float* dt_lo = dt_hi + NB * NB;
  const size_t diag_smem = kDiagSmemFloats * sizeof(float);
  B200Q_TRY(cudaFuncSetAttribute(chol_diag_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)diag_smem));
  using tgemm::Split;
  int rc;
#define B200Q_RC(expr) do { rc = (expr); if (rc != B200Q_OK) return rc; } while (0)

  reverse_in_kernel<<<grid_for((K * K + 255) / 256, 8), 256, 0, st>>>(H, K, ldh, A, lda);
  B200Q_LAUNCH_CHECK();

  // One pass over the block columns does the Cholesky factorisation A = L L^T and the inverse
  // X = L^-1 together.  Before step k, in the rows below block row k: block columns < k hold the
  // accumulators S[i,j] = -sum_{m<k} L[i,m] X[m,j] of the forward substitution, block columns
  // >= k hold the Schur complement of the factorisation.  Step k:
  //   diagonal block        -> L_kk, X[k,k] = L_kk^-1
  //   X[k,:k]  = X[k,k] S[k,:k]
  //   P        = A[k+1:,k] X[k,k]^T                       (= L[k+1:,k])
  //   S[i,k]   = -P X[k,k]                                (in place of P)
  //   S[i,:k] -= P X[k,:k]   and   A[i,j] -= P P^T (j > k, lower tiles)      one GEMM launch
  //
  // Look-ahead: the update of step k is split in the tiles step k+1 reads (block row k+1 and
  // block column k+1: tgemm::kSkipBlockFirst, on the caller's stream) and the rest
  // (kSkipBlockRest), which runs on a helper stream beside step k+1's diagonal block and panel
  // work.  Both parts of step k+1 touch tiles the rest of step k also updates, so they wait for it;
  // the operand panels alternate between two buffers because the helper may still read step k's
  // while step k+1's are written.
  tgemm::SideStream* side = tgemm::side_stream(st);
  bool side_busy = false;
  for (int k = 0; k < nb; ++k) {
    const int k0 = k * NB;
    const int n = (int)min((int64_t)NB, K - k0);
    const int rem = (int)(K - k0 - n);
    float* Dk = Dinv + (int64_t)k * NB * NB;
    float* rowk = A + (int64_t)k0 * lda;        // block row k, columns < k0: n x k0
    float* sb_hi = sb_base + (int64_t)(k & 1) * 2 * cap;
    float* sb_lo = sb_hi + cap;
    const int64_t ldn = tgemm::split_ld(n);
    chol_diag_kernel<<<1, kDiagThreads, diag_smem, st>>>(A, lda, k0, n, Dk, status);
    B200Q_LAUNCH_CHECK();
    if (k0 == 0 && rem <= 0) break;
    B200Q_RC(tgemm::split(Dk, NB, n, n, d_hi, d_lo, st));
    if (k0 > 0) {
      // X[k,:k0] <- X[k,k] * S[k,:k0]
      B200Q_RC(tgemm::split_transposed(rowk, lda, n, k0, sb_hi, sb_lo, st));
      B200Q_RC(tgemm::launch(tgemm::kNT, Split{d_hi, d_lo, ldn}, Split{sb_hi, sb_lo, ldn}, rowk, lda, n, k0, n, 1.0f,
                             0.0f, tgemm::kAllTiles, status + 2, st));
    }
    if (rem <= 0) break;
    float* P = A + (int64_t)(k0 + n) * lda + k0;  // panel below the diagonal block: rem x n
    // P <- P * X[k,k]^T   (out[r][c] = sum_m P[r][m] * X[c][m])
    B200Q_RC(tgemm::split(P, lda, rem, n, sa_hi, sa_lo, st));
    B200Q_RC(tgemm::launch(tgemm::kNT, Split{sa_hi, sa_lo, ldn}, Split{d_hi, d_lo, ldn}, P, lda, rem, n, n, 1.0f, 0.0f,
                           tgemm::kAllTiles, status + 2, st));
    // operand rows of the update, indexed by absolute column: X[k,:k0]^T, then (after the gap of
    // block k) the new panel
    float* ph = sb_hi + (int64_t)(k0 + n) * NB;
    float* pl = sb_lo + (int64_t)(k0 + n) * NB;
    B200Q_RC(tgemm::split(P, lda, rem, n, ph, pl, st));
    if (k0 > 0) B200Q_RC(tgemm::split_transposed(rowk, lda, n, k0, sb_hi, sb_lo, st));
    // S[i,k] = -P * X[k,k]  (in place on the panel; the operand is read from its split copy)
    B200Q_RC(tgemm::split_transposed(Dk, NB, n, n, dt_hi, dt_lo, st));
    B200Q_RC(tgemm::launch(tgemm::kNT, Split{ph, pl, ldn}, Split{dt_hi, dt_lo, ldn}, P, lda, rem, n, n, -1.0f, 0.0f,
                           tgemm::kAllTiles, status + 2, st));
    // rows below block k: columns < k0 take -P X[k,:k0], columns > block k take -P P^T
    float* C = A + (int64_t)(k0 + n) * lda;
    if (!side) {
      B200Q_RC(tgemm::launch(tgemm::kNT, Split{ph, pl, ldn}, Split{sb_hi, sb_lo, ldn}, C, lda, rem, (int)K, n, -1.0f,
                             1.0f, tgemm::kSkipBlockTiles, status + 2, st, k));
      continue;
    }
    B200Q_TRY(cudaEventRecord(side->ready, st));
    B200Q_TRY(cudaStreamWaitEvent(side->stream, side->ready, 0));
    if (side_busy) B200Q_TRY(cudaStreamWaitEvent(st, side->done, 0));   // rest of step k-1
    B200Q_RC(tgemm::launch(tgemm::kNT, Split{ph, pl, ldn}, Split{sb_hi, sb_lo, ldn}, C, lda, rem, (int)K, n, -1.0f,
                           1.0f, tgemm::kSkipBlockFirst, status + 2, st, k));
    B200Q_RC(tgemm::launch(tgemm::kNT, Split{ph, pl, ldn}, Split{sb_hi, sb_lo, ldn}, C, lda, rem, (int)K, n, -1.0f,
                           1.0f, tgemm::kSkipBlockRest, status + 2, side->stream, k, kNumSMs - tgemm::side_reserve()));
    B200Q_TRY(cudaEventRecord(side->done, side->stream));
    side_busy = true;
  }
  if (side_busy) B200Q_TRY(cudaStreamWaitEvent(st, side->done, 0));
#undef B200Q_RC

  reverse_out_kernel<<<grid_for((K * K + 255) / 256, 8), 256, 0, st>>>(A, K, lda, H, ldh);
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

size_t b200q_gptq_factor_batched_workspace_bytes(int64_t K, int count) {
  if (K <= 0 || count <= 0) return 0;
  return (size_t)K * (size_t)K * sizeof(float) * (size_t)count;
}

int b200q_gptq_factor_batched(float* const* H, float* const* scratch, int count, int64_t K, int64_t ldh, int* status,
                              void* stream) {
  if (!H || !scratch || !status || count <= 0 || K <= 0 || ldh < K) return B200Q_ERR_ARG;
  if (K > 4096) return B200Q_ERR_UNSUPPORTED;
  FactorBatch fb;
  fb.H = H; fb.A = scratch; fb.status = status; fb.K = K; fb.ldh = ldh;
  cudaStream_t st = (cudaStream_t)stream;
  B200Q_TRY(cudaMemsetAsync(status, 0, sizeof(int) * 4 * (size_t)count, st));
  B200Q_TRY(cudaFuncSetAttribute(factor_small_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)kFactorSmallSmem));
  factor_small_kernel<<<count, kDiagThreads, kFactorSmallSmem, st>>>(fb);
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

}  // extern "C"

// fp32-accurate tile GEMM of the solve, exposed for testing and reuse:
//   C[M,N] = beta*C + alpha * A[M,Kd] * (trans_b ? B[N,Kd]^T : B[Kd,N]),  Kd <= 128.
extern "C" size_t b200q_gemm_tf32x3_workspace_bytes(int64_t M, int64_t N, int64_t Kd) {
  if (M <= 0 || N <= 0 || Kd <= 0) return 0;
  const int64_t kp = tgemm::split_ld(Kd);
  const int64_t a = (M + 127) / 128 * 128 * kp, b = (N + 127) / 128 * 128 * kp;
  return (size_t)(2 * a + 2 * b) * sizeof(float);
}
extern "C" int b200q_gemm_tf32x3(int trans_b, const float* A, int64_t lda, const float* B, int64_t ldb, float* C,
                                 int64_t ldc, int64_t M, int64_t N, int64_t Kd, float alpha, float beta,
                                 int lower_tiles, void* workspace, int* status, void* stream) {
  if (!A || !B || !C || !workspace || M <= 0 || N <= 0 || Kd <= 0 || Kd > 128) return B200Q_ERR_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t kp = tgemm::split_ld(Kd);
  const int64_t asz = (M + 127) / 128 * 128 * kp, bsz = (N + 127) / 128 * 128 * kp;
  float* a_hi = (float*)workspace;
  float* a_lo = a_hi + asz;
  float* b_hi = a_lo + asz;
  float* b_lo = b_hi + bsz;
  int rc = tgemm::split(A, lda, (int)M, (int)Kd, a_hi, a_lo, st);
  if (rc) return rc;
  if (trans_b) rc = tgemm::split(B, ldb, (int)N, (int)Kd, b_hi, b_lo, st);
  else rc = tgemm::split_transposed(B, ldb, (int)Kd, (int)N, b_hi, b_lo, st);
  if (rc) return rc;
  return tgemm::launch(tgemm::kNT, tgemm::Split{a_hi, a_lo, kp}, tgemm::Split{b_hi, b_lo, kp}, C, ldc, (int)M, (int)N, (int)Kd, alpha, beta,
                       lower_tiles ? tgemm::kLowerTiles : tgemm::kAllTiles, status, st);
}
