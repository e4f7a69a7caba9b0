// fp32 SIMT GEMM used by the GPTQ factorisation and the sweep's trailing update.
//
//   C[M,N] = beta * C + alpha * A[M,Kd] * op(B)      op(B) = B[Kd,N]   (kNN)
//                                                     op(B) = B[N,Kd]^T (kNT)
// 128x128 output tile per CTA, 256 threads, 8x8 register tile per thread, 16-deep k-chunks
// staged through registers into double-buffered shared memory.  Tiles can be restricted to
// the lower block triangle (j-tile <= i-tile) for symmetric updates.  C may alias A or B
// only in the "panel" use where Kd <= 128 and each CTA reads everything it needs before its
// first store (see gemm_panel_inplace).
#pragma once

#include "common.cuh"

namespace b200q {
namespace sgemm {

constexpr int BM = 128, BN = 128, BK = 16, THREADS = 256;

enum Trans { kNN = 0, kNT = 1 };
enum TileMask { kAllTiles = 0, kLowerTiles = 1 };

struct Args {
  const float* A; int64_t lda;
  const float* B; int64_t ldb;
  float* C; int64_t ldc;
  int M, N, Kd;
  float alpha, beta;
  int tiles_m, tiles_n;
  int mask;
};

__device__ __forceinline__ void tile_from_index(const Args& a, int64_t t, int& tm, int& tn) {
  if (a.mask == kLowerTiles) {
    // t enumerates pairs (tm >= tn)
    int i = (int)((sqrt(8.0 * (double)t + 1.0) - 1.0) * 0.5);
    while ((int64_t)i * (i + 1) / 2 > t) --i;
    while ((int64_t)(i + 1) * (i + 2) / 2 <= t) ++i;
    tm = i;
    tn = (int)(t - (int64_t)i * (i + 1) / 2);
  } else {
    tm = (int)(t / a.tiles_n);
    tn = (int)(t - (int64_t)tm * a.tiles_n);
  }
}

template <int TRANS>
__global__ void __launch_bounds__(THREADS, 2) sgemm_kernel(Args a, int64_t num_tiles) {
  __shared__ __align__(16) float As[2][BK][BM + 4];
  __shared__ __align__(16) float Bs[2][BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;  // 16 x 16 threads; each owns rows {ty*4.., 64+ty*4..} x cols {tx*4.., 64+tx*4..}
  const bool vecA = ((a.lda & 3) == 0) && ((((uintptr_t)a.A) & 15) == 0);
  const bool vecB = ((a.ldb & 3) == 0) && ((((uintptr_t)a.B) & 15) == 0);

  for (int64_t t = blockIdx.x; t < num_tiles; t += gridDim.x) {
    int tm, tn;
    tile_from_index(a, t, tm, tn);
    const int m0 = tm * BM, n0 = tn * BN;
    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[i][j] = 0.0f;

    // global -> register staging: A chunk is 128 rows x 16 k = 512 float4, 2 per thread
    // (row = idx / 4, k4 = idx % 4).  B chunk: NN: 16 k x 128 n = 512 float4 (k = idx / 32,
    // n4 = idx % 32); NT: like A with n as the row.
    float4 ra[2], rb[2];
    auto load_chunk = [&](int k0) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int idx = tid + h * THREADS;
        {
          const int r = idx >> 2, k4 = (idx & 3) * 4;
          const int gm = m0 + r, gk = k0 + k4;
          float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
          if (gm < a.M) {
            const float* p = a.A + (int64_t)gm * a.lda + gk;
            if (vecA && gk + 3 < a.Kd) v = *reinterpret_cast<const float4*>(p);
            else {
              if (gk < a.Kd) v.x = p[0];
              if (gk + 1 < a.Kd) v.y = p[1];
              if (gk + 2 < a.Kd) v.z = p[2];
              if (gk + 3 < a.Kd) v.w = p[3];
            }
          }
          ra[h] = v;
        }
        if (TRANS == kNT) {
          const int r = idx >> 2, k4 = (idx & 3) * 4;
          const int gn = n0 + r, gk = k0 + k4;
          float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
          if (gn < a.N) {
            const float* p = a.B + (int64_t)gn * a.ldb + gk;
            if (vecB && gk + 3 < a.Kd) v = *reinterpret_cast<const float4*>(p);
            else {
              if (gk < a.Kd) v.x = p[0];
              if (gk + 1 < a.Kd) v.y = p[1];
              if (gk + 2 < a.Kd) v.z = p[2];
              if (gk + 3 < a.Kd) v.w = p[3];
            }
          }
          rb[h] = v;
        } else {
          const int k = idx >> 5, n4 = (idx & 31) * 4;
          const int gk = k0 + k, gn = n0 + n4;
          float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
          if (gk < a.Kd) {
            const float* p = a.B + (int64_t)gk * a.ldb + gn;
            if (vecB && gn + 3 < a.N) v = *reinterpret_cast<const float4*>(p);
            else {
              if (gn < a.N) v.x = p[0];
              if (gn + 1 < a.N) v.y = p[1];
              if (gn + 2 < a.N) v.z = p[2];
              if (gn + 3 < a.N) v.w = p[3];
            }
          }
          rb[h] = v;
        }
      }
    };
    auto store_chunk = [&](int buf) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int idx = tid + h * THREADS;
        {
          const int r = idx >> 2, k4 = (idx & 3) * 4;
          As[buf][k4 + 0][r] = ra[h].x; As[buf][k4 + 1][r] = ra[h].y;
          As[buf][k4 + 2][r] = ra[h].z; As[buf][k4 + 3][r] = ra[h].w;
        }
        if (TRANS == kNT) {
          const int r = idx >> 2, k4 = (idx & 3) * 4;
          Bs[buf][k4 + 0][r] = rb[h].x; Bs[buf][k4 + 1][r] = rb[h].y;
          Bs[buf][k4 + 2][r] = rb[h].z; Bs[buf][k4 + 3][r] = rb[h].w;
        } else {
          const int k = idx >> 5, n4 = (idx & 31) * 4;
          *reinterpret_cast<float4*>(&Bs[buf][k][n4]) = rb[h];
        }
      }
    };

    const int chunks = (a.Kd + BK - 1) / BK;
    load_chunk(0);
    store_chunk(0);
    __syncthreads();
    for (int c = 0; c < chunks; ++c) {
      const int buf = c & 1;
      if (c + 1 < chunks) load_chunk((c + 1) * BK);
#pragma unroll
      for (int k = 0; k < BK; ++k) {
        const float4 a0 = *reinterpret_cast<const float4*>(&As[buf][k][ty * 4]);
        const float4 a1 = *reinterpret_cast<const float4*>(&As[buf][k][64 + ty * 4]);
        const float4 b0 = *reinterpret_cast<const float4*>(&Bs[buf][k][tx * 4]);
        const float4 b1 = *reinterpret_cast<const float4*>(&Bs[buf][k][64 + tx * 4]);
        const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
        const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
      }
      if (c + 1 < chunks) store_chunk(buf ^ 1);
      __syncthreads();
    }

    // epilogue: C = beta*C + alpha*acc
    const bool vecC = ((a.ldc & 3) == 0) && ((((uintptr_t)a.C) & 15) == 0);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int gm = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
      if (gm >= a.M) continue;
#pragma unroll
      for (int jh = 0; jh < 2; ++jh) {
        const int gn = n0 + (jh == 0 ? tx * 4 : 64 + tx * 4);
        float* p = a.C + (int64_t)gm * a.ldc + gn;
        const float* v = &acc[i][jh * 4];
        if (vecC && gn + 3 < a.N) {
          float4 c4 = make_float4(0.f, 0.f, 0.f, 0.f);
          if (a.beta != 0.0f) c4 = *reinterpret_cast<const float4*>(p);
          c4.x = a.beta * c4.x + a.alpha * v[0];
          c4.y = a.beta * c4.y + a.alpha * v[1];
          c4.z = a.beta * c4.z + a.alpha * v[2];
          c4.w = a.beta * c4.w + a.alpha * v[3];
          *reinterpret_cast<float4*>(p) = c4;
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (gn + j < a.N) {
              float c = (a.beta != 0.0f) ? p[j] : 0.0f;
              p[j] = a.beta * c + a.alpha * v[j];
            }
        }
      }
    }
    __syncthreads();
  }
}

// Host launcher.  Returns a cudaError_t from the launch.
inline cudaError_t launch(int trans, const float* A, int64_t lda, const float* B, int64_t ldb, float* C,
                          int64_t ldc, int M, int N, int Kd, float alpha, float beta, int mask,
                          cudaStream_t st) {
  if (M <= 0 || N <= 0 || Kd <= 0) return cudaSuccess;
  Args a;
  a.A = A; a.lda = lda; a.B = B; a.ldb = ldb; a.C = C; a.ldc = ldc;
  a.M = M; a.N = N; a.Kd = Kd; a.alpha = alpha; a.beta = beta; a.mask = mask;
  a.tiles_m = (M + BM - 1) / BM; a.tiles_n = (N + BN - 1) / BN;
  int64_t tiles = (mask == kLowerTiles) ? (int64_t)a.tiles_m * (a.tiles_m + 1) / 2
                                        : (int64_t)a.tiles_m * a.tiles_n;
  int grid = grid_for(tiles, 2);
  if (trans == kNT) sgemm_kernel<kNT><<<grid, THREADS, 0, st>>>(a, tiles);
  else sgemm_kernel<kNN><<<grid, THREADS, 0, st>>>(a, tiles);
  count_launch();
  return cudaGetLastError();
}

}  // namespace sgemm
}  // namespace b200q
