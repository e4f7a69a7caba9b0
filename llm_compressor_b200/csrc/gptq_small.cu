// GPTQ solve for MANY SMALL modules at once (the experts of a mixture-of-experts layer).
//
// The blocked kernels of gptq_solve.cu / gptq_sweep.cu spend one launch per step of every chain;
// a layer with hundreds of small modules then needs tens of thousands of launches and is bound by
// the host.  Here one launch serves a whole batch of equally shaped problems, given as device
// arrays of pointers:
//   * sweep_fused_kernel: a CTA owns 64 rows of one module through ALL column blocks - the
//     128-column block sweep (the lane-per-row scheme of sweep_block_kernel) followed by the
//     trailing update of those rows, W[rows, after] -= Err * U[block, after], as a float32 FMA
//     tile product inside the CTA (the error panel in shared memory, slices of U streamed in by
//     asynchronous copies);
//   * factor_small_kernel (gptq_solve.cu): a CTA factors one small Hessian completely.
#include "common.cuh"

namespace b200q {
namespace small {

constexpr int NB = 128;
constexpr int kRows = 64;                  // rows of a module per CTA (2 row-owning warps)
constexpr int kThreads = 128;
constexpr int kSweepWarps = kRows / 32;
constexpr int kSub = 16;
constexpr int kWLD = kRows + 4;            // stride of a column of the block's tile: columns start 16-byte aligned
constexpr int kColChunk = 64;              // columns of the trailing update per pass

struct SweepBatch {
  float* const* W; const float* const* U; const void* const* scale; const void* const* zp;
  const int32_t* const* col_group; const float* const* gscale; float* const* losses;
  int64_t N, K, ldw, ldu;
  int strategy, group_size, block_h, zp_kind;
  int64_t groups_per_row;
  QRange qr;
};

// Two CTAs fit one SM (about 100 KB each): while one of them is in its latency-bound sweep phase
// the other one's trailing update keeps the FMA pipes busy.
__host__ __device__ constexpr size_t sweep_smem_bytes() {
  return ((size_t)NB * NB + (size_t)NB * kWLD) * sizeof(float);
}

__device__ __forceinline__ void cp_async16(float* dst_smem, const float* src, int src_bytes) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst_smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

template <int SDT, bool GLOBAL, int KIND>
__global__ void __launch_bounds__(kThreads, 2) sweep_fused_kernel(SweepBatch b) {
  constexpr bool SB = Elem<SDT>::is_bf16 && !GLOBAL;
  const float qmin = b.qr.qmin, qmax = b.qr.qmax;
  extern __shared__ float sm[];
  float* sU = sm;                          // [128][128] diagonal block; during the trailing update two [128][64] slices of U
  float* sW = sU + NB * NB;                // [128 cols][kWLD]: the block's columns of this CTA's rows, then their errors
  __shared__ float s_rd[NB];
  __shared__ int s_grp[NB];
  __shared__ int s_same[NB / kSub];
  const int job = blockIdx.y;
  float* __restrict__ W = b.W[job];
  const float* __restrict__ U = b.U ? b.U[job] : nullptr;
  const void* scale = b.scale[job];
  const void* zp = b.zp ? b.zp[job] : nullptr;
  const int32_t* col_group = b.col_group ? b.col_group[job] : nullptr;
  const float g = GLOBAL ? *b.gscale[job] : 1.0f;
  const bool has_zp = zp != nullptr;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row_base = (int64_t)blockIdx.x * kRows;
  const int64_t row = row_base + warp * 32 + lane;          // meaningful for the sweeping warps
  const bool sweeper = warp < kSweepWarps;
  const bool live = sweeper && row < b.N;
  const bool vecw = ((b.ldw & 3) == 0) && ((((uintptr_t)W) & 15) == 0);
  const bool vecu = U && ((b.ldu & 3) == 0) && ((((uintptr_t)U) & 15) == 0);
  int64_t pbase = 0;
  if (sweeper) {
    switch (b.strategy) {
      case B200Q_TENSOR: pbase = 0; break;
      case B200Q_CHANNEL: pbase = row; break;
      case B200Q_BLOCK: pbase = (row / b.block_h) * b.groups_per_row; break;
      default: pbase = row * b.groups_per_row; break;
    }
  }
  float loss = 0.0f;
  for (int64_t i1 = 0; i1 < b.K; i1 += NB) {
    const int bs = (int)((b.K - i1) < NB ? (b.K - i1) : NB);
    const int64_t i2 = i1 + bs;
    // ---- diagonal block of U, reciprocal pivots, parameter column of every column
#pragma unroll 4
    for (int idx = threadIdx.x; idx < NB * NB / 4; idx += kThreads) {
      const int r = idx >> 5, c = (idx & 31) << 2;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (r < bs && c + 3 >= r) {
        if (!U) {
          v.x = (r == c) ? 1.0f : 0.0f; v.y = (r == c + 1) ? 1.0f : 0.0f;
          v.z = (r == c + 2) ? 1.0f : 0.0f; v.w = (r == c + 3) ? 1.0f : 0.0f;
        } else {
          const float* src = U + (i1 + r) * b.ldu + (i1 + c);
          if (vecu && c + 3 < bs) {
            v = *reinterpret_cast<const float4*>(src);
          } else {
            if (c < bs) v.x = src[0];
            if (c + 1 < bs) v.y = src[1];
            if (c + 2 < bs) v.z = src[2];
            if (c + 3 < bs) v.w = src[3];
          }
        }
      }
      *reinterpret_cast<float4*>(sU + idx * 4) = v;
    }
    for (int i = threadIdx.x; i < NB; i += kThreads) {
      float d = 1.0f;
      int grp = 0;
      if (i < bs) {
        if (U) d = U[(i1 + i) * b.ldu + (i1 + i)];
        const int col = (int)i1 + i;
        grp = (b.strategy == B200Q_TENSOR || b.strategy == B200Q_CHANNEL)
                  ? 0 : (col_group ? col_group[col] : col / b.group_size);
      }
      s_rd[i] = __frcp_rn(d);
      s_grp[i] = grp;
    }
    __syncthreads();
    if (threadIdx.x < NB / kSub) {   // does one (scale, zero point) govern the whole sub-block?
      bool same = true;
      for (int t = 1; t < kSub; ++t) same = same && s_grp[threadIdx.x * kSub + t] == s_grp[threadIdx.x * kSub];
      s_same[threadIdx.x] = same ? 1 : 0;
    }
    __syncthreads();
    // ---- the block's columns, swept by the row-owning warps (a lane per row)
    if (sweeper) {
      float* myW = sW + warp * 32;
      {
        const float* src = W + row * b.ldw + i1;
#pragma unroll 8
        for (int c = 0; c < NB; c += 4) {
          float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
          if (live) {
            if (vecw && c + 3 < bs) {
              v = *reinterpret_cast<const float4*>(src + c);
            } else {
              if (c < bs) v.x = src[c];
              if (c + 1 < bs) v.y = src[c + 1];
              if (c + 2 < bs) v.z = src[c + 2];
              if (c + 3 < bs) v.w = src[c + 3];
            }
          }
          myW[(c + 0) * kWLD + lane] = v.x; myW[(c + 1) * kWLD + lane] = v.y;
          myW[(c + 2) * kWLD + lane] = v.z; myW[(c + 3) * kWLD + lane] = v.w;
        }
      }
      int cur_grp = -1;
      float s = 1.0f, z = 0.0f, rs = 1.0f;
#pragma unroll 1
      for (int sub = 0; sub * kSub < bs; ++sub) {
        const int c0 = sub * kSub;
        // parameters of the sub-block's columns, fetched before the dependent chain starts (columns
        // at or beyond bs are zero columns with a unit pivot: they run through and change nothing)
        float sv[kSub], rsv[kSub], zv[kSub];
        if (s_same[sub]) {   // uniform
          const int grp = s_grp[c0];
          if (grp != cur_grp) {
            cur_grp = grp;
            if (live) {
              const int64_t pi = pbase + grp;
              s = Elem<SDT>::load((const typename Elem<SDT>::type*)scale + pi);
              if (GLOBAL) s = __fdiv_rn(s, g);
              rs = __frcp_rn(s);
              if (has_zp) z = load_zp(zp, b.zp_kind, pi);
            }
          }
#pragma unroll
          for (int t = 0; t < kSub; ++t) { sv[t] = s; rsv[t] = rs; zv[t] = z; }
        } else {             // act-order: every column may have its own group
          cur_grp = -1;
#pragma unroll
          for (int t = 0; t < kSub; ++t) {
            float st = 1.0f, zt = 0.0f;
            if (live) {
              const int64_t pi = pbase + s_grp[c0 + t];
              st = Elem<SDT>::load((const typename Elem<SDT>::type*)scale + pi);
              if (GLOBAL) st = __fdiv_rn(st, g);
              if (has_zp) zt = load_zp(zp, b.zp_kind, pi);
            }
            sv[t] = st; rsv[t] = __frcp_rn(st); zv[t] = zt;
          }
        }
        float w[kSub], e[kSub], rd[kSub];
#pragma unroll
        for (int t = 0; t < kSub; ++t) { w[t] = myW[(c0 + t) * kWLD + lane]; rd[t] = s_rd[c0 + t]; }
#pragma unroll
        for (int t = 0; t < kSub; ++t) {
          const int i = c0 + t;
          const float wi = w[t];
          const float q = fake_quant_f32<KIND, SB>(wi, sv[t], rsv[t], zv[t], qmin, qmax);
          const float diff = __fsub_rn(wi, q);
          const float tt = __fmul_rn(diff, rd[t]);
          loss = fmaf(tt, tt, loss);
          e[t] = tt;
          w[t] = q;
          const float4* urow = reinterpret_cast<const float4*>(sU + i * NB + c0);
#pragma unroll
          for (int k4 = (t + 1) / 4; k4 < kSub / 4; ++k4) {
            const float4 u = urow[k4];
            if (4 * k4 + 0 > t) w[4 * k4 + 0] = __fsub_rn(w[4 * k4 + 0], __fmul_rn(tt, u.x));
            if (4 * k4 + 1 > t) w[4 * k4 + 1] = __fsub_rn(w[4 * k4 + 1], __fmul_rn(tt, u.y));
            if (4 * k4 + 2 > t) w[4 * k4 + 2] = __fsub_rn(w[4 * k4 + 2], __fmul_rn(tt, u.z));
            if (4 * k4 + 3 > t) w[4 * k4 + 3] = __fsub_rn(w[4 * k4 + 3], __fmul_rn(tt, u.w));
          }
        }
        // the sub-block's columns are final: out to the weight, and their errors take their
        // place in the tile for the trailing update
        if (live) {
          float* dst = W + row * b.ldw + i1 + c0;
          if (vecw && c0 + kSub <= bs) {
#pragma unroll
            for (int t = 0; t < kSub; t += 4)
              *reinterpret_cast<float4*>(dst + t) = make_float4(w[t], w[t + 1], w[t + 2], w[t + 3]);
          } else {
#pragma unroll
            for (int t = 0; t < kSub; ++t)
              if (c0 + t < bs) dst[t] = w[t];
          }
        }
#pragma unroll
        for (int t = 0; t < kSub; ++t) myW[(c0 + t) * kWLD + lane] = e[t];
        // the later columns of the block take this sub-block's corrections: v -= e * u as a packed
        // product and a packed sum with -e, eight columns (four independent chains) per pass
        uint64_t ne2[kSub];
#pragma unroll
        for (int t = 0; t < kSub; ++t) asm("mov.b64 %0, {%1, %1};" : "=l"(ne2[t]) : "f"(-e[t]));
#pragma unroll 1
        for (int c = c0 + kSub; c < bs; c += 8) {
          uint64_t v[4];
#pragma unroll
          for (int h = 0; h < 4; ++h)
            asm("mov.b64 %0, {%1, %2};" : "=l"(v[h]) : "f"(myW[(c + 2 * h) * kWLD + lane]), "f"(myW[(c + 2 * h + 1) * kWLD + lane]));
#pragma unroll
          for (int t = 0; t < kSub; ++t) {
            const ulonglong2 ua = *reinterpret_cast<const ulonglong2*>(sU + (c0 + t) * NB + c);
            const ulonglong2 ub = *reinterpret_cast<const ulonglong2*>(sU + (c0 + t) * NB + c + 4);
            const uint64_t u[4] = {ua.x, ua.y, ub.x, ub.y};
#pragma unroll
            for (int h = 0; h < 4; ++h) {
              uint64_t pr;
              asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(pr) : "l"(ne2[t]), "l"(u[h]));
              asm("add.rn.f32x2 %0, %1, %2;" : "=l"(v[h]) : "l"(v[h]), "l"(pr));
            }
          }
#pragma unroll
          for (int h = 0; h < 4; ++h) {
            float lo, hi;
            asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v[h]));
            myW[(c + 2 * h) * kWLD + lane] = lo; myW[(c + 2 * h + 1) * kWLD + lane] = hi;
          }
        }
      }
    }
    __syncthreads();
    // ---- trailing update of this CTA's rows: W[rows, i2:] -= Err[rows, bs] * U[i1:i2, i2:],
    // 64 columns at a time; the slices of U arrive by asynchronous copies, one slice ahead
    if (U && i2 < b.K) {
      const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;     // 8 x 16 threads, 8 rows x 4 columns each
      const float* sErr = sW;                                     // [k][kWLD]
      const int nchunks = (int)((b.K - i2 + kColChunk - 1) / kColChunk);
      auto stage = [&](int chunk) {
        float* buf = sU + (chunk & 1) * (NB * kColChunk);
        const int64_t j0 = i2 + (int64_t)chunk * kColChunk;
#pragma unroll 4
        for (int idx = threadIdx.x; idx < NB * kColChunk / 4; idx += kThreads) {
          const int k = idx >> 4, c = (idx & 15) << 2;
          float* dst = buf + k * kColChunk + c;
          const int64_t col = j0 + c;
          if (vecu) {
            int bytes = 0;
            if (k < bs && col < b.K) bytes = (b.K - col) >= 4 ? 16 : (int)(b.K - col) * 4;
            cp_async16(dst, bytes ? U + (i1 + k) * b.ldu + col : U, bytes);
          } else {
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (k < bs) {
              const float* src = U + (i1 + k) * b.ldu + col;
              if (col < b.K) v.x = src[0];
              if (col + 1 < b.K) v.y = src[1];
              if (col + 2 < b.K) v.z = src[2];
              if (col + 3 < b.K) v.w = src[3];
            }
            *reinterpret_cast<float4*>(dst) = v;
          }
        }
        cp_async_commit();
      };
      stage(0);
      for (int chunk = 0; chunk < nchunks; ++chunk) {
        if (chunk + 1 < nchunks) {
          stage(chunk + 1);
          cp_async_wait<1>();
        } else {
          cp_async_wait<0>();
        }
        __syncthreads();
        const float* buf = sU + (chunk & 1) * (NB * kColChunk);
        const int64_t j0 = i2 + (int64_t)chunk * kColChunk;
        const int64_t col = j0 + tx * 4;
        const bool whole = vecw && col + 3 < b.K;
        // this thread's part of W, on its way while the products are formed
        float4 wv[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int64_t rr = row_base + ty * 8 + i;
          wv[i] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (rr < b.N) {
            const float* src = W + rr * b.ldw + col;
            if (whole) {
              wv[i] = *reinterpret_cast<const float4*>(src);
            } else {
              if (col < b.K) wv[i].x = src[0];
              if (col + 1 < b.K) wv[i].y = src[1];
              if (col + 2 < b.K) wv[i].z = src[2];
              if (col + 3 < b.K) wv[i].w = src[3];
            }
          }
        }
        float acc[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) acc[i][jj] = 0.0f;
#pragma unroll 8
        for (int k = 0; k < bs; ++k) {
          const float4 a0 = *reinterpret_cast<const float4*>(sErr + k * kWLD + ty * 8);
          const float4 a1 = *reinterpret_cast<const float4*>(sErr + k * kWLD + ty * 8 + 4);
          const float4 u = *reinterpret_cast<const float4*>(buf + k * kColChunk + tx * 4);
          const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            acc[i][0] = fmaf(a[i], u.x, acc[i][0]); acc[i][1] = fmaf(a[i], u.y, acc[i][1]);
            acc[i][2] = fmaf(a[i], u.z, acc[i][2]); acc[i][3] = fmaf(a[i], u.w, acc[i][3]);
          }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int64_t rr = row_base + ty * 8 + i;
          if (rr >= b.N) continue;
          float* dst = W + rr * b.ldw + col;
          const float4 r = make_float4(__fsub_rn(wv[i].x, acc[i][0]), __fsub_rn(wv[i].y, acc[i][1]),
                                       __fsub_rn(wv[i].z, acc[i][2]), __fsub_rn(wv[i].w, acc[i][3]));
          if (whole) {
            *reinterpret_cast<float4*>(dst) = r;
          } else {
            if (col < b.K) dst[0] = r.x;
            if (col + 1 < b.K) dst[1] = r.y;
            if (col + 2 < b.K) dst[2] = r.z;
            if (col + 3 < b.K) dst[3] = r.w;
          }
        }
        __syncthreads();
      }
    }
  }
  if (live) b.losses[job][row] = loss * 0.5f;
}

}  // namespace small
}  // namespace b200q

using namespace b200q;

extern "C" {

int b200q_gptq_sweep_batched(float* const* W, const float* const* U, const void* const* scale, int sdtype,
                             const void* const* zp, const int32_t* const* col_group, const float* const* gscale,
                             float* const* losses, int count, int64_t N, int64_t K, int64_t ldw, int64_t ldu,
                             const b200q_qargs* qa, int blocksize, void* stream) {
  using namespace b200q::small;
  if (!W || !scale || !losses || !qa || count <= 0 || N <= 0 || K <= 0 || ldw < K || (U && ldu < K)) return B200Q_ERR_ARG;
  if (blocksize != NB) return B200Q_ERR_UNSUPPORTED;
  if (count > 65535) return B200Q_ERR_ARG;
  SweepBatch b;
  int rc = make_qrange(qa, &b.qr); if (rc) return rc;
  ParamMap pm;
  rc = make_param_map(qa, N, K, nullptr, &pm); if (rc) return rc;
  b.W = W; b.U = U; b.scale = scale; b.zp = zp; b.col_group = col_group; b.gscale = gscale; b.losses = losses;
  b.N = N; b.K = K; b.ldw = ldw; b.ldu = ldu;
  b.strategy = qa->strategy;
  b.group_size = (qa->strategy == B200Q_BLOCK) ? qa->block_w : qa->group_size;
  if (b.group_size <= 0) b.group_size = 1;
  b.block_h = qa->block_h > 0 ? qa->block_h : 1;
  b.zp_kind = qa->zp_kind;
  b.groups_per_row = pm.groups_per_row;
  void (*kern)(SweepBatch) = nullptr;
#define B200Q_SWEEP_PICK(SDT)                                                                              \
  do {                                                                                                     \
    if (b.qr.kind == kInt) kern = gscale ? sweep_fused_kernel<SDT, true, kInt> : sweep_fused_kernel<SDT, false, kInt>;      \
    else if (b.qr.kind == kFp8) kern = gscale ? sweep_fused_kernel<SDT, true, kFp8> : sweep_fused_kernel<SDT, false, kFp8>; \
    else kern = gscale ? sweep_fused_kernel<SDT, true, kFp4> : sweep_fused_kernel<SDT, false, kFp4>;       \
  } while (0)
  if (sdtype == B200Q_BF16) B200Q_SWEEP_PICK(B200Q_BF16);
  else if (sdtype == B200Q_F32) B200Q_SWEEP_PICK(B200Q_F32);
  else return B200Q_ERR_UNSUPPORTED;
#undef B200Q_SWEEP_PICK
  B200Q_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sweep_smem_bytes()));
  dim3 grid((unsigned)((N + kRows - 1) / kRows), (unsigned)count, 1);
  kern<<<grid, kThreads, sweep_smem_bytes(), (cudaStream_t)stream>>>(b);
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

}  // extern "C"
