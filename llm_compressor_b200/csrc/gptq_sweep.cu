// GPTQ solve, part 2: the blockwise column sweep.
//
// Rows of W are independent, so they are spread over lanes: a warp owns 32 rows of the current
// 128-column block and each lane sweeps its own row (see sweep_block_kernel).  The 128x128
// diagonal block of U sits in shared memory.  The quantisation error of the block goes to a
// [N,128] scratch panel and the update of all later columns is one fp32-accurate tensor-core
// tile GEMM  W[:, after] -= Err * U[block, after].
//
// Rounding follows the reference's sequence of separate float32 operations (product, then
// subtraction; true divisions), so that the propagated errors agree.
#include <cstdlib>

#include "common.cuh"
#include "tgemm_tf32.cuh"

namespace b200q {
namespace sweep {

constexpr int kMaxBlock = 128;
constexpr size_t kSweepHeaderBytes = 256;   // status word at the start of the workspace

struct Params {
  float* W; int64_t ldw; int64_t N; int64_t K;
  const float* U; int64_t ldu;
  const void* scale; const void* zp; const int32_t* col_group; const float* gscale;
  int strategy, group_size, block_h, zp_kind;
  int64_t groups_per_row;
  QRange qr;
  float* err_hi; float* err_lo; int64_t lde;   // the block's errors [N, lde] as the hi / lo operand split of the
                                               // trailing update's tile products (null: no trailing update)
  float* losses;
  int i1, bs;                // block start and width (<= 128)
  int first;                 // first block: losses are overwritten
};

// SB: scale tensor is bf16 (and no global scale) -> dequantised value rounded to bf16.
//
// Lane-per-row version.  A warp owns 32 rows; lane r keeps row r of the current 16-column
// sub-block in registers, so the quantisation of a column is done once per row (not once per
// lane) and the rank-1 corrections inside the sub-block are plain register arithmetic with the
// row of U broadcast from shared memory.  The other columns of the 128-column block sit in a
// shared-memory tile (column-major, one word per row and column: lanes hit distinct banks) and
// take the 16 corrections of a finished sub-block in one pass, column by column, in the same
// order of operations as the column-at-a-time formulation (product, then subtraction), so the
// results are bit-identical to it.
constexpr int kMaxWarps = 8;      // warps of a CTA that own row batches
constexpr int kCtaThreads = 256;  // all threads help with the loads of the U block
constexpr int kSub = 16;          // columns kept in registers at a time (code size grows with its square)

__host__ __device__ inline size_t sweep_smem_bytes(int warps) {
  return ((size_t)kMaxBlock * kMaxBlock + (size_t)kMaxBlock * (32 * warps + 1) + 64) * sizeof(float);
}

// KIND: the code type (CodeKind), a compile-time constant so that the quantisation of a column - the
// critical path of the whole sweep - is a short inline sequence without dispatch.
template <int SDT, bool GLOBAL, int KIND>
__global__ void __launch_bounds__(kCtaThreads) sweep_block_kernel(Params p, int warps) {
  constexpr bool SB = Elem<SDT>::is_bf16 && !GLOBAL;
  const float qmin = p.qr.qmin, qmax = p.qr.qmax;
  extern __shared__ float sm[];
  const int WLD = 32 * warps + 1;
  float* sU = sm;                                   // [128][128] row i, local column c (identity when U is null)
  float* sW = sU + kMaxBlock * kMaxBlock;           // [128][WLD] column c, row slot
  __shared__ float s_rd[kMaxBlock];                 // 1 / U[i][i]
  __shared__ int s_grp[kMaxBlock];                  // parameter column (group / block column) of each column
  __shared__ int s_same[kMaxBlock / kSub];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bs = p.bs;
  // U block (only c >= r is ever read): 16-byte loads when the layout allows, several in flight
  {
    const bool vec = p.U && ((p.ldu & 3) == 0) && ((((uintptr_t)p.U) & 15) == 0) && ((p.i1 & 3) == 0);
    constexpr int kQuads = kMaxBlock * kMaxBlock / 4;
#pragma unroll 4
    for (int idx = threadIdx.x; idx < kQuads; idx += blockDim.x) {
      const int r = idx >> 5, c = (idx & 31) << 2;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (r < bs && c + 3 >= r) {
        if (!p.U) {
          v.x = (r == c) ? 1.0f : 0.0f; v.y = (r == c + 1) ? 1.0f : 0.0f;
          v.z = (r == c + 2) ? 1.0f : 0.0f; v.w = (r == c + 3) ? 1.0f : 0.0f;
        } else {
          const float* src = p.U + (int64_t)(p.i1 + r) * p.ldu + (p.i1 + c);
          if (vec && c + 3 < bs) {
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
  }
  for (int i = threadIdx.x; i < kMaxBlock; i += blockDim.x) {
    float d = 1.0f;
    int grp = 0;
    if (i < bs) {
      if (p.U) d = p.U[(int64_t)(p.i1 + i) * p.ldu + (p.i1 + i)];
      const int col = p.i1 + i;
      grp = (p.strategy == B200Q_TENSOR || p.strategy == B200Q_CHANNEL)
                ? 0 : (p.col_group ? p.col_group[col] : col / p.group_size);
    }
    s_rd[i] = __frcp_rn(d);
    s_grp[i] = grp;
  }
  __syncthreads();
  if (threadIdx.x < kMaxBlock / kSub) {   // does one (scale, zero point) govern the whole sub-block?
    bool same = true;
    for (int t = 1; t < kSub; ++t) same = same && s_grp[threadIdx.x * kSub + t] == s_grp[threadIdx.x * kSub];
    s_same[threadIdx.x] = same ? 1 : 0;
  }
  __syncthreads();
  const float g = GLOBAL ? *p.gscale : 1.0f;
  const bool has_zp = p.zp != nullptr;
  float* myW = sW + warp * 32;   // this warp's 32 row slots
  const int64_t batches = (p.N + 31) / 32;
  if (warp >= warps) return;   // no CTA-wide barrier below this point

  for (int64_t batch = (int64_t)blockIdx.x * warps + warp; batch < batches; batch += (int64_t)gridDim.x * warps) {
    const int64_t row0 = batch * 32, row = row0 + lane;
    const bool live = row < p.N;
    // tile in: coalesced rows, transposed into the column-major tile
#pragma unroll 8
    for (int r = 0; r < 32; ++r) {
      const int64_t rr = row0 + r;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int c = lane + 32 * k;
        float v = 0.0f;
        if (rr < p.N && c < bs) v = p.W[rr * p.ldw + p.i1 + c];
        myW[c * WLD + r] = v;
      }
    }
    __syncwarp();
    int64_t pbase;
    switch (p.strategy) {
      case B200Q_TENSOR: pbase = 0; break;
      case B200Q_CHANNEL: pbase = row; break;
      case B200Q_BLOCK: pbase = (row / p.block_h) * p.groups_per_row; break;
      default: pbase = row * p.groups_per_row; break;
    }
    float loss = 0.0f;
    int cur_grp = -1;
    float s = 1.0f, z = 0.0f, rs = 1.0f;
#pragma unroll 1
    for (int sub = 0; sub * kSub < bs; ++sub) {
      const int c0 = sub * kSub;
      // Quantisation parameters of the sub-block's columns, fetched before the dependent chain
      // starts.  Columns at or beyond bs (the ragged last block) are zero columns with a unit
      // pivot and zero rows of U: they run through the same code and change nothing.
      float sv[kSub], rsv[kSub], zv[kSub];
      if (s_same[sub]) {   // uniform
        const int grp = s_grp[c0];
        if (grp != cur_grp) {
          cur_grp = grp;
          if (live) {
            const int64_t pi = pbase + grp;
            s = Elem<SDT>::load((const typename Elem<SDT>::type*)p.scale + pi);
            if (GLOBAL) s = __fdiv_rn(s, g);
            rs = __frcp_rn(s);
            if (has_zp) z = load_zp(p.zp, p.zp_kind, pi);
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
            st = Elem<SDT>::load((const typename Elem<SDT>::type*)p.scale + pi);
            if (GLOBAL) st = __fdiv_rn(st, g);
            if (has_zp) zt = load_zp(p.zp, p.zp_kind, pi);
          }
          sv[t] = st; rsv[t] = __frcp_rn(st); zv[t] = zt;
        }
      }
      float w[kSub], e[kSub], rd[kSub];
#pragma unroll
      for (int t = 0; t < kSub; ++t) { w[t] = myW[(c0 + t) * WLD + lane]; rd[t] = s_rd[c0 + t]; }
#pragma unroll
      for (int t = 0; t < kSub; ++t) {
        const int i = c0 + t;
        const float wi = w[t];
        const float q = fake_quant_f32<KIND, SB>(wi, sv[t], rsv[t], zv[t], qmin, qmax);
        const float diff = __fsub_rn(wi, q);
        // loss and error use the reciprocal of the pivot (an ulp from the reference's divisions)
        const float tt = __fmul_rn(diff, rd[t]);
        loss = fmaf(tt, tt, loss);
        e[t] = tt;
        w[t] = q;
        const float4* urow = reinterpret_cast<const float4*>(sU + i * kMaxBlock + c0);
#pragma unroll
        for (int k4 = (t + 1) / 4; k4 < kSub / 4; ++k4) {
          const float4 u = urow[k4];
          if (4 * k4 + 0 > t) w[4 * k4 + 0] = __fsub_rn(w[4 * k4 + 0], __fmul_rn(tt, u.x));
          if (4 * k4 + 1 > t) w[4 * k4 + 1] = __fsub_rn(w[4 * k4 + 1], __fmul_rn(tt, u.y));
          if (4 * k4 + 2 > t) w[4 * k4 + 2] = __fsub_rn(w[4 * k4 + 2], __fmul_rn(tt, u.z));
          if (4 * k4 + 3 > t) w[4 * k4 + 3] = __fsub_rn(w[4 * k4 + 3], __fmul_rn(tt, u.w));
        }
      }
      // quantised values back into the tile; the errors go straight to the panel the trailing
      // update reads: 16 consecutive floats per row
#pragma unroll
      for (int t = 0; t < kSub; ++t) myW[(c0 + t) * WLD + lane] = w[t];
      if (live && p.err_hi) {
        float4* dh = reinterpret_cast<float4*>(p.err_hi + row * p.lde + c0);
        float4* dl = reinterpret_cast<float4*>(p.err_lo + row * p.lde + c0);
#pragma unroll
        for (int t = 0; t < kSub; t += 4) {
          float h[4], l[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) { h[j] = tgemm::tf32_rn(e[t + j]); l[j] = tgemm::tf32_rn(e[t + j] - h[j]); }
          dh[t / 4] = make_float4(h[0], h[1], h[2], h[3]);
          dl[t / 4] = make_float4(l[0], l[1], l[2], l[3]);
        }
      }
      // the later columns of the block take this sub-block's corrections: v -= e * u as a packed
      // product and a packed sum with -e (two float32 lanes per instruction, each rounded like the
      // scalar operations)
      uint64_t ne2[kSub];
#pragma unroll
      for (int t = 0; t < kSub; ++t) asm("mov.b64 %0, {%1, %1};" : "=l"(ne2[t]) : "f"(-e[t]));
      // eight columns per pass: four independent chains of packed sums hide the latency of the adds
      // (the tile is 128 columns wide, so a ragged block's last pass stays inside it)
#pragma unroll 1
      for (int c = c0 + kSub; c < bs; c += 8) {
        uint64_t v[4];
#pragma unroll
        for (int h = 0; h < 4; ++h)
          asm("mov.b64 %0, {%1, %2};" : "=l"(v[h]) : "f"(myW[(c + 2 * h) * WLD + lane]), "f"(myW[(c + 2 * h + 1) * WLD + lane]));
#pragma unroll
        for (int t = 0; t < kSub; ++t) {
          const ulonglong2 ua = *reinterpret_cast<const ulonglong2*>(sU + (c0 + t) * kMaxBlock + c);
          const ulonglong2 ub = *reinterpret_cast<const ulonglong2*>(sU + (c0 + t) * kMaxBlock + c + 4);
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
          myW[(c + 2 * h) * WLD + lane] = lo; myW[(c + 2 * h + 1) * WLD + lane] = hi;
        }
      }
    }
    if (live && p.err_hi) {   // zero padding of the operand rows up to their leading dimension
      for (int c = (bs + kSub - 1) / kSub * kSub; c < (int)p.lde; c += 4) {
        *reinterpret_cast<float4*>(p.err_hi + row * p.lde + c) = make_float4(0.f, 0.f, 0.f, 0.f);
        *reinterpret_cast<float4*>(p.err_lo + row * p.lde + c) = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
    __syncwarp();
    // tile out
    for (int r = 0; r < 32; ++r) {
      const int64_t rr = row0 + r;
      if (rr >= p.N) break;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int c = lane + 32 * k;
        if (c < bs) p.W[rr * p.ldw + p.i1 + c] = myW[c * WLD + r];
      }
    }
    if (live) {
      const float half = loss * 0.5f;
      p.losses[row] = p.first ? half : p.losses[row] + half;
    }
    __syncwarp();
  }
}

}  // namespace sweep
}  // namespace b200q

using namespace b200q;

extern "C" {

size_t b200q_gptq_sweep_workspace_bytes(int64_t N, int64_t K, int blocksize) {
  using b200q::sweep::kSweepHeaderBytes;
  if (N <= 0 || K <= 0 || blocksize <= 0) return 0;
  // error panel [N][128] + two sets of (hi/lo copies of it, hi/lo copies of a 128-row panel of U):
  // consecutive blocks alternate between the sets because of the look-ahead
  const size_t np = (size_t)((N + 127) / 128 * 128), kp = (size_t)((K + 127) / 128 * 128);
  return kSweepHeaderBytes + (np * 128 * 5 + 4 * 128 * kp) * sizeof(float) + 64;
}

int b200q_gptq_sweep(float* Wf, int64_t N, int64_t K, int64_t ldf, const float* U, int64_t ldu, const void* scale,
                     int sdtype, const void* zp, const int32_t* col_group, const float* gscale,
                     const b200q_qargs* qa, int blocksize, float* losses, void* workspace, void* stream) {
  using namespace b200q::sweep;
  if (!Wf || !scale || !qa || !losses || !workspace || N <= 0 || K <= 0 || ldf < K) return B200Q_ERR_ARG;
  if (U && ldu < K) return B200Q_ERR_ARG;
  if (((uintptr_t)workspace) & 15) return B200Q_ERR_ARG;
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
  // header of the workspace: a status word that a bounded wait expiring inside one of the
  // trailing-update GEMMs sets to B200Q_ERR_DEVICE (cleared here, read by the caller afterwards)
  int* gemm_status = (int*)workspace;
  float* ws_f = (float*)((char*)workspace + kSweepHeaderBytes);
  p.err_hi = p.err_lo = nullptr;
  p.lde = tgemm::split_ld(blocksize);
  const size_t np128 = (size_t)((N + 127) / 128 * 128) * 128, kp128 = (size_t)((K + 127) / 128 * 128) * 128;
  float* sa_base = ws_f + np128;             // [2][hi, lo][np128]: the sweep kernel writes a block's errors here
  float* sb_base = sa_base + 4 * np128;      // [2][hi, lo][kp128]
  p.losses = losses;
  cudaStream_t st = (cudaStream_t)stream;
  B200Q_TRY(cudaMemsetAsync(gemm_status, 0, sizeof(int), st));
  // warps per CTA: one 32-row batch per warp; few rows -> small CTAs so that every SM gets work
  const int64_t batches = (N + 31) / 32;
  int warps = (int)((batches + kNumSMs - 1) / kNumSMs);
  warps = warps < 1 ? 1 : (warps > kMaxWarps ? kMaxWarps : warps);
  void (*kern)(Params, int) = nullptr;
#define B200Q_SWEEP_PICK(SDT)                                                                              \
  do {                                                                                                     \
    if (p.qr.kind == kInt) kern = gscale ? sweep_block_kernel<SDT, true, kInt> : sweep_block_kernel<SDT, false, kInt>;      \
    else if (p.qr.kind == kFp8) kern = gscale ? sweep_block_kernel<SDT, true, kFp8> : sweep_block_kernel<SDT, false, kFp8>; \
    else kern = gscale ? sweep_block_kernel<SDT, true, kFp4> : sweep_block_kernel<SDT, false, kFp4>;       \
  } while (0)
  if (sdtype == B200Q_BF16) B200Q_SWEEP_PICK(B200Q_BF16);
  else if (sdtype == B200Q_F32) B200Q_SWEEP_PICK(B200Q_F32);
  else return B200Q_ERR_UNSUPPORTED;
#undef B200Q_SWEEP_PICK
  // always the largest size: host threads on other streams launch the same kernel with other sizes
  B200Q_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)sweep_smem_bytes(kMaxWarps)));
  // With the look-ahead the far part of a trailing update runs beside the next block's sweep and
  // leaves `reserve` SMs to it: pack the row batches into that many CTAs when they fit (a warp is
  // latency-bound, several per SM cost little).
  tgemm::SideStream* side = U ? tgemm::side_stream(st) : nullptr;
  static const int kSweepReserve = [] {
    const char* e = getenv("B200Q_SWEEP_RESERVE");
    const int v = e ? atoi(e) : 32;
    return v < 8 ? 8 : (v > kNumSMs / 2 ? kNumSMs / 2 : v);
  }();
  int reserve = tgemm::side_reserve();
  if (side && batches <= (int64_t)kSweepReserve * kMaxWarps) {
    reserve = kSweepReserve;
    const int w = (int)((batches + reserve - 1) / reserve);
    if (w > warps) warps = w;
  }
  int64_t ctas = (batches + warps - 1) / warps;
  const int grid = (int)(ctas < 2 * kNumSMs ? ctas : 2 * kNumSMs);
  const size_t smem = sweep_smem_bytes(warps);
  // Look-ahead: the trailing update of a block is split in the next 128 columns (which the next
  // block's sweep reads; caller's stream) and the columns after them, which a helper stream
  // updates while the next block is swept.
  bool side_busy = false;
  int blk = 0;
  auto split_u = [&](int64_t j1, int which, cudaStream_t on) -> int {
    // hi / lo operand form of U[j1 : j1 + bs, j1 + bs :] (independent of the sweep: kept off its chain)
    const int bsj = (int)((K - j1) < blocksize ? (K - j1) : blocksize);
    const int64_t j2 = j1 + bsj;
    float* hi = sb_base + (size_t)which * 2 * kp128;
    return tgemm::split_transposed(U + j1 * ldu + j2, ldu, bsj, (int)(K - j2), hi, hi + kp128, on);
  };
  if (U && K > blocksize) { rc = split_u(0, 0, st); if (rc) return rc; }
  for (int64_t i1 = 0; i1 < K; i1 += blocksize, ++blk) {
    const int bs = (int)((K - i1) < blocksize ? (K - i1) : blocksize);
    const int64_t i2 = i1 + bs;
    const bool trailing = i2 < K && U;
    float* sa_hi = sa_base + (size_t)(blk & 1) * 2 * np128;
    float* sa_lo = sa_hi + np128;
    p.i1 = (int)i1; p.bs = bs; p.first = (i1 == 0);
    p.err_hi = trailing ? sa_hi : nullptr; p.err_lo = trailing ? sa_lo : nullptr;
    p.lde = tgemm::split_ld(bs);
    kern<<<grid, kCtaThreads, smem, st>>>(p, warps);
    B200Q_LAUNCH_CHECK();
    if (trailing) {
      // W[:, i2:] -= Err[N, bs] * U[i1:i2, i2:]   (3xTF32 on the tensor cores)
      const int rest = (int)(K - i2);
      float* sb_hi = sb_base + (size_t)(blk & 1) * 2 * kp128;
      float* sb_lo = sb_hi + kp128;
      const int64_t ld = tgemm::split_ld(bs);
      const tgemm::Split A{sa_hi, sa_lo, ld};
      const bool more = K - i2 > blocksize;     // the next block has a trailing update too
      if (!side) {
        rc = tgemm::launch(tgemm::kNT, A, tgemm::Split{sb_hi, sb_lo, ld}, Wf + i2, ldf, (int)N, rest, bs, -1.0f, 1.0f,
                           tgemm::kAllTiles, gemm_status, st);
        if (rc) return rc;
        if (more) { rc = split_u(i2, (blk + 1) & 1, st); if (rc) return rc; }
        continue;
      }
      const int near = rest < 128 ? rest : 128;
      B200Q_TRY(cudaEventRecord(side->ready, st));
      B200Q_TRY(cudaStreamWaitEvent(side->stream, side->ready, 0));
      // the far columns of the block before, and this block's operand form of U made behind them
      if (side_busy) B200Q_TRY(cudaStreamWaitEvent(st, side->done, 0));
      rc = tgemm::launch(tgemm::kNT, A, tgemm::Split{sb_hi, sb_lo, ld}, Wf + i2, ldf, (int)N, near, bs, -1.0f, 1.0f,
                         tgemm::kAllTiles, gemm_status, st);
      if (rc) return rc;
      if (rest > near) {
        rc = tgemm::launch(tgemm::kNT, A, tgemm::Split{sb_hi + (int64_t)near * ld, sb_lo + (int64_t)near * ld, ld},
                           Wf + i2 + near, ldf, (int)N, rest - near, bs, -1.0f, 1.0f, tgemm::kAllTiles, gemm_status,
                           side->stream, 0, kNumSMs - reserve);
        if (rc) return rc;
        // the next block's slice of U: its buffer was last read by the block before this one
        // (near part before `ready`, far part earlier on the helper stream)
        if (more) { rc = split_u(i2, (blk + 1) & 1, side->stream); if (rc) return rc; }
        B200Q_TRY(cudaEventRecord(side->done, side->stream));
        side_busy = true;
      } else if (more) {
        // no far part (blocks narrower than the 128 near columns): the helper stream is idle and
        // was waited for above, the slice is made on the caller's stream
        rc = split_u(i2, (blk + 1) & 1, st); if (rc) return rc;
      }
    }
  }
  if (side_busy) B200Q_TRY(cudaStreamWaitEvent(st, side->done, 0));
  return B200Q_OK;
}

}  // extern "C"
