// fp32-accurate tile GEMM on the tensor cores (tcgen05, kind::tf32, "3xTF32").
//
//   C[M,N] = beta * C + alpha * A[M,Kd] * B[N,Kd]^T,   Kd <= 128 (the GPTQ block width)
//
// Each float32 operand x is given as two tf32-exact arrays hi = tf32(x), lo = tf32(x - hi)
// (split_kernel; split_transposed_kernel for an operand stored [Kd][N]); every k-step issues three
// MMAs into one TMEM accumulator, hi*hi + hi*lo + lo*hi, which keeps ~22 significant bits per
// product with float32 accumulation: as accurate as the SIMT float32 GEMM it replaces for the
// factorisation and the sweep's trailing updates, at tensor-core speed.
//
// Structure: persistent CTAs, each with a contiguous range of the row-major tile list.  Warp 0 =
// TMA producer: the A operand of a block row (all k-chunks, hi and lo, 128 KiB) is loaded once and
// stays in shared memory while the tiles of that row are computed; B chunks (hi, lo of 32 k-values,
// 32 KiB) stream through a two-stage ring; the C tile is prefetched into L2.  Warp 1 = MMA issuer
// and TMEM owner (two 128-column accumulators).  Warps 2-9 = epilogue: the loads of the old C
// values are issued before the wait for the accumulator, tcgen05.ld, a transpose through a
// per-warp shared-memory tile so that every global access is a row-contiguous float4, alpha /
// beta, bounds.  Tile sets: all, lower block triangle, and the sets of the one-pass factorisation
// (see tgemm_tf32.cuh).  All mbarrier waits are bounded; no cluster launch, no multicast.
#include <cuda.h>

#include <cstdlib>
#include <mutex>

#include "common.cuh"
#include "tgemm_tf32.cuh"

namespace b200q {
namespace tgemm {

constexpr int kTile = 128;          // output tile is 128 x 128
constexpr int kChunkK = 32;         // fp32 elements per 128-byte row
constexpr int kOpBytes = kTile * kChunkK * 4;    // one hi or lo part of one 32-deep k-chunk: 16 KiB
constexpr int kMaxChunks = 4;                     // Kd <= 128
constexpr int kABytes = kMaxChunks * 2 * kOpBytes;   // resident A operand: 4 chunks x (hi, lo) = 128 KiB
constexpr int kStages = 2;                        // ring of B chunks
constexpr int kStageBytes = 2 * kOpBytes;         // B_hi, B_lo of one chunk: 32 KiB
constexpr int kEpiWarps = 8;                      // two warps per TMEM lane quarter, two column chunks each
constexpr int kEpiBytes = kEpiWarps * 32 * 33 * 4;   // per-warp staging tiles of the epilogue
constexpr int kOperandBytes = kABytes + kStages * kStageBytes;
constexpr int kSmemBytes = kOperandBytes + 1024 + 256 + kEpiBytes;
constexpr int kThreads = 64 + 32 * kEpiWarps;
constexpr int kTmemCols = 256;
constexpr long long kWaitCycles = 4000000000LL;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred P1;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P1, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, P1;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > kWaitCycles) { *abort_flag = 1; return false; }
  }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
// shared-memory matrix descriptor, 128-byte swizzle, descriptor version 1
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFFu);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// D fp32, A/B tf32, A K-major, B K-major (NT) or MN-major (NN), M = N = 128
__host__ __device__ constexpr uint32_t instr_desc(bool b_mn_major) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((b_mn_major ? 1u : 0u) << 16) |
         ((uint32_t)(kTile >> 3) << 17) | ((uint32_t)(kTile >> 4) << 24);
}

struct Params {
  float* C; int64_t ldc;
  int M, N, Kd;
  float alpha, beta;
  int tiles_m, tiles_n, mask;
  int skip;   // kSkipBlockTiles: index of the skipped column block
  int64_t num_tiles;
  int trans;
  int prefetch_c;
  int* status;
};

__device__ __forceinline__ void tile_from_index(const Params& p, int64_t t, int& tm, int& tn) {
  if (p.mask == kLowerTiles) {
    int i = (int)((sqrt(8.0 * (double)t + 1.0) - 1.0) * 0.5);
    while ((int64_t)i * (i + 1) / 2 > t) --i;
    while ((int64_t)(i + 1) * (i + 2) / 2 <= t) ++i;
    tm = i;
    tn = (int)(t - (int64_t)i * (i + 1) / 2);
  } else if (p.mask == kSkipBlockFirst) {
    if (t < p.skip) { tm = 0; tn = (int)t; }
    else if (t == p.skip) { tm = 0; tn = p.skip + 1; }
    else { tm = (int)(t - p.skip); tn = p.skip + 1; }
  } else if (p.mask == kSkipBlockRest) {
    const int64_t left = (int64_t)(p.tiles_m - 1) * p.skip;
    if (t < left) {
      tm = 1 + (int)(t / p.skip);
      tn = (int)(t - (int64_t)(tm - 1) * p.skip);
    } else {
      const int64_t u = t - left;
      int i = (int)((sqrt(8.0 * (double)u + 1.0) - 1.0) * 0.5);
      while ((int64_t)i * (i + 1) / 2 > u) --i;
      while ((int64_t)(i + 1) * (i + 2) / 2 <= u) ++i;
      tm = i + 1;
      tn = p.skip + 2 + (int)(u - (int64_t)i * (i + 1) / 2);
    }
  } else if (p.mask == kSkipBlockTiles) {
    const int64_t left = (int64_t)p.tiles_m * p.skip;
    if (t < left) {
      tm = (int)(t / p.skip);
      tn = (int)(t - (int64_t)tm * p.skip);
    } else {
      const int64_t u = t - left;
      int i = (int)((sqrt(8.0 * (double)u + 1.0) - 1.0) * 0.5);
      while ((int64_t)i * (i + 1) / 2 > u) --i;
      while ((int64_t)(i + 1) * (i + 2) / 2 <= u) ++i;
      tm = i;
      tn = p.skip + 1 + (int)(u - (int64_t)i * (i + 1) / 2);
    }
  } else {
    tm = (int)(t / p.tiles_n);
    tn = (int)(t - (int64_t)tm * p.tiles_n);
  }
}

__global__ void __launch_bounds__(kThreads, 1)
tgemm_kernel(const __grid_constant__ CUtensorMap a_hi, const __grid_constant__ CUtensorMap a_lo,
             const __grid_constant__ CUtensorMap b_hi, const __grid_constant__ CUtensorMap b_lo,
             const __grid_constant__ CUtensorMap c_map, Params p) {
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* aligned = smem_raw + (base - raw);
  uint64_t* bars = reinterpret_cast<uint64_t*>(aligned + kOperandBytes);
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (kStages + s); };
  auto accf_bar = [&](int b) { return bar0 + 8u * (2 * kStages + b); };
  auto acce_bar = [&](int b) { return bar0 + 8u * (2 * kStages + 2 + b); };
  const uint32_t afull_bar = bar0 + 8u * (2 * kStages + 4), aempty_bar = bar0 + 8u * (2 * kStages + 5);
  const uint32_t b_base = base + kABytes;   // ring of B chunks behind the resident A operand
  __shared__ uint32_t s_tmem_base;
  __shared__ volatile int s_abort;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(accf_bar(b), 1); mbar_init(acce_bar(b), kEpiWarps); }
    mbar_init(afull_bar, 1); mbar_init(aempty_bar, 1);
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)),
                 "r"((uint32_t)kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = s_tmem_base;
  const int chunks = (p.Kd + kChunkK - 1) / kChunkK;
  // Every CTA takes a contiguous range of the tile list.  The list is row-major, so consecutive
  // tiles of a CTA mostly share their block row: the A operand of a block row (all k-chunks, hi
  // and lo) is loaded once and stays in shared memory while only B chunks stream through the ring.
  const int64_t t_begin = p.num_tiles * blockIdx.x / gridDim.x;
  const int64_t t_end = p.num_tiles * (blockIdx.x + 1) / gridDim.x;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0, a_par = 0;
      int cur_tm = -1;
      bool ok = true;
      for (int64_t t = t_begin; t < t_end && ok; ++t) {
        int tm, tn;
        tile_from_index(p, t, tm, tn);
        if (p.prefetch_c) {
          // pull the C tile into L2 while this tile's operands stream in: the epilogue's
          // read-modify-write then meets L2 latency instead of HBM latency
#pragma unroll
          for (int q = 0; q < 4; ++q)
            asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(&c_map),
                         "r"(tn * kTile + q * 32), "r"(tm * kTile) : "memory");
        }
        if (tm != cur_tm) {
          if (cur_tm >= 0) {   // the MMAs of the previous block row have read A
            if (!mbar_wait(aempty_bar, a_par, &s_abort)) { ok = false; break; }
            a_par ^= 1u;
          }
          cur_tm = tm;
          mbar_expect_tx(afull_bar, (uint32_t)(chunks * 2 * kOpBytes));
          for (int c = 0; c < chunks; ++c) {
            // A parts: box [32 k][128 rows] at (k, row)
            tma_load_2d(base + (c * 2) * kOpBytes, &a_hi, afull_bar, c * kChunkK, tm * kTile);
            tma_load_2d(base + (c * 2 + 1) * kOpBytes, &a_lo, afull_bar, c * kChunkK, tm * kTile);
          }
        }
        for (int c = 0; c < chunks; ++c) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, &s_abort)) { ok = false; break; }
          mbar_expect_tx(full_bar(stage), kStageBytes);
          const uint32_t sb = b_base + stage * kStageBytes;
          tma_load_2d(sb, &b_hi, full_bar(stage), c * kChunkK, tn * kTile);
          tma_load_2d(sb + kOpBytes, &b_lo, full_bar(stage), c * kChunkK, tn * kTile);
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    int stage = 0;
    uint32_t phase = 0, a_par = 0;
    int local = 0, cur_tm = -1;
    bool ok = true;
    const uint32_t idesc = instr_desc(false);
    for (int64_t t = t_begin; t < t_end && ok; ++t, ++local) {
      int tm, tn, next_tm = -1, next_tn;
      tile_from_index(p, t, tm, tn);
      if (t + 1 < t_end) tile_from_index(p, t + 1, next_tm, next_tn);
      const int buf = local & 1;
      const uint32_t acc_phase = (uint32_t)((local >> 1) & 1);
      if (!mbar_wait(acce_bar(buf), acc_phase ^ 1u, &s_abort)) { ok = false; break; }
      if (tm != cur_tm) {
        if (!mbar_wait(afull_bar, a_par, &s_abort)) { ok = false; break; }
        a_par ^= 1u;
        cur_tm = tm;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t d_tmem = tmem_base + (uint32_t)(buf * kTile);
      for (int c = 0; c < chunks; ++c) {
        if (!mbar_wait(full_bar(stage), phase, &s_abort)) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (lane == 0) {
          const uint32_t sa = base + (c * 2) * kOpBytes;
          const uint32_t sb = b_base + stage * kStageBytes;
#pragma unroll
          for (int kk = 0; kk < kChunkK / 8; ++kk) {
            // K-major, 128-byte rows: 8-row groups 1024 bytes apart; a k-step of 8 tf32 is 32 bytes
            const uint64_t ah = make_desc(sa + kk * 32, 16, 1024);
            const uint64_t al = make_desc(sa + kOpBytes + kk * 32, 16, 1024);
            const uint64_t bh = make_desc(sb + kk * 32, 16, 1024);
            const uint64_t bl = make_desc(sb + kOpBytes + kk * 32, 16, 1024);
            mma_tf32(d_tmem, ah, bh, idesc, (c | kk) ? 1u : 0u);
            mma_tf32(d_tmem, ah, bl, idesc, 1u);
            mma_tf32(d_tmem, al, bh, idesc, 1u);
          }
          tc_commit(empty_bar(stage));
          if (c == chunks - 1) {
            tc_commit(accf_bar(buf));
            if (next_tm >= 0 && next_tm != tm) tc_commit(aempty_bar);   // A may be replaced
          }
        }
        __syncwarp();
        if (++stage == kStages) { stage = 0; phase ^= 1u; }
      }
    }
  } else {
    const int q = warp & 3;
    int local = 0;
    bool ok = true;
    const bool vec = ((p.ldc & 3) == 0) && ((((uintptr_t)p.C) & 15) == 0);
    // per-warp staging tile [32 rows][33]: accumulator rows come out of TMEM one row per lane;
    // going through shared memory lets every global access cover whole 128-byte row segments
    float* stage = reinterpret_cast<float*>(aligned + kOperandBytes + 256) + (warp - 2) * (32 * 33);
    const int sub_row = lane >> 3, sub_col = (lane & 7) * 4;  // 4 rows x 8 float4 per instruction
    for (int64_t t = t_begin; t < t_end && ok; ++t, ++local) {
      int tm, tn;
      tile_from_index(p, t, tm, tn);
      const int buf = local & 1;
      const uint32_t acc_phase = (uint32_t)((local >> 1) & 1);
      const int row0 = tm * kTile + q * 32;
      // warps 2-5 take column chunks 0 and 1, warps 6-9 chunks 2 and 3
      const int c_first = (warp - 2) >= 4 ? 2 : 0;
      // the old values of C do not depend on the accumulator: their loads go out before the wait
      // for the MMAs, so that memory latency and tensor-core time overlap
      float4 h[2][8];
      bool fast[2];
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int col0 = tn * kTile + (c_first + k) * 32;
        fast[k] = vec && col0 + 31 < p.N;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int row = row0 + i * 4 + sub_row;
          h[k][i] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (fast[k] && p.beta != 0.0f && row < p.M)
            h[k][i] = *reinterpret_cast<const float4*>(p.C + (int64_t)row * p.ldc + col0 + sub_col);
        }
      }
      if (!mbar_wait(accf_bar(buf), acc_phase, &s_abort)) { ok = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int c = c_first + k;
        const int col0 = tn * kTile + c * 32;
        if (col0 >= p.N) break;
        uint32_t r[32];
        tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * kTile + c * 32), r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int j = 0; j < 32; ++j) stage[lane * 33 + j] = __uint_as_float(r[j]) * p.alpha;
        __syncwarp();
        const int cc = col0 + sub_col;
        if (fast[k]) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int lr = i * 4 + sub_row, row = row0 + lr;
            if (row < p.M) {
              const float* sp = stage + lr * 33 + sub_col;
              float4 o;
              o.x = p.beta * h[k][i].x + sp[0]; o.y = p.beta * h[k][i].y + sp[1];
              o.z = p.beta * h[k][i].z + sp[2]; o.w = p.beta * h[k][i].w + sp[3];
              *reinterpret_cast<float4*>(p.C + (int64_t)row * p.ldc + cc) = o;
            }
          }
        } else {
          for (int i = 0; i < 8; ++i) {
            const int lr = i * 4 + sub_row, row = row0 + lr;
            if (row >= p.M) continue;
            for (int j = 0; j < 4; ++j)
              if (cc + j < p.N) {
                float* d = p.C + (int64_t)row * p.ldc + cc + j;
                const float old = (p.beta != 0.0f) ? *d : 0.0f;
                *d = p.beta * old + stage[lr * 33 + sub_col + j];
              }
          }
        }
        __syncwarp();
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(acce_bar(buf));
    }
  }

  if (s_abort) {
    if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, B200Q_ERR_DEVICE);
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) __nanosleep(1000);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)kTmemCols)
                 : "memory");
  }
}

// hi = tf32(x) (round to nearest even on 10 mantissa bits), lo = tf32(x - hi); both stored as
// float32 words whose low 13 mantissa bits are zero.  dst rows are zero-padded to ld_dst.
__global__ void split_kernel(const float* __restrict__ src, int64_t ld_src, int rows, int cols,
                             float* __restrict__ hi, float* __restrict__ lo, int64_t ld_dst) {
  const int64_t total = (int64_t)rows * ld_dst;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / ld_dst, c = i - r * ld_dst;
    float h = 0.0f, l = 0.0f;
    if (c < cols) {
      const float x = src[r * ld_src + c];
      h = tf32_rn(x);
      l = tf32_rn(x - h);
    }
    hi[i] = h;
    lo[i] = l;
  }
}

// Transposing variant: src is [rows][cols]; hi/lo are [cols][ld_dst] (row c holds src[:, c]),
// zero-padded to ld_dst.  Turns a [Kd][N] operand into the K-major [N][Kd] form the MMA reads.
__global__ void __launch_bounds__(256) split_transposed_kernel(const float* __restrict__ src, int64_t ld_src,
                                                                      int rows, int cols, float* __restrict__ hi,
                                                                      float* __restrict__ lo, int64_t ld_dst) {
  __shared__ float tile[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  const int tiles_c = (cols + 31) / 32, tiles_r = (int)(ld_dst / 32);
  for (int64_t t = blockIdx.x; t < (int64_t)tiles_c * tiles_r; t += gridDim.x) {
    const int tc = (int)(t % tiles_c), tr = (int)(t / tiles_c);
    for (int r = ty; r < 32; r += 8) {
      const int gr = tr * 32 + r, gc = tc * 32 + tx;
      tile[r][tx] = (gr < rows && gc < cols) ? src[(int64_t)gr * ld_src + gc] : 0.0f;
    }
    __syncthreads();
    for (int c = ty; c < 32; c += 8) {
      const int gc = tc * 32 + c, gr = tr * 32 + tx;  // output row = source column
      if (gc < cols) {
        const float x = tile[tx][c];
        const float h = tf32_rn(x);
        hi[(int64_t)gc * ld_dst + gr] = h;
        lo[(int64_t)gc * ld_dst + gr] = tf32_rn(x - h);
      }
    }
    __syncthreads();
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
inline EncodeTiledFn encode_fn() {
  // function-local static: initialised once, thread-safely (several host threads start solving at
  // the same moment)
  static const EncodeTiledFn fn = [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      return (EncodeTiledFn)sym;
    return (EncodeTiledFn) nullptr;
  }();
  return fn;
}
// fp32 matrix [rows][cols] (cols contiguous, ld elements per row), boxes of [box_rows][32 cols]
inline bool make_map(CUtensorMap* m, const float* base, int64_t rows, int64_t cols, int64_t ld, int box_rows) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return false;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 4};
  cuuint32_t box[2] = {32u, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  return enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// src [rows][cols] -> hi/lo [rows][split_ld(cols)]
int split(const float* src, int64_t ld_src, int rows, int cols, float* hi, float* lo, cudaStream_t st) {
  if (rows <= 0 || cols <= 0) return B200Q_OK;
  const int64_t ld = split_ld(cols);
  split_kernel<<<grid_for(((int64_t)rows * ld + 255) / 256, 8), 256, 0, st>>>(src, ld_src, rows, cols, hi, lo, ld);
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

// src [rows][cols] -> hi/lo [cols][split_ld(rows)]
int split_transposed(const float* src, int64_t ld_src, int rows, int cols, float* hi, float* lo,
                            cudaStream_t st) {
  if (rows <= 0 || cols <= 0) return B200Q_OK;
  const int64_t ld = split_ld(rows);
  const int64_t tiles = (int64_t)((cols + 31) / 32) * (ld / 32);
  split_transposed_kernel<<<grid_for(tiles, 8), 256, 0, st>>>(src, ld_src, rows, cols, hi, lo, ld);
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

// Tensor maps are cached per (array, leading dimension): a map covers the whole capacity of a
// split buffer (rows up to 2^30, OOB rows never exist), so one encode serves every launch that
// reads that buffer.  Rows beyond the operand's extent hold stale values; they only reach output
// rows / columns that the epilogue masks.  Columns beyond Kd are zero (the split pads them).
struct MapKey { const float* base; int64_t ld; };
struct MapCache {
  static constexpr int kSlots = 16;
  MapKey key[kSlots];
  CUtensorMap map[kSlots];
  int used = 0, next = 0;
  // Copies the map out: a later get() may evict the slot it came from.
  bool get(const float* base, int64_t ld, CUtensorMap* out) {
    for (int i = 0; i < used; ++i)
      if (key[i].base == base && key[i].ld == ld) { *out = map[i]; return true; }
    int slot = (used < kSlots) ? used++ : (next++ % kSlots);
    key[slot] = MapKey{nullptr, 0};
    if (!make_map(&map[slot], base, (int64_t)1 << 30, ld, ld, kTile)) return false;
    key[slot] = MapKey{base, ld};
    *out = map[slot];
    return true;
  }
};
inline MapCache& map_cache() {
  static thread_local MapCache c;
  return c;
}

// A: [M][Kd] split;  B: [N][Kd] split (K-major; [Kd][N] operands go through split_transposed).
int launch(int trans, Split A, Split B, float* C, int64_t ldc, int M, int N, int Kd, float alpha, float beta,
           int mask, int* status, cudaStream_t st, int mask_arg, int max_ctas) {
  if (M <= 0 || N <= 0 || Kd <= 0) return B200Q_OK;
  if (mask == kSkipBlockRest && M <= kTile) return B200Q_OK;   // a single row block has no rest
  if (Kd > 128 || (A.ld & 31) || (B.ld & 31) || A.ld < Kd || B.ld < Kd) return B200Q_ERR_ARG;
  if (trans != kNT) return B200Q_ERR_UNSUPPORTED;
  MapCache& mc = map_cache();
  CUtensorMap mah, mal, mbh, mbl;
  if (!mc.get(A.hi, A.ld, &mah) || !mc.get(A.lo, A.ld, &mal) || !mc.get(B.hi, B.ld, &mbh) ||
      !mc.get(B.lo, B.ld, &mbl)) {
    set_last_error("cuTensorMapEncodeTiled (tgemm)", cudaErrorInvalidValue);
    return B200Q_ERR_CUDA;
  }
  Params p;
  p.C = C; p.ldc = ldc; p.M = M; p.N = N; p.Kd = Kd; p.alpha = alpha; p.beta = beta; p.mask = mask; p.trans = trans;
  p.tiles_m = (M + kTile - 1) / kTile; p.tiles_n = (N + kTile - 1) / kTile;
  p.skip = mask_arg;
  p.num_tiles = (mask == kLowerTiles) ? (int64_t)p.tiles_m * (p.tiles_m + 1) / 2
              : (mask == kSkipBlockTiles) ? (int64_t)p.tiles_m * mask_arg + (int64_t)p.tiles_m * (p.tiles_m + 1) / 2
              : (mask == kSkipBlockFirst) ? (int64_t)mask_arg + p.tiles_m
              : (mask == kSkipBlockRest) ? (int64_t)(p.tiles_m - 1) * mask_arg + (int64_t)p.tiles_m * (p.tiles_m - 1) / 2
              : (int64_t)p.tiles_m * p.tiles_n;
  p.status = status;
  static thread_local int attr_device = -1;
  int dev = 0;
  B200Q_TRY(cudaGetDevice(&dev));
  if (attr_device != dev) {
    B200Q_TRY(cudaFuncSetAttribute(tgemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    attr_device = dev;
  }
  // map of C for the L2 prefetch (needs 16-byte aligned rows); any valid map when unused
  CUtensorMap mc_c = mah;
  p.prefetch_c = 0;
  if (beta != 0.0f && (ldc & 3) == 0 && (((uintptr_t)C) & 15) == 0 &&
      make_map(&mc_c, C, M, N, ldc, kTile))
    p.prefetch_c = 1;
  int grid = (int)(p.num_tiles < kNumSMs ? p.num_tiles : kNumSMs);
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  tgemm_kernel<<<grid, kThreads, kSmemBytes, st>>>(mah, mal, mbh, mbl, mc_c, p);
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int side_reserve() {
  static const int r = [] {
    const char* e = getenv("B200Q_SIDE_RESERVE");
    int v = e ? atoi(e) : 16;   // measured best for K = 14336 among 0 / 16 / 32 / 48
    return v < 0 ? 0 : (v > kNumSMs / 2 ? kNumSMs / 2 : v);
  }();
  return r;
}

SideStream* side_stream(cudaStream_t like) {
  // one helper per (device, caller stream), kept for the life of the process: host threads come
  // and go, the streams they launch on do not
  struct Entry { int device; cudaStream_t like; SideStream s; };
  constexpr int kMax = 64;
  static Entry entries[kMax];
  static int used = 0;
  static std::mutex mu;
  int dev = 0, prio = 0;
  static const bool enabled = [] { const char* e = getenv("B200Q_LOOKAHEAD"); return !(e && e[0] == '0'); }();
  if (!enabled) return nullptr;
  if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  for (int i = 0; i < used; ++i)
    if (entries[i].device == dev && entries[i].like == like) return &entries[i].s;
  if (used == kMax) return nullptr;
  if (cudaStreamGetPriority(like, &prio) != cudaSuccess) { (void)cudaGetLastError(); prio = 0; }
  Entry& e = entries[used];
  e.device = dev; e.like = like;
  if (cudaStreamCreateWithPriority(&e.s.stream, cudaStreamNonBlocking, prio) != cudaSuccess ||
      cudaEventCreateWithFlags(&e.s.ready, cudaEventDisableTiming) != cudaSuccess ||
      cudaEventCreateWithFlags(&e.s.done, cudaEventDisableTiming) != cudaSuccess) {
    (void)cudaGetLastError();
    return nullptr;
  }
  ++used;
  return &e.s;
}

}  // namespace tgemm
}  // namespace b200q
