// GPTQ Hessian accumulation as a symmetric rank-k update on the 5th-generation tensor cores.
//
//   H_lower += alpha * X^T X        X: [T, K] bf16 row-major, H: [K, K] fp32
//
// Two kernels.  syrk_pair_kernel (further down) is the one that runs: CTA pairs on 256 x 256
// tiles with tcgen05.mma.cta_group::2.  syrk_kernel, described next, is the single-CTA version
// it grew out of; it is used when a cluster of two cannot be launched or when
// B200Q_SYRK_SINGLE_CTA=1 asks for it (A/B measurements).
//
// Persistent, warp-specialised kernel, one CTA per SM:
//   warp 0      TMA producer: 64-token x 64-column boxes of X into a 4-stage shared-memory
//               ring (128-byte swizzle).  The contraction runs over tokens, so both operands
//               are "MN-major": the contiguous dimension of X is the M / N dimension.
//   warp 1      issues tcgen05.mma (M=128, N=256, K=16, bf16 in, fp32 accumulate in TMEM) and
//               owns the TMEM allocation (2 accumulators x 256 columns = all 512 columns).
//   warps 2-5   epilogue: tcgen05.ld the accumulator, scale by alpha, add into H.
// Work units are (128 x 256 tile on or below the diagonal) x (token split); with more than one
// split the epilogue adds with red.global (fp32 atomics), otherwise with plain load/add/store.
//
// Every wait on an mbarrier is bounded: on expiry the kernel records a status, lets copies in
// flight land, frees TMEM and returns.
#include <cuda.h>

#include <cstdlib>
#include <mutex>

#include <atomic>

#include "common.cuh"

namespace b200q {
namespace syrk {

constexpr int kTileM = 128;        // rows of H per tile
constexpr int kTileN = 256;        // columns of H per tile
constexpr int kBlockT = 64;        // tokens per pipeline stage
constexpr int kStages = 4;
constexpr int kChunk = 64;         // columns per TMA box (128 bytes of bf16)
constexpr int kChunkBytes = kChunk * kBlockT * 2;            // 8 KiB
constexpr int kABytes = (kTileM / kChunk) * kChunkBytes;     // 16 KiB
constexpr int kBBytes = (kTileN / kChunk) * kChunkBytes;     // 32 KiB
constexpr int kStageBytes = kABytes + kBBytes;               // 48 KiB
constexpr int kEpiBytes = 4 * 32 * 33 * 4;  // per-warp staging tiles of the epilogue
constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/ + kEpiBytes;
constexpr int kThreads = 192;
constexpr int kTmemCols = 512;
constexpr long long kWaitCycles = 4000000000LL;  // ~2 s at 2 GHz

// ---- PTX wrappers ------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
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
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false if the barrier did not flip in time or another role aborted.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int* status, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > kWaitCycles) {
      *abort_flag = 1;
      if (status) atomicCAS(status, 0, code);
      return false;
    }
  }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tcgen05_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
__device__ __forceinline__ void tcgen05_mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                                 uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void red_add_v4(float* p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c),
               "f"(d)
               : "memory");
}

// Shared-memory matrix descriptor for an MN-major operand stored as 64-column chunks of
// [tokens][64] bf16 rows (128 bytes) with the 128-byte swizzle:
//   leading byte offset = distance between 64-column chunks, stride byte offset = distance
//   between groups of 8 token rows (1024 bytes); version 1; layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFFu);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;  // descriptor version for sm_100
  d |= (uint64_t)2 << 61;  // SWIZZLE_128B
  return d;
}
// Instruction descriptor: D fp32, A and B bf16, both MN-major, M=128, N=256, dense.
constexpr uint32_t kInstrDesc = (1u << 4)                     // c_format = F32
                                | (1u << 7) | (1u << 10)      // a_format, b_format = BF16
                                | (1u << 15) | (1u << 16)     // a_major, b_major = MN
                                | ((uint32_t)(kTileN >> 3) << 17) | ((uint32_t)(kTileM >> 4) << 24);

// Tile list: block row bi (128 rows) pairs with 256-column blocks bj <= bi/2.
__device__ __forceinline__ void decode_tile(int idx, int& bi, int& bj) {
  int b = 0, cum = 0;
  while (true) {
    int cnt = (b >> 1) + 1;
    if (idx < cum + cnt) break;
    cum += cnt;
    ++b;
  }
  bi = b;
  bj = idx - cum;
}
inline int num_tiles(int nb) {  // nb = number of 128-row blocks
  int n = 0;
  for (int b = 0; b < nb; ++b) n += (b >> 1) + 1;
  return n;
}

struct Params {
  float* H;
  int64_t ldh;
  int K;
  int64_t T;
  int tiles;
  int nb;                    // block rows of the tile grid
  int splits;
  int64_t tokens_per_split;  // multiple of kBlockT
  int tile_major;            // pair kernel: a CTA pair takes whole tiles, all token splits of a tile one after
                             // the other, and adds them into H without atomics (bitwise reproducible)
  float alpha;
  int* status;
};

__global__ void __launch_bounds__(kThreads, 1)
syrk_kernel(const __grid_constant__ CUtensorMap xmap, Params p) {
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;  // stages need 1024-byte alignment (swizzle atom)
  unsigned char* aligned = smem_raw + (base - raw);
  uint64_t* bars = reinterpret_cast<uint64_t*>(aligned + kStages * kStageBytes);
  // barrier layout: full[kStages], empty[kStages], acc_full[2], acc_empty[2]
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (kStages + s); };
  auto accf_bar = [&](int b) { return bar0 + 8u * (2 * kStages + b); };
  auto acce_bar = [&](int b) { return bar0 + 8u * (2 * kStages + 2 + b); };
  __shared__ uint32_t s_tmem_base;
  __shared__ volatile int s_abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(accf_bar(b), 1); mbar_init(acce_bar(b), 4); }
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&s_tmem_base)),
                 "r"((uint32_t)kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = s_tmem_base;

  const int total_units = p.tiles * p.splits;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x) {
        int bi, bj;
        decode_tile(u % p.tiles, bi, bj);
        const int split = u / p.tiles;
        const int64_t t_begin = (int64_t)split * p.tokens_per_split;
        const int64_t t_end = min(p.T, t_begin + p.tokens_per_split);
        const int iters = (int)((t_end - t_begin + kBlockT - 1) / kBlockT);
        for (int it = 0; it < iters; ++it) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, &s_abort, p.status, 1)) { ok = false; break; }
          mbar_expect_tx(full_bar(stage), kStageBytes);
          const uint32_t sa = base + stage * kStageBytes;
          const int t0 = (int)(t_begin + (int64_t)it * kBlockT);
#pragma unroll
          for (int c = 0; c < kTileM / kChunk; ++c)
            tma_load_2d(sa + c * kChunkBytes, &xmap, full_bar(stage), bi * kTileM + c * kChunk, t0);
#pragma unroll
          for (int c = 0; c < kTileN / kChunk; ++c)
            tma_load_2d(sa + kABytes + c * kChunkBytes, &xmap, full_bar(stage),
                        bj * kTileN + c * kChunk, t0);
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    int stage = 0;
    uint32_t phase = 0;
    int local = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x, ++local) {
      const int split = u / p.tiles;
      const int64_t t_begin = (int64_t)split * p.tokens_per_split;
      const int64_t t_end = min(p.T, t_begin + p.tokens_per_split);
      const int iters = (int)((t_end - t_begin + kBlockT - 1) / kBlockT);
      if (iters <= 0) continue;
      const int buf = local & 1;
      const uint32_t acc_phase = (uint32_t)((local >> 1) & 1);
      if (!mbar_wait(acce_bar(buf), acc_phase ^ 1u, &s_abort, p.status, 2)) { ok = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t d_tmem = tmem_base + (uint32_t)(buf * kTileN);
      for (int it = 0; it < iters; ++it) {
        if (!mbar_wait(full_bar(stage), phase, &s_abort, p.status, 3)) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (lane == 0) {
          const uint32_t sa = base + stage * kStageBytes;
#pragma unroll
          for (int kk = 0; kk < kBlockT / 16; ++kk) {
            const uint64_t da = make_desc(sa + kk * 2048, kChunkBytes, 1024);
            const uint64_t db = make_desc(sa + kABytes + kk * 2048, kChunkBytes, 1024);
            tcgen05_mma_bf16(d_tmem, da, db, kInstrDesc, (it | kk) ? 1u : 0u);
          }
          tcgen05_commit(empty_bar(stage));  // frees the stage once these MMAs have read it
          if (it == iters - 1) tcgen05_commit(accf_bar(buf));
        }
        __syncwarp();
        if (++stage == kStages) { stage = 0; phase ^= 1u; }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    float* stage = reinterpret_cast<float*>(aligned + kStages * kStageBytes + 256) + (warp - 2) * (32 * 33);
    const int sub_row = lane >> 3, sub_col = (lane & 7) * 4;  // 4 rows x 8 float4 per instruction
    int local = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x, ++local) {
      int bi, bj;
      decode_tile(u % p.tiles, bi, bj);
      const int split = u / p.tiles;
      const int64_t t_begin = (int64_t)split * p.tokens_per_split;
      const int64_t t_end = min(p.T, t_begin + p.tokens_per_split);
      if (t_end <= t_begin) continue;
      const int buf = local & 1;
      const uint32_t acc_phase = (uint32_t)((local >> 1) & 1);
      if (!mbar_wait(accf_bar(buf), acc_phase, &s_abort, p.status, 4)) { ok = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int row0 = bi * kTileM + q * 32;
      const int col_base = bj * kTileN;
      const int row_blk_end = bi * kTileM + kTileM;  // columns >= this belong to the upper part
#pragma unroll 1
      for (int c = 0; c < kTileN / 32; ++c) {
        const int col0 = col_base + c * 32;
        if (col0 >= row_blk_end || col0 >= p.K) break;  // warp-uniform
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * kTileN + c * 32), r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        // TMEM hands out one accumulator row per lane; transposing the 32x32 chunk through shared
        // memory makes every global access a whole 128-byte row segment (8 lanes x 16 bytes)
#pragma unroll
        for (int j = 0; j < 32; ++j) stage[lane * 33 + j] = __uint_as_float(r[j]) * p.alpha;
        __syncwarp();
        const int cc = col0 + sub_col;
        if (cc < p.K) {  // K % 8 == 0, so a float4 is inside or outside as a whole
          if (p.splits > 1) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int lr = i * 4 + sub_row, row = row0 + lr;
              if (row < p.K) {
                const float* sp = stage + lr * 33 + sub_col;
                red_add_v4(p.H + (int64_t)row * p.ldh + cc, sp[0], sp[1], sp[2], sp[3]);
              }
            }
          } else {
            float4 h[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int row = row0 + i * 4 + sub_row;
              h[i] = make_float4(0.f, 0.f, 0.f, 0.f);
              if (row < p.K) h[i] = *reinterpret_cast<const float4*>(p.H + (int64_t)row * p.ldh + cc);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int lr = i * 4 + sub_row, row = row0 + lr;
              if (row < p.K) {
                const float* sp = stage + lr * 33 + sub_col;
                h[i].x += sp[0]; h[i].y += sp[1]; h[i].z += sp[2]; h[i].w += sp[3];
                *reinterpret_cast<float4*>(p.H + (int64_t)row * p.ldh + cc) = h[i];
              }
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

  // ---------------------------------------------------------------------- teardown
  if (s_abort) {
    // let TMA copies and MMAs already issued drain before shared memory and TMEM are given up
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) __nanosleep(1000);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"((uint32_t)kTmemCols)
                 : "memory");
  }
}

// =========================================================================================
// CTA-pair version: two CTAs on neighbouring SMs (a cluster of 2) share one 256 x 256 tile.
// One tcgen05.mma.cta_group::2 (M=256, N=256, K=16) is issued by the even CTA and runs on both
// SMs' tensor cores; each CTA stages only ITS 128 rows of A and ITS 128 columns of B, so every
// SM moves 8 KiB of operands through shared memory per MMA instead of 12 KiB and the ring
// holds 6 stages.  The accumulator rows of a CTA's half tile land in that CTA's own TMEM and
// its own epilogue warps add them into H.
//
// Barriers: full[stage] lives in the even CTA and counts the bytes of both CTAs' loads (each
// TMA names the even CTA's barrier); empty[stage] and acc_full[buf] exist in both CTAs and are
// signalled together by one tcgen05.commit; acc_empty[buf] lives in the even CTA and collects
// the eight epilogue warps of the pair.  Loads carry no multicast: every CTA fetches its own
// boxes.
constexpr int kPairTile = 256;
constexpr int kPairStages = 6;
constexpr int kPairHalfBytes = (128 / kChunk) * kChunkBytes;          // 16 KiB: 128 columns x 64 tokens
constexpr int kPairStageBytes = 2 * kPairHalfBytes;                   // A half + B half
constexpr int kPairSmemBytes = kPairStages * kPairStageBytes + 1024 + 256 + kEpiBytes;
constexpr uint32_t kPairInstrDesc = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | (1u << 16)
                                    | ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(addr), "r"(rank));
  return out;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load whose completion bytes go to a barrier that may live in the peer CTA of the pair
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster_addr,
                                                 int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}
// arrives on the barrier at this shared-memory offset in both CTAs of the pair once all MMAs
// issued so far have completed
__device__ __forceinline__ void tcgen05_commit_pair(uint32_t bar) {
  const uint16_t both = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(bar), "h"(both)
      : "memory");
}
__device__ __forceinline__ void tcgen05_mma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                                      uint32_t idesc, uint32_t accumulate) {
  const uint32_t z = 0;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(z)
      : "memory");
}

// Tile list of the pair kernel: 256-row block bi pairs with 256-column blocks bj <= bi.
// Order: bands of kBand block rows, column by column inside a band.  The ~74 tiles in flight
// then cover about kBand row panels and 74 / kBand column panels of X, which L2 holds, instead of
// one row panel and every column panel.
constexpr int kBand = 8;
__device__ __forceinline__ void decode_pair_tile(int idx, int nb, int& bi, int& bj) {
  int r0 = 0;
  while (true) {
    const int r1 = min(nb, r0 + kBand) - 1;            // last row of this band
    const int rows = r1 - r0 + 1;
    const int full = (r0 + 1) * rows;                  // columns 0..r0 hold every row of the band
    const int tri = rows * (rows - 1) / 2;             // columns r0+1..r1 hold the rows >= column
    if (idx < full) { bj = idx / rows; bi = r0 + idx - bj * rows; return; }
    if (idx < full + tri) {
      int rem = idx - full, c = r0 + 1;
      while (rem >= r1 - c + 1) { rem -= r1 - c + 1; ++c; }
      bj = c; bi = c + rem;
      return;
    }
    idx -= full + tri;
    r0 += kBand;
  }
}

// The i-th unit (tile, token split) of a CTA pair.  Default: units are dealt out round robin over
// all pairs, split-major (the splits of a tile land on different pairs and meet in H through
// atomics).  tile_major: a pair owns whole tiles.
__device__ __forceinline__ bool pair_unit(const Params& p, int pair, int num_pairs, int i, int& tile, int& split) {
  if (p.tile_major) {
    tile = pair + (i / p.splits) * num_pairs;
    split = i % p.splits;
    return tile < p.tiles;
  }
  const int u = pair + i * num_pairs;
  tile = u % p.tiles;
  split = u / p.tiles;
  return u < p.tiles * p.splits;
}

__global__ void __launch_bounds__(kThreads, 1)
syrk_pair_kernel(const __grid_constant__ CUtensorMap xmap, Params p) {
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* aligned = smem_raw + (base - raw);
  uint64_t* bars = reinterpret_cast<uint64_t*>(aligned + kPairStages * kPairStageBytes);
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (kPairStages + s); };
  auto accf_bar = [&](int b) { return bar0 + 8u * (2 * kPairStages + b); };
  auto acce_bar = [&](int b) { return bar0 + 8u * (2 * kPairStages + 2 + b); };
  __shared__ uint32_t s_tmem_base;
  __shared__ volatile int s_abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();       // 0: issues the MMAs, 1: its peer
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(accf_bar(b), 1); mbar_init(acce_bar(b), 8); }
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&s_tmem_base)),
                 "r"((uint32_t)kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();   // the peer's barriers are initialised before anything signals them
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = s_tmem_base;

  const int total_units = p.tiles * p.splits;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int tile, split;
      for (int i = 0; ok && pair_unit(p, pair, num_pairs, i, tile, split); ++i) {
        int bi, bj;
        decode_pair_tile(tile, p.nb, bi, bj);
        const int64_t t_begin = (int64_t)split * p.tokens_per_split;
        const int64_t t_end = min(p.T, t_begin + p.tokens_per_split);
        const int iters = (int)((t_end - t_begin + kBlockT - 1) / kBlockT);
        const int a_col = bi * kPairTile + (int)rank * 128, b_col = bj * kPairTile + (int)rank * 128;
        for (int it = 0; it < iters; ++it) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, &s_abort, p.status, 1)) { ok = false; break; }
          if (rank == 0) mbar_expect_tx(full_bar(stage), 2 * kPairStageBytes);
          const uint32_t full0 = map_to_cta(full_bar(stage), 0);
          const uint32_t sa = base + stage * kPairStageBytes;
          const int t0 = (int)(t_begin + (int64_t)it * kBlockT);
#pragma unroll
          for (int c = 0; c < 128 / kChunk; ++c) {
            tma_load_2d_pair(sa + c * kChunkBytes, &xmap, full0, a_col + c * kChunk, t0);
            tma_load_2d_pair(sa + kPairHalfBytes + c * kChunkBytes, &xmap, full0, b_col + c * kChunk, t0);
          }
          if (++stage == kPairStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (even CTA only)
    if (rank == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      int tile, split;
      for (; ok && pair_unit(p, pair, num_pairs, local, tile, split); ++local) {
        const int64_t t_begin = (int64_t)split * p.tokens_per_split;
        const int64_t t_end = min(p.T, t_begin + p.tokens_per_split);
        const int iters = (int)((t_end - t_begin + kBlockT - 1) / kBlockT);
        if (iters <= 0) continue;
        const int buf = local & 1;
        const uint32_t acc_phase = (uint32_t)((local >> 1) & 1);
        if (!mbar_wait(acce_bar(buf), acc_phase ^ 1u, &s_abort, p.status, 2)) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * kPairTile);
        for (int it = 0; it < iters; ++it) {
          if (!mbar_wait(full_bar(stage), phase, &s_abort, p.status, 3)) { ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          if (lane == 0) {
            const uint32_t sa = base + stage * kPairStageBytes;
#pragma unroll
            for (int kk = 0; kk < kBlockT / 16; ++kk) {
              const uint64_t da = make_desc(sa + kk * 2048, kChunkBytes, 1024);
              const uint64_t db = make_desc(sa + kPairHalfBytes + kk * 2048, kChunkBytes, 1024);
              tcgen05_mma_bf16_pair(d_tmem, da, db, kPairInstrDesc, (it | kk) ? 1u : 0u);
            }
            tcgen05_commit_pair(empty_bar(stage));
            if (it == iters - 1) tcgen05_commit_pair(accf_bar(buf));
          }
          __syncwarp();
          if (++stage == kPairStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
    const int q = warp & 3;
    float* stage = reinterpret_cast<float*>(aligned + kPairStages * kPairStageBytes + 256) + (warp - 2) * (32 * 33);
    const int sub_row = lane >> 3, sub_col = (lane & 7) * 4;
    int local = 0;
    bool ok = true;
    int tile, split;
    for (; ok && pair_unit(p, pair, num_pairs, local, tile, split); ++local) {
      int bi, bj;
      decode_pair_tile(tile, p.nb, bi, bj);
      const int64_t t_begin = (int64_t)split * p.tokens_per_split;
      const int64_t t_end = min(p.T, t_begin + p.tokens_per_split);
      if (t_end <= t_begin) continue;
      const int buf = local & 1;
      const uint32_t acc_phase = (uint32_t)((local >> 1) & 1);
      if (!mbar_wait(accf_bar(buf), acc_phase, &s_abort, p.status, 4)) { ok = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int row_blk = bi * kPairTile + (int)rank * 128;   // this CTA's 128 rows of the tile
      const int row0 = row_blk + q * 32;
      const int col_base = bj * kPairTile;
      const int row_blk_end = row_blk + 128;  // columns >= this belong to the upper part
#pragma unroll 1
      for (int c = 0; c < kPairTile / 32; ++c) {
        const int col0 = col_base + c * 32;
        if (col0 >= row_blk_end || col0 >= p.K || row_blk >= p.K) break;  // warp-uniform
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * kPairTile + c * 32), r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int j = 0; j < 32; ++j) stage[lane * 33 + j] = __uint_as_float(r[j]) * p.alpha;
        __syncwarp();
        const int cc = col0 + sub_col;
        if (cc < p.K) {
          if (p.splits > 1 && !p.tile_major) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int lr = i * 4 + sub_row, row = row0 + lr;
              if (row < p.K) {
                const float* sp = stage + lr * 33 + sub_col;
                red_add_v4(p.H + (int64_t)row * p.ldh + cc, sp[0], sp[1], sp[2], sp[3]);
              }
            }
          } else {
            float4 h[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int row = row0 + i * 4 + sub_row;
              h[i] = make_float4(0.f, 0.f, 0.f, 0.f);
              if (row < p.K) h[i] = *reinterpret_cast<const float4*>(p.H + (int64_t)row * p.ldh + cc);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int lr = i * 4 + sub_row, row = row0 + lr;
              if (row < p.K) {
                const float* sp = stage + lr * 33 + sub_col;
                h[i].x += sp[0]; h[i].y += sp[1]; h[i].z += sp[2]; h[i].w += sp[3];
                *reinterpret_cast<float4*>(p.H + (int64_t)row * p.ldh + cc) = h[i];
              }
            }
          }
        }
        __syncwarp();
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) {
        if (rank == 0) mbar_arrive(acce_bar(buf));
        else mbar_arrive_cluster(map_to_cta(acce_bar(buf), 0));
      }
    }
  }

  // ---------------------------------------------------------------------- teardown
  if (s_abort) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) __nanosleep(1000);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();   // neither CTA gives up shared memory or TMEM while the other may still use it
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"((uint32_t)kTmemCols)
                 : "memory");
  }
}

// H[i][j] = H[j][i] = scale * H[i][j] for j <= i, by 32x32 blocks through shared memory.
__global__ void __launch_bounds__(256) finalize_kernel(float* __restrict__ H, int64_t K, int64_t ldh,
                                                       float scale) {
  __shared__ float tile[32][33];
  const int nb = (int)((K + 31) / 32);
  const int64_t nblk = (int64_t)nb * (nb + 1) / 2;
  for (int64_t blk = blockIdx.x; blk < nblk; blk += gridDim.x) {
    // blk -> (bi >= bj)
    int bi = (int)((sqrt(8.0 * (double)blk + 1.0) - 1.0) * 0.5);
    while ((int64_t)bi * (bi + 1) / 2 > blk) --bi;
    while ((int64_t)(bi + 1) * (bi + 2) / 2 <= blk) ++bi;
    const int bj = (int)(blk - (int64_t)bi * (bi + 1) / 2);
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    for (int r = ty; r < 32; r += 8) {
      int64_t i = (int64_t)bi * 32 + r, j = (int64_t)bj * 32 + tx;
      float v = 0.0f;
      if (i < K && j < K) {
        v = H[i * ldh + j] * scale;
        if (bi != bj || j <= i) H[i * ldh + j] = v;
      }
      tile[r][tx] = v;
    }
    __syncthreads();
    for (int r = ty; r < 32; r += 8) {
      // element (j-block row r, i-block col tx) of the mirrored block
      int64_t j = (int64_t)bj * 32 + r, i = (int64_t)bi * 32 + tx;
      if (i < K && j < K && (bi != bj || j < i)) H[j * ldh + i] = tile[tx][r];
    }
    __syncthreads();
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
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

// Number of CTA pairs that can be resident at once on the current device (one CTA per SM), or 0
// when the pair kernel is switched off (B200Q_SYRK_SINGLE_CTA=1) or cannot be launched.
static int pair_capacity() {
  static std::mutex mu;
  static int cached[64];
  static bool have[64] = {false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  std::lock_guard<std::mutex> lock(mu);
  if (have[dev]) return cached[dev];
  int pairs = 0;
  const char* off = getenv("B200Q_SYRK_SINGLE_CTA");
  if (!(off && off[0] == '1')) {
    if (cudaFuncSetAttribute(syrk_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmemBytes) ==
        cudaSuccess) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(2 * kNumSMs, 1, 1);
      cfg.blockDim = dim3(kThreads, 1, 1);
      cfg.dynamicSmemBytes = kPairSmemBytes;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, syrk_pair_kernel, &cfg) == cudaSuccess && n > 0)
        pairs = n < kNumSMs / 2 ? n : kNumSMs / 2;
    }
    (void)cudaGetLastError();
  }
  cached[dev] = pairs;
  have[dev] = true;
  return pairs;
}

}  // namespace syrk
}  // namespace b200q

using namespace b200q;

// Token splits add their partial tiles with floating-point atomics, whose order varies from run to
// run (H then differs in its last bits).  With this flag set a CTA pair owns whole tiles and adds
// the token splits of a tile one after the other without atomics: bitwise reproducible, the
// accumulation chains bounded all the same, slower when the tiles alone do not fill the GPU.
static std::atomic<int> g_reproducible{0};

static int64_t max_chain_tokens() {
  static const int64_t v = [] {
    // default 8192 tokens: the float32 accumulation of the tensor cores drifts by about 3e-9 per
    // token (relative, one-sided), and a GPTQ solve at K = 14336 on a Hessian accumulated in chains
    // of 32768 tokens differed in 1.2 % of its codes from the solve on a float64-accumulated one;
    // at 8192 it is 0.2 %, at 2048 the 0.05 % that a float32 matmul accumulation gives
    const char* e = getenv("B200Q_SYRK_MAX_CHAIN");
    const long long x = e ? atoll(e) : 8192;
    return (int64_t)(x < 512 ? 512 : x);
  }();
  return v;
}

extern "C" {

int b200q_hessian_syrk(const void* X, int64_t T, int64_t K, int64_t ldx, float* H, int64_t ldh,
                       float alpha, int* status, void* stream) {
  using namespace b200q::syrk;
  if (!X || !H || T < 0 || K <= 0 || ldx < K || ldh < K) return B200Q_ERR_ARG;
  if (K % 8 || ldx % 8 || ((uintptr_t)X) % 16 || ((uintptr_t)H) % 16 || ldh % 4) return B200Q_ERR_ARG;
  if (T == 0) return B200Q_OK;
  if (K > (1 << 20) || T > (int64_t)2000000000) return B200Q_ERR_UNSUPPORTED;
  EncodeTiledFn encode = get_encode_fn();
  if (!encode) { set_last_error("cuTensorMapEncodeTiled entry point", cudaErrorUnknown); return B200Q_ERR_CUDA; }

  CUtensorMap map;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)T};
  cuuint64_t strides[1] = {(cuuint64_t)ldx * 2};
  cuuint32_t box[2] = {(cuuint32_t)kChunk, (cuuint32_t)kBlockT};
  cuuint32_t estr[2] = {1, 1};
  CUresult cr = encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(X), dims, strides, box,
                       estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                       CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (cr != CUDA_SUCCESS) { set_last_error("cuTensorMapEncodeTiled", cudaErrorInvalidValue); return B200Q_ERR_CUDA; }

  Params p;
  p.H = H; p.ldh = ldh; p.K = (int)K; p.T = T; p.alpha = alpha; p.status = status;
  p.tile_major = 0;
  cudaStream_t st = (cudaStream_t)stream;
  const int pairs = pair_capacity();
  if (pairs > 0) {
    // CTA pairs on 256 x 256 tiles
    const int nb2 = (int)((K + kPairTile - 1) / kPairTile);
    p.tiles = nb2 * (nb2 + 1) / 2;
    p.nb = nb2;
    const int64_t max_splits = (T + 511) / 512;
    int best = 1;
    double best_eff = 0.0;
    for (int s = 1; s <= (int)(max_splits < 64 ? max_splits : 64); ++s) {
      const int64_t units = (int64_t)p.tiles * s;
      const int64_t waves = (units + pairs - 1) / pairs;
      const double eff = (double)units / (double)(waves * pairs);
      if (eff > best_eff + 0.02) { best_eff = eff; best = s; }
    }
    {
      // bound the length of one tensor-core accumulation chain: its float32 error grows with it
      const int64_t need = (T + max_chain_tokens() - 1) / max_chain_tokens();
      if (best < need) best = (int)(need < 64 ? need : 64);
    }
    p.tile_major = g_reproducible.load(std::memory_order_relaxed) ? 1 : 0;
    if (p.tile_major) {
      // whole tiles per pair: the splits only bound the accumulation chains
      const int64_t need = (T + max_chain_tokens() - 1) / max_chain_tokens();
      best = (int)(need < 1 ? 1 : (need > 64 ? 64 : need));
    }
    p.splits = best;
    const int64_t tps = (T + p.splits - 1) / p.splits;
    p.tokens_per_split = ((tps + kBlockT - 1) / kBlockT) * kBlockT;
    // rounding the split length up can leave the last split empty; in tile-major order an empty
    // unit would sit between used ones and upset the alternation of the two accumulators
    if (p.tile_major) p.splits = (int)((T + p.tokens_per_split - 1) / p.tokens_per_split);
    const int64_t units = p.tile_major ? (int64_t)p.tiles : (int64_t)p.tiles * p.splits;   // pairs that get work
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(2 * (units < pairs ? units : pairs)), 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = kPairSmemBytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    B200Q_TRY(cudaLaunchKernelEx(&cfg, syrk_pair_kernel, map, p));
    B200Q_LAUNCH_CHECK();
    return B200Q_OK;
  }
  const int nb = (int)((K + kTileM - 1) / kTileM);
  p.tiles = num_tiles(nb);
  p.nb = nb;
  // token splits: enough units to fill the machine several times over, each split long enough
  // (>= 512 tokens) to hide its epilogue behind the next unit's main loop
  const int64_t max_splits = (T + 511) / 512;
  int best = 1;
  double best_eff = 0.0;
  for (int s = 1; s <= (int)(max_splits < 64 ? max_splits : 64); ++s) {
    int64_t units = (int64_t)p.tiles * s;
    int64_t waves = (units + kNumSMs - 1) / kNumSMs;
    double eff = (double)units / (double)(waves * kNumSMs);
    // prefer fewer splits unless the gain is real (atomics + epilogues are not free)
    if (eff > best_eff + 0.02) { best_eff = eff; best = s; }
  }
  p.splits = g_reproducible.load(std::memory_order_relaxed) ? 1 : best;
  int64_t tps = (T + p.splits - 1) / p.splits;
  p.tokens_per_split = ((tps + kBlockT - 1) / kBlockT) * kBlockT;

  B200Q_TRY(cudaFuncSetAttribute(syrk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
  int64_t units = (int64_t)p.tiles * p.splits;
  int grid = (int)(units < kNumSMs ? units : kNumSMs);
  syrk_kernel<<<grid, kThreads, kSmemBytes, st>>>(map, p);
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

void b200q_set_reproducible(int on) { g_reproducible.store(on ? 1 : 0, std::memory_order_relaxed); }
int b200q_get_reproducible(void) { return g_reproducible.load(std::memory_order_relaxed); }

int b200q_hessian_finalize(float* H, int64_t K, int64_t ldh, float scale, void* stream) {
  if (!H || K <= 0 || ldh < K) return B200Q_ERR_ARG;
  int64_t nb = (K + 31) / 32;
  int64_t nblk = nb * (nb + 1) / 2;
  b200q::syrk::finalize_kernel<<<grid_for(nblk, 8), 256, 0, (cudaStream_t)stream>>>(H, K, ldh, scale);
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

}  // extern "C"
