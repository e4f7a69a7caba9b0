// TMA-fed variant of the fused round-to-nearest group kernel (bf16 weights).
//
// The register kernels of stream_kernels.cuh issue their loads and then have to wait for them:
// with the arithmetic now cheap they are bound by memory latency, not by HBM or by issue slots.
// Here the loads are decoupled from the arithmetic.  Every warp owns a ring of three 4 KiB
// shared-memory tiles; one lane asks the TMA unit for the tile two steps ahead
// (cp.async.bulk.tensor, completion on an mbarrier) while the warp works on the current one, so
// each SM keeps up to 2 x 16 tiles = 128 KiB in flight whatever the warps are doing.
//
// A tile is 2048 consecutive elements of one row, seen by the tensor map as 32 rows of 128 bytes
// and written with the 128-byte swizzle, so that lane i reads "its" row i (64 consecutive
// elements, 8 chunks of 16 bytes) without bank conflicts: the chunk c of row i sits at column
// c ^ (i & 7).  A lane therefore holds whole groups (g <= 64) or an aligned part of one (g = 128,
// 256: 2 or 4 neighbouring lanes), its 8 code words are contiguous and leave in 16-byte stores, and
// the scales of a lane's groups leave in one store.  Waits on the mbarriers are bounded; an expired
// wait sets the library's device flag (b200q_take_wait_status) and ends the warp's work.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace b200q {
namespace tma {

constexpr int kWarps = 8;
constexpr int kStages = 3;
constexpr int kTileBytes = 4096;
constexpr int kTileElems = 2048;
constexpr int kSmemBytes = kWarps * kStages * kTileBytes + 1024 + kWarps * kStages * 8;
constexpr long long kWaitCycles = 2000000000LL;   // about one second

__device__ int g_wait_expired;   // set by any streaming kernel whose bounded wait ran out

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred P1;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P1, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, P1;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (clock64() - t0 > kWaitCycles) return false;
  }
  return true;
}
__device__ __forceinline__ void tile_request(uint32_t dst, const CUtensorMap* map, uint32_t bar, int tc, int row) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((uint32_t)kTileBytes) : "memory");
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(0), "r"(tc * 32), "r"(row) : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

// G: group size (16, 32, 64, 128 or 256).
template <int MODE, bool GLOBAL, int G>
__global__ void __launch_bounds__(kWarps * 32, 2) rtn_group_tma_kernel(
    const __grid_constant__ CUtensorMap wmap, int N, int K, QParamCfg qc, QRange qr,
    const float* __restrict__ gscale, void* __restrict__ scale_out, void* __restrict__ zp_out,
    uint8_t* __restrict__ scale_store, void* __restrict__ out, int drop_request) {
  // drop_request >= 0 (test hook, -1 in normal use): warp 0 of CTA 0 leaves out its drop_request-th
  // tile request, so that its wait for that tile runs into the bound and the status path is exercised
  using namespace stream;
  using T = __nv_bfloat16;
  constexpr int CPG = G / 8;                         // chunks per group
  constexpr int GPL = CPG >= 8 ? 1 : 8 / CPG;        // groups per lane
  constexpr int L = CPG >= 8 ? CPG / 8 : 1;          // lanes per group
  constexpr int RC = CPG >= 8 ? 8 : CPG;             // chunks of one group held by a lane
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw0 = smem_u32(smem_raw);
  const uint32_t base = (raw0 + 1023u) & ~1023u;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t tiles0 = base + (uint32_t)(warp * kStages) * kTileBytes;
  const uint32_t bars0 = base + (uint32_t)(kWarps * kStages) * kTileBytes + (uint32_t)(warp * kStages) * 8u;
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < kStages; ++s)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bars0 + 8u * s), "r"(1u) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const float gs = GLOBAL ? *gscale : 1.0f;
  const bool mx = qc.scale_kind == B200Q_SCALE_E8M0, sym = qc.symmetric != 0;
  const int tpr = K / kTileElems, cpr = K >> 3, gpr = K / G;
  const int64_t total = (int64_t)N * tpr;
  const int64_t stride = (int64_t)gridDim.x * kWarps;
  const int64_t first = (int64_t)blockIdx.x * kWarps + warp;
  const bool victim = drop_request >= 0 && blockIdx.x == 0 && warp == 0;
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < kStages - 1; ++s) {
      const int64_t t = first + s * stride;
      if (t < total && !(victim && drop_request == s))
        tile_request(tiles0 + s * kTileBytes, &wmap, bars0 + 8u * s, (int)(t % tpr), (int)(t / tpr));
    }
  }
  int it = 0;
  for (int64_t t = first; t < total; t += stride, ++it) {
    const int s = it % kStages;
    // (the vote also orders every lane's reads of the previous tile before its buffer is refilled)
    if (!__all_sync(0xffffffffu, mbar_wait(bars0 + 8u * s, (uint32_t)((it / kStages) & 1)))) {
      // give up: record it, let a request that may still be in flight land (bounded), and leave
      if (lane == 0) atomicExch(&g_wait_expired, 1);
      if (t + stride < total) (void)mbar_wait(bars0 + 8u * ((it + 1) % kStages), (uint32_t)(((it + 1) / kStages) & 1));
      break;
    }
    if (lane == 0) {
      const int64_t tn = t + (kStages - 1) * stride;
      const int sn = (it + kStages - 1) % kStages;
      if (tn < total && !(victim && drop_request == it + kStages - 1))
        tile_request(tiles0 + sn * kTileBytes, &wmap, bars0 + 8u * sn, (int)(tn % tpr), (int)(tn / tpr));
    }
    const int row = (int)(t / tpr), tc = (int)(t - (int64_t)row * tpr);
    uint4 raw[8];
    {
      const uint32_t rowaddr = tiles0 + s * kTileBytes + lane * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c) raw[c] = lds128(rowaddr + (((uint32_t)c ^ ((uint32_t)lane & 7u)) << 4));
    }
    const int c0 = tc * (kTileElems / 8) + lane * 8;           // first chunk of this lane within the row
    uint32_t a[8], b[8];
    uint32_t sc_bits[GPL];     // bf16 scales of this lane's groups
    uint32_t zp_bytes = 0, st_bytes = 0;
    if constexpr (GLOBAL) {
      // NVFP4: per 16 elements  scale = e4m3(global * bf16(amax / 6)),  code = e2m1(x / (scale / global)).
      // Everything a group needs is formed with single instructions: the FP8 round trip by the
      // hardware converters, 1 / (scale / global) as global * (1 / scale) to a few ulps, which the
      // interval test of nvfp4_8 allows for (its margin is widened to 2^-20 here).  A chunk whose
      // interval test fails is redone exactly, with the true float32 division, after the fast pass.
      static_assert(GPL == 4 && RC == 2, "NVFP4 uses groups of 16 elements");
      uint32_t redo = 0;
#pragma unroll
      for (int q = 0; q < GPL; ++q) {
        const uint4 r0 = raw[2 * q], r1 = raw[2 * q + 1];
        // largest magnitude of the group: sign bits off, packed unsigned maximum
        uint32_t m = __vimax3_u16x2(r0.x & 0x7FFF7FFFu, r0.y & 0x7FFF7FFFu, r0.z & 0x7FFF7FFFu);
        m = __vimax3_u16x2(m, r0.w & 0x7FFF7FFFu, r1.x & 0x7FFF7FFFu);
        m = __vimax3_u16x2(m, r1.y & 0x7FFF7FFFu, r1.z & 0x7FFF7FFFu);
        m = __vimax3_u16x2(m, r1.w & 0x7FFF7FFFu, m);
        const float amax = __uint_as_float(max(m & 0xFFFFu, m >> 16) << 16);
        float sc = fminf(gs * bf16r(amax * qc.inv_half_range), 448.0f);
        uint16_t f8;
        asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(f8) : "f"(0.0f), "f"(sc));
        uint32_t h2;
        asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(f8));
        sc = __half2float(__ushort_as_half((unsigned short)(h2 & 0xFFFFu)));
        uint32_t bits = f8 & 0xFFu;
        if (sc == 0.0f) { sc = qc.eps; bits = 0x20u; }     // 0.125
        sc_bits[q] = __float_as_uint(sc) >> 16;             // exact: an FP8 value has few mantissa bits
        st_bytes |= bits << (8 * q);
        const float rs = gs * __frcp_rn(sc);
        const bool fast = rs >= 0x1p-100f && rs <= 0x1p100f;
        bool u0 = true, u1 = true;
        if (fast) {
          a[2 * q] = nvfp4_8(r0, rs, u0, 0x1p-20f);
          a[2 * q + 1] = nvfp4_8(r1, rs, u1, 0x1p-20f);
        }
        redo |= (u0 ? 1u : 0u) << (2 * q) | (u1 ? 1u : 0u) << (2 * q + 1);
      }
      if (redo) {
#pragma unroll 1
        for (int c = 0; c < 8; ++c) {
          if (!((redo >> c) & 1u)) continue;
          const float sc = __uint_as_float(sc_bits[c >> 1] << 16);
          uint4 rc = raw[0];
#pragma unroll
          for (int k = 1; k < 8; ++k) if (k == c) rc = raw[k];
          const uint2 r = chunk_codes_exact<MODE, false>(rc, __fdiv_rn(sc, gs), 0.0f, qr);
#pragma unroll
          for (int k = 0; k < 8; ++k) if (k == c) a[k] = r.x;
        }
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) b[k] = 0;
    } else {
#pragma unroll
    for (int q = 0; q < GPL; ++q) {
      const uint4(&graw)[RC] = *reinterpret_cast<const uint4(*)[RC]>(&raw[q * RC]);
      RangeQ mm;
      mm.first(graw[0]);
#pragma unroll
      for (int k = 1; k < RC; ++k) mm.add(graw[k]);
      float lo, hi;
      mm.finish(lo, hi);
#pragma unroll
      for (int o = L >> 1; o > 0; o >>= 1) {
        lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
        hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
      }
      float sc, z;
      qparams_one<true>(lo, hi, qc, gs, sc, z);
      sc_bits[q] = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(sc));
      if (qc.zp_kind == B200Q_ZP_FP8) zp_bytes |= (uint32_t)e4m3_bits(z) << (8 * q);
      else zp_bytes |= ((uint32_t)(int)z & 0xFFu) << (8 * q);
      if (qc.scale_kind == B200Q_SCALE_FP8) st_bytes |= (uint32_t)e4m3_bits(sc) << (8 * q);
      else if (qc.scale_kind == B200Q_SCALE_E8M0) st_bytes |= (uint32_t)e8m0_of(sc) << (8 * q);
      const GroupQ gq = make_group_q<true>(sc, z);
      uint32_t(&ga)[RC] = *reinterpret_cast<uint32_t(*)[RC]>(&a[q * RC]);
      uint32_t(&gb)[RC] = *reinterpret_cast<uint32_t(*)[RC]>(&b[q * RC]);
      if (mx) lane_codes<MODE, false, true, RC, true, false, true>(graw, gq, qr, ga, gb);
      else if (sym) lane_codes<MODE, false, true, RC, false, false, true>(graw, gq, qr, ga, gb);
      else lane_codes<MODE, false, true, RC, false, true, false>(graw, gq, qr, ga, gb);
    }
    }
    // codes: 8 consecutive words (or word pairs) per lane
    const int64_t wi = (int64_t)row * cpr + c0;
    if constexpr (MODE == stream::kInt4 || MODE == stream::kFp4) {
      uint4* o = reinterpret_cast<uint4*>((uint32_t*)out + wi);
      o[0] = make_uint4(a[0], a[1], a[2], a[3]);
      o[1] = make_uint4(a[4], a[5], a[6], a[7]);
    } else {
      uint4* o = reinterpret_cast<uint4*>(reinterpret_cast<uint2*>(out) + wi);
#pragma unroll
      for (int k = 0; k < 4; ++k) o[k] = make_uint4(a[2 * k], b[2 * k], a[2 * k + 1], b[2 * k + 1]);
    }
    // parameters: one store per kind for all groups of the lane
    if (L == 1 || (lane & (L - 1)) == 0) {
      const int64_t gi = (int64_t)row * gpr + (c0 / CPG);
      T* so = (T*)scale_out + gi;
      if constexpr (GPL == 1) {
        *reinterpret_cast<uint16_t*>(so) = (uint16_t)sc_bits[0];
        if (zp_out) ((uint8_t*)zp_out)[gi] = (uint8_t)zp_bytes;
        if (scale_store) scale_store[gi] = (uint8_t)st_bytes;
      } else if constexpr (GPL == 2) {
        *reinterpret_cast<uint32_t*>(so) = sc_bits[0] | (sc_bits[1] << 16);
        if (zp_out) *reinterpret_cast<uint16_t*>((uint8_t*)zp_out + gi) = (uint16_t)zp_bytes;
        if (scale_store) *reinterpret_cast<uint16_t*>(scale_store + gi) = (uint16_t)st_bytes;
      } else {
        static_assert(GPL == 4, "groups of 16, 32, 64, 128 or 256 elements");
        *reinterpret_cast<uint2*>(so) = make_uint2(sc_bits[0] | (sc_bits[1] << 16), sc_bits[2] | (sc_bits[3] << 16));
        if (zp_out) *reinterpret_cast<uint32_t*>((uint8_t*)zp_out + gi) = zp_bytes;
        if (scale_store) *reinterpret_cast<uint32_t*>(scale_store + gi) = st_bytes;
      }
    }
  }
}

}  // namespace tma
}  // namespace b200q
