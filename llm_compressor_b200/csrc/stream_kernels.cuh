// Row-streaming kernels of the observer / quantize / pack path, tuned for HBM bandwidth.
//
// Thread layout: a CTA of 256 threads is TX chunk-columns by 256/TX rows (TX = 32..256, a
// power of two no larger than the row needs); a thread owns 8 consecutive elements (one
// 16-byte load of bf16) and walks its row in steps of TX chunks, two chunks in flight per
// iteration.  No integer division on the hot path.  The lanes that share a quantisation
// group (g/8 consecutive lanes, g a power of two in 8..256) reduce with xor shuffles.
#pragma once

#include "common.cuh"

namespace b200q {
namespace stream {

constexpr int kThreads = 256;

struct RowTiling {
  int tx;        // chunk-columns per CTA (power of two, 32..256)
  int rows;      // rows per CTA = 256 / tx
  int grid;
};
inline RowTiling make_tiling(int64_t N, int64_t K, int ctas_per_sm) {
  RowTiling t;
  int64_t cpr = K >> 3;
  t.tx = 32;
  while (t.tx < 256 && t.tx < cpr) t.tx <<= 1;
  t.rows = kThreads / t.tx;
  int64_t need = (N + t.rows - 1) / t.rows;
  t.grid = grid_for(need, ctas_per_sm);
  return t;
}

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
template <int DT>
__device__ __forceinline__ void load8s(const void* base, int64_t off, float (&v)[8]) {
  if constexpr (DT == B200Q_BF16) {
    uint4 u = ldg_stream((const __nv_bfloat16*)base + off);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
  } else {
    uint4 a = ldg_stream((const float*)base + off), b = ldg_stream((const float*)base + off + 4);
    v[0] = __uint_as_float(a.x); v[1] = __uint_as_float(a.y); v[2] = __uint_as_float(a.z); v[3] = __uint_as_float(a.w);
    v[4] = __uint_as_float(b.x); v[5] = __uint_as_float(b.y); v[6] = __uint_as_float(b.z); v[7] = __uint_as_float(b.w);
  }
}

enum PackKind { kFake = 0, kInt4 = 1, kByte = 2, kFp4 = 3, kInt8Word = 4 };

// codes of 8 elements -> storage.  `word_index` counts 8-element chunks from the start of `out`.
template <int MODE, int XDT>
__device__ __forceinline__ void store_codes(void* out, int64_t word_index, int64_t fake_off, const float (&q)[8],
                                            int kind) {
  if constexpr (MODE == kFake) {
    if constexpr (XDT == B200Q_BF16) {
      uint32_t w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        __nv_bfloat162 h = __floats2bfloat162_rn(q[2 * i], q[2 * i + 1]);
        w[i] = *reinterpret_cast<uint32_t*>(&h);
      }
      *reinterpret_cast<uint4*>((__nv_bfloat16*)out + fake_off) = make_uint4(w[0], w[1], w[2], w[3]);
    } else {
      float4* p = reinterpret_cast<float4*>((float*)out + fake_off);
      p[0] = make_float4(q[0], q[1], q[2], q[3]);
      p[1] = make_float4(q[4], q[5], q[6], q[7]);
    }
  } else if constexpr (MODE == kInt4) {
    uint32_t w = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) w |= ((uint32_t)((int)q[i] + 8) & 0xFu) << (4 * i);
    ((uint32_t*)out)[word_index] = w;
  } else if constexpr (MODE == kFp4) {
    uint32_t w = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) w |= e2m1_nibble(q[i]) << (4 * i);
    ((uint32_t*)out)[word_index] = w;
  } else {
    uint32_t w0 = 0, w1 = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t b0, b1;
      if (kind == kFp8) { b0 = e4m3_bits(q[i]); b1 = e4m3_bits(q[i + 4]); }
      else if (MODE == kInt8Word) { b0 = (uint32_t)((int)q[i] + 128) & 0xFFu; b1 = (uint32_t)((int)q[i + 4] + 128) & 0xFFu; }
      else { b0 = (uint32_t)(int)q[i] & 0xFFu; b1 = (uint32_t)(int)q[i + 4] & 0xFFu; }
      w0 |= b0 << (8 * i);
      w1 |= b1 << (8 * i);
    }
    reinterpret_cast<uint2*>(out)[word_index] = make_uint2(w0, w1);
  }
}

// ---------------------------------------------------------------------------------------
// Packed fast paths for 8 bf16 elements that share one scale.  They produce exactly what
// quant_code<CB> + store_codes produce, in about a third of the instructions:
//   q = x * (1/s) in float32 (a couple of ulps from the IEEE quotient), two values rounded to
//   bf16 with one cvt, zero point / clamp / round-to-integer done on bf16x2 registers (the
//   integer rounding is an addition of 192: bf16 has unit spacing in [128,256)), FP8 / FP4
//   codes made by the hardware converters (round-to-nearest-even, saturating: the same tie
//   rules as the reference's table).
// `unsafe` is set when a quotient is within 3 float ulps of a bf16 rounding midpoint; the
// caller then recomputes the chunk with true divisions.  Power-of-two (MX) scales make x*(1/s)
// exact, so they never need that.
__device__ __forceinline__ uint32_t cvt_bf16x2(float hi, float lo) {
  uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}
__device__ __forceinline__ uint32_t bf2_add(uint32_t a, uint32_t b) {
  __nv_bfloat162 r = __hadd2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
  return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t bf2_clamp(uint32_t a, uint32_t lo, uint32_t hi) {
  __nv_bfloat162 r = __hmin2(__hmax2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&lo)),
                             *reinterpret_cast<__nv_bfloat162*>(&hi));
  return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t bf2_splat(float v) {
  __nv_bfloat162 r = __float2bfloat162_rn(v);
  return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ bool near_bf16_midpoint(float q) {
  return ((__float_as_uint(q) + 0x8003u) & 0xFFFFu) <= 6u;  // low half-word in [0x7FFD, 0x8003]
}

// common front end: 4 words of bf16 pairs -> 4 words of clamped bf16 pairs bf16(bf16(x/s)+zp)
//
// Midpoint test, two quotients at a time: the low half-words of both products are packed into
// one word and 0x8004 is added to each (one 32-bit add; a carry out of the low half only widens
// the window of the high half by one), which maps "within 3 ulps of the bf16 midpoint 0x8000" to
// half-words 1..8.  The four words of a chunk are reduced with the packed 16-bit minimum and one
// test "some half-word below 16" decides; false alarms only cost the exact path.
template <bool EXACT, bool ADD_ZP>
__device__ __forceinline__ void front8_bf16(const uint4& raw, float rs, uint32_t zp2, uint32_t lo2, uint32_t hi2,
                                            uint32_t (&v)[4], bool& unsafe) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  uint32_t m[4];
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    const float q0 = __uint_as_float(w[p] << 16) * rs;
    const float q1 = __uint_as_float(w[p] & 0xFFFF0000u) * rs;
    if (!EXACT) m[p] = __byte_perm(__float_as_uint(q0), __float_as_uint(q1), 0x5410) + 0x80048004u;
    const uint32_t c = cvt_bf16x2(q1, q0);
    v[p] = bf2_clamp(ADD_ZP ? bf2_add(c, zp2) : c, lo2, hi2);
  }
  if (!EXACT) {
    const uint32_t mm = __vimin3_u16x2(__vimin3_u16x2(m[0], m[1], m[2]), m[3], m[3]) & 0xFFF0FFF0u;
    unsafe = ((mm & 0xFFFFu) == 0u) || ((mm >> 16) == 0u);
  } else {
    unsafe = false;
  }
}
// int4: 8 nibbles (value + 8) in one word
__device__ __forceinline__ uint32_t tail8_int4(const uint32_t (&v)[4]) {
  const uint32_t magic = 0x43404340u;  // bf16x2 {192, 192}
  uint32_t t[4];
#pragma unroll
  for (int p = 0; p < 4; ++p) t[p] = bf2_add(v[p], magic);  // low 4 mantissa bits = two's-complement nibble
  // bytes 0 and 2 of each word carry the nibbles of elements 2p and 2p+1
  uint32_t a = __byte_perm(t[0], t[1], 0x6420) & 0x0F0F0F0Fu;   // n0 n1 n2 n3, one per byte
  uint32_t b = __byte_perm(t[2], t[3], 0x6420) & 0x0F0F0F0Fu;   // n4 n5 n6 n7
  a |= a >> 4;                                                   // byte0 = n0|n1<<4, byte2 = n2|n3<<4
  b |= b >> 4;
  return __byte_perm(a, b, 0x6420) ^ 0x88888888u;
}
__device__ __forceinline__ void tail8_fp8(const uint32_t (&v)[4], uint32_t& w0, uint32_t& w1) {
  uint32_t h[4];
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    float2 f = make_float2(__uint_as_float(v[p] << 16), __uint_as_float(v[p] & 0xFFFF0000u));
    h[p] = (uint32_t)__nv_cvt_float2_to_fp8x2(f, __NV_SATFINITE, __NV_E4M3);
  }
  w0 = h[0] | (h[1] << 16);
  w1 = h[2] | (h[3] << 16);
}
__device__ __forceinline__ uint32_t cvt_e2m1x8(const float (&f)[8]) {
  uint32_t out;
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
      "mov.b32 %0, {b0, b1, b2, b3};\n\t}"
      : "=r"(out)
      : "f"(f[0]), "f"(f[1]), "f"(f[2]), "f"(f[3]), "f"(f[4]), "f"(f[5]), "f"(f[6]), "f"(f[7]));
  return out;
}
__device__ __forceinline__ uint32_t tail8_fp4(const uint32_t (&v)[4]) {
  float f[8];
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    f[2 * p] = __uint_as_float(v[p] << 16);
    f[2 * p + 1] = __uint_as_float(v[p] & 0xFFFF0000u);
  }
  return cvt_e2m1x8(f);
}
// NVFP4: float32 arithmetic (the effective scale scale/global_scale is float32).  The code
// is a monotone function of the quotient, so equal codes at both ends of a small interval
// around x*(1/s) settle it; otherwise `unsafe`.
__device__ __forceinline__ uint32_t nvfp4_8(const uint4& raw, float rs, bool& unsafe) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  // both ends of an interval that holds the exact quotient (reciprocal, its scaling and the
  // product each round by 2^-24 or less; the margin is 2^-21).  The fused "+ 0" turns a -0.0
  // weight into +0 like the reference's "+ zero_point".
  const float rlo = rs * (1.0f - 0x1p-21f), rhi = rs * (1.0f + 0x1p-21f);
  float lo[8], hi[8];
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    const float x0 = __uint_as_float(w[p] << 16), x1 = __uint_as_float(w[p] & 0xFFFF0000u);
    lo[2 * p] = __fmaf_rn(x0, rlo, 0.0f); hi[2 * p] = __fmaf_rn(x0, rhi, 0.0f);
    lo[2 * p + 1] = __fmaf_rn(x1, rlo, 0.0f); hi[2 * p + 1] = __fmaf_rn(x1, rhi, 0.0f);
  }
  const uint32_t c = cvt_e2m1x8(lo);
  unsafe = cvt_e2m1x8(hi) != c;
  return c;
}

// ---------------------------------------------------------------------------------------
// per-group min / max
template <int DT>
__global__ void __launch_bounds__(kThreads) minmax_group_kernel(const void* __restrict__ W, int N, int K,
                                                                int64_t ldw, int g, int tx_log2,
                                                                void* __restrict__ mn_out,
                                                                void* __restrict__ mx_out) {
  using E = Elem<DT>;
  using T = typename E::type;
  const int TX = 1 << tx_log2, rows = kThreads >> tx_log2;
  const int tx = threadIdx.x & (TX - 1), ty = threadIdx.x >> tx_log2;
  const int lanes = g >> 3, cpr = K >> 3, gpr = K / g;
  const int cend = (cpr + 31) & ~31;
  for (int row = blockIdx.x * rows + ty; row < N; row += gridDim.x * rows) {
    const T* wrow = (const T*)W + (int64_t)row * ldw;
    for (int c = tx; c < cend; c += 2 * TX) {
      const int c1 = c + TX;
      const bool l0 = c < cpr, l1 = c1 < cpr;
      float v0[8], v1[8];
      if (l0) load8s<DT>(wrow, (int64_t)c * 8, v0);
      if (l1) load8s<DT>(wrow, (int64_t)c1 * 8, v1);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const bool live = h ? l1 : l0;
        const int cc = h ? c1 : c;
        if (h == 1 && c1 >= cend) break;  // warp-uniform
        float lo = INFINITY, hi = -INFINITY;
        if (live) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float x = h ? v1[i] : v0[i];
            lo = fminf(lo, x); hi = fmaxf(hi, x);
          }
        }
        for (int o = lanes >> 1; o > 0; o >>= 1) {
          lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
          hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
        }
        if (live && (cc & (lanes - 1)) == 0) {
          const int64_t gi = (int64_t)row * gpr + (cc * 8) / g;
          E::store((T*)mn_out + gi, lo);
          E::store((T*)mx_out + gi, hi);
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------
// fused round-to-nearest for grouped schemes: statistics -> qparams -> codes -> packed.
// QParamCfg, qparams_one, store_zp and e8m0_of come from the including file.
template <int DT, int MODE, bool GLOBAL>
__global__ void __launch_bounds__(kThreads) rtn_group_kernel(
    const void* __restrict__ W, int N, int K, int64_t ldw, int g, int tx_log2, QParamCfg qc, QRange qr,
    const float* __restrict__ gscale, void* __restrict__ scale_out, void* __restrict__ zp_out,
    uint8_t* __restrict__ scale_store, void* __restrict__ out) {
  using E = Elem<DT>;
  using T = typename E::type;
  constexpr bool XB = E::is_bf16;
  constexpr bool SB = XB && !GLOBAL;
  constexpr bool CB = XB && SB;
  const float gs = GLOBAL ? *gscale : 1.0f;
  const int TX = 1 << tx_log2, rows = kThreads >> tx_log2;
  const int tx = threadIdx.x & (TX - 1), ty = threadIdx.x >> tx_log2;
  const int lanes = g >> 3, cpr = K >> 3, gpr = K / g;
  const int cend = (cpr + 31) & ~31;
  for (int row = blockIdx.x * rows + ty; row < N; row += gridDim.x * rows) {
    const T* wrow = (const T*)W + (int64_t)row * ldw;
    for (int c = tx; c < cend; c += 2 * TX) {
      const int c1 = c + TX;
      const bool l0 = c < cpr, l1 = c1 < cpr;
      float v[2][8];
      if (l0) load8s<DT>(wrow, (int64_t)c * 8, v[0]);
      if (l1) load8s<DT>(wrow, (int64_t)c1 * 8, v[1]);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const bool live = h ? l1 : l0;
        const int cc = h ? c1 : c;
        if (h == 1 && c1 >= cend) break;  // warp-uniform
        float lo = INFINITY, hi = -INFINITY;
        if (live) {
#pragma unroll
          for (int i = 0; i < 8; ++i) { lo = fminf(lo, v[h][i]); hi = fmaxf(hi, v[h][i]); }
        }
        for (int o = lanes >> 1; o > 0; o >>= 1) {
          lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
          hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
        }
        if (!live) continue;
        float s, z;
        qparams_one<XB>(lo, hi, qc, gs, s, z);
        if ((cc & (lanes - 1)) == 0) {
          const int64_t gi = (int64_t)row * gpr + (cc * 8) / g;
          E::store((T*)scale_out + gi, s);
          if (zp_out) store_zp(zp_out, qc.zp_kind, gi, z);
          if (scale_store) scale_store[gi] = (qc.scale_kind == B200Q_SCALE_FP8) ? e4m3_bits(s) : e8m0_of(s);
        }
        const float se = GLOBAL ? __fdiv_rn(s, gs) : s;
        const float rs = __frcp_rn(se);
        float q[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) q[i] = quant_code_fast<CB>(v[h][i], se, rs, z, qr);
        store_codes<MODE, DT>(out, (int64_t)row * cpr + cc, 0, q, qr.kind);
      }
    }
  }
}

// bf16 weights: same as rtn_group_kernel<B200Q_BF16, ...> with the packed fast paths.
__device__ __forceinline__ void minmax8_bf16(const uint4& raw, float& lo, float& hi) {
  const __nv_bfloat162* w = reinterpret_cast<const __nv_bfloat162*>(&raw);
  __nv_bfloat162 mx = __hmax2(__hmax2(w[0], w[1]), __hmax2(w[2], w[3]));
  __nv_bfloat162 mn = __hmin2(__hmin2(w[0], w[1]), __hmin2(w[2], w[3]));
  hi = fmaxf(__bfloat162float(mx.x), __bfloat162float(mx.y));
  lo = fminf(__bfloat162float(mn.x), __bfloat162float(mn.y));
}
// min / max kept as bf16 pairs across several chunks, widened once at the end
struct MinMax2 {
  __nv_bfloat162 mn, mx;
  __device__ __forceinline__ void first(const uint4& raw) {
    const __nv_bfloat162* w = reinterpret_cast<const __nv_bfloat162*>(&raw);
    mx = __hmax2(__hmax2(w[0], w[1]), __hmax2(w[2], w[3]));
    mn = __hmin2(__hmin2(w[0], w[1]), __hmin2(w[2], w[3]));
  }
  __device__ __forceinline__ void add(const uint4& raw) {
    const __nv_bfloat162* w = reinterpret_cast<const __nv_bfloat162*>(&raw);
    mx = __hmax2(__hmax2(mx, w[0]), __hmax2(__hmax2(w[1], w[2]), w[3]));
    mn = __hmin2(__hmin2(mn, w[0]), __hmin2(__hmin2(w[1], w[2]), w[3]));
  }
  __device__ __forceinline__ void finish(float& lo, float& hi) const {
    hi = fmaxf(__bfloat162float(mx.x), __bfloat162float(mx.y));
    lo = fminf(__bfloat162float(mn.x), __bfloat162float(mn.y));
  }
};
__device__ __forceinline__ void unpack8_bf16(const uint4& raw, float (&v)[8]) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}

// codes of one chunk with one (scale, zp): fast path, exact redo when flagged
template <int MODE, bool GLOBAL, bool SCALE_BF16>
__device__ __forceinline__ void chunk_codes_bf16(const uint4& raw, float se, float z, bool pow2_scale, QRange qr,
                                                 uint32_t& w0, uint32_t& w1) {
  constexpr bool CB = SCALE_BF16 && !GLOBAL;
  const float rs = __frcp_rn(se);
  bool unsafe = false;
  if constexpr (!CB) {
    if constexpr (MODE == kFp4) {
      w0 = nvfp4_8(raw, rs, unsafe);
    } else {
      unsafe = true;
    }
  } else if constexpr (MODE == kInt8Word || MODE == kByte) {
    if (qr.kind == kFp8) {
      uint32_t v[4];
      const uint32_t lim = 0x43E043E0u;  // bf16x2 {448, 448}
      if (pow2_scale) front8_bf16<true, true>(raw, rs, bf2_splat(z), lim ^ 0x80008000u, lim, v, unsafe);
      else front8_bf16<false, true>(raw, rs, bf2_splat(z), lim ^ 0x80008000u, lim, v, unsafe);
      tail8_fp8(v, w0, w1);
    } else {
      unsafe = true;  // int8 keeps the per-element path
    }
  } else {
    uint32_t v[4];
    const uint32_t lo2 = bf2_splat(qr.qmin), hi2 = bf2_splat(qr.qmax);
    // integer codes do not see the sign of zero, so a zero zero-point need not be added
    if (MODE == kInt4 && z == 0.0f) front8_bf16<false, false>(raw, rs, 0u, lo2, hi2, v, unsafe);
    else if (pow2_scale) front8_bf16<true, true>(raw, rs, bf2_splat(z), lo2, hi2, v, unsafe);
    else front8_bf16<false, true>(raw, rs, bf2_splat(z), lo2, hi2, v, unsafe);
    w0 = (MODE == kInt4) ? tail8_int4(v) : tail8_fp4(v);
  }
  if (unsafe) {
    float x[8], q[8];
    unpack8_bf16(raw, x);
#pragma unroll
    for (int i = 0; i < 8; ++i) q[i] = quant_code<CB>(x[i], se, z, qr);
    uint32_t a = 0, b = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (MODE == kInt4) a |= ((uint32_t)((int)q[i] + 8) & 0xFu) << (4 * i);
      else if (MODE == kFp4) a |= e2m1_nibble(q[i]) << (4 * i);
      else {
        uint32_t by = (qr.kind == kFp8) ? e4m3_bits(q[i])
                    : (MODE == kInt8Word) ? ((uint32_t)((int)q[i] + 128) & 0xFFu) : ((uint32_t)(int)q[i] & 0xFFu);
        if (i < 4) a |= by << (8 * i); else b |= by << (8 * (i - 4));
      }
    }
    w0 = a; w1 = b;
  }
}

// Lanes and chunks of a group: the g/8 chunks of a group are shared by L lanes, each taking R
// chunks L apart, so that one load instruction of the L lanes covers L*16 contiguous bytes and
// the group's fixed cost (statistics, qparams, reciprocal) is paid once per R*8 elements.
struct GroupSplit { int L, R; };
inline GroupSplit make_group_split(int g, int rmax = 8) {
  const int chunks = g >> 3;
  GroupSplit s;
  // groups of up to 32 elements: one lane per group (no shuffles, contiguous wide stores); wider
  // groups are shared by lanes so that a load instruction stays dense (one lane per 128-element
  // group measured 0.41 of the HBM peak against 0.60-0.65)
  s.R = chunks >= 16 ? 8 : (chunks >= 8 ? 4 : chunks);
  if (s.R > rmax) s.R = rmax;   // measured: 8 pays when statistics are computed, 4 when they are given
  s.L = chunks / s.R;
  return s;
}

// R consecutive chunks of one lane -> storage with the widest stores their alignment allows
// (chunk index wi0 is a multiple of R).
template <int MODE, int R>
__device__ __forceinline__ void store_lane_codes(void* out, int64_t wi0, const uint32_t (&a)[R], const uint32_t (&b)[R]) {
  if constexpr (MODE == kInt4 || MODE == kFp4) {
    uint32_t* o = (uint32_t*)out + wi0;
    if constexpr (R % 4 == 0) {
#pragma unroll
      for (int k = 0; k < R; k += 4) *reinterpret_cast<uint4*>(o + k) = make_uint4(a[k], a[k + 1], a[k + 2], a[k + 3]);
    } else if constexpr (R == 2) {
      *reinterpret_cast<uint2*>(o) = make_uint2(a[0], a[1]);
    } else {
      o[0] = a[0];
    }
  } else {
    uint2* o = reinterpret_cast<uint2*>(out) + wi0;
    if constexpr (R % 2 == 0) {
#pragma unroll
      for (int k = 0; k < R; k += 2) *reinterpret_cast<uint4*>(o + k) = make_uint4(a[k], b[k], a[k + 1], b[k + 1]);
    } else {
      o[0] = make_uint2(a[0], b[0]);
    }
  }
}

template <int MODE, bool GLOBAL, int R>
__global__ void __launch_bounds__(kThreads) rtn_group_bf16_kernel(
    const void* __restrict__ W, int N, int K, int64_t ldw, int g, int l_log2, int tx_log2, QParamCfg qc, QRange qr,
    const float* __restrict__ gscale, void* __restrict__ scale_out, void* __restrict__ zp_out,
    uint8_t* __restrict__ scale_store, void* __restrict__ out) {
  using T = __nv_bfloat16;
  const float gs = GLOBAL ? *gscale : 1.0f;
  const int TX = 1 << tx_log2, rows = kThreads >> tx_log2;
  const int tx = threadIdx.x & (TX - 1), ty = threadIdx.x >> tx_log2;
  const int L = 1 << l_log2, cpg = g >> 3, cpr = K >> 3, gpr = K / g;
  const int slots = gpr << l_log2;            // thread slots per row
  const int send = (slots + 31) & ~31;
  const bool pow2_scale = qc.scale_kind == B200Q_SCALE_E8M0;
  for (int row = blockIdx.x * rows + ty; row < N; row += gridDim.x * rows) {
    const T* wrow = (const T*)W + (int64_t)row * ldw;
    for (int t = tx; t < send; t += TX) {
      const bool live = t < slots;
      const int grp = t >> l_log2, j = t & (L - 1);
      const int c0 = grp * cpg + j;           // first chunk of this lane
      uint4 raw[R];
#pragma unroll
      for (int k = 0; k < R; ++k)
        raw[k] = live ? ldg_stream(wrow + (int64_t)(c0 + k * L) * 8) : make_uint4(0, 0, 0, 0);
      float lo = INFINITY, hi = -INFINITY;
      if (live) {
        MinMax2 mm;
        mm.first(raw[0]);
#pragma unroll
        for (int k = 1; k < R; ++k) mm.add(raw[k]);
        mm.finish(lo, hi);
      }
      for (int o = L >> 1; o > 0; o >>= 1) {
        lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
        hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
      }
      if (!live) continue;
      float s, z;
      qparams_one<true>(lo, hi, qc, gs, s, z);
      if (j == 0) {
        const int64_t gi = (int64_t)row * gpr + grp;
        ((T*)scale_out)[gi] = __float2bfloat16_rn(s);
        if (zp_out) store_zp(zp_out, qc.zp_kind, gi, z);
        if (scale_store) scale_store[gi] = (qc.scale_kind == B200Q_SCALE_FP8) ? e4m3_bits(s) : e8m0_of(s);
      }
      const float se = GLOBAL ? __fdiv_rn(s, gs) : s;
      if (l_log2 == 0) {   // one lane per group: its R chunks are contiguous
        uint32_t a[R], b[R];
#pragma unroll
        for (int k = 0; k < R; ++k) {
          a[k] = 0; b[k] = 0;
          chunk_codes_bf16<MODE, GLOBAL, true>(raw[k], se, z, pow2_scale, qr, a[k], b[k]);
        }
        store_lane_codes<MODE, R>(out, (int64_t)row * cpr + c0, a, b);
        continue;
      }
#pragma unroll
      for (int k = 0; k < R; ++k) {
        uint32_t w0 = 0, w1 = 0;
        chunk_codes_bf16<MODE, GLOBAL, true>(raw[k], se, z, pow2_scale, qr, w0, w1);
        const int64_t wi = (int64_t)row * cpr + c0 + k * L;
        if (MODE == kInt4 || MODE == kFp4) ((uint32_t*)out)[wi] = w0;
        else reinterpret_cast<uint2*>(out)[wi] = make_uint2(w0, w1);
      }
    }
  }
}

// per-group min / max of bf16 weights with the lane / chunk split of the fused kernel
template <int R>
__global__ void __launch_bounds__(kThreads) minmax_group_bf16_kernel(const void* __restrict__ W, int N, int K,
                                                                     int64_t ldw, int g, int l_log2, int tx_log2,
                                                                     void* __restrict__ mn_out,
                                                                     void* __restrict__ mx_out) {
  using T = __nv_bfloat16;
  const int TX = 1 << tx_log2, rows = kThreads >> tx_log2;
  const int tx = threadIdx.x & (TX - 1), ty = threadIdx.x >> tx_log2;
  const int L = 1 << l_log2, cpg = g >> 3, gpr = K / g;
  const int slots = gpr << l_log2;
  const int send = (slots + 31) & ~31;
  for (int row = blockIdx.x * rows + ty; row < N; row += gridDim.x * rows) {
    const T* wrow = (const T*)W + (int64_t)row * ldw;
    for (int t = tx; t < send; t += TX) {
      const bool live = t < slots;
      const int grp = t >> l_log2, j = t & (L - 1);
      const int c0 = grp * cpg + j;
      uint4 raw[R];
#pragma unroll
      for (int k = 0; k < R; ++k)
        raw[k] = live ? ldg_stream(wrow + (int64_t)(c0 + k * L) * 8) : make_uint4(0, 0, 0, 0);
      float lo = INFINITY, hi = -INFINITY;
      if (live) {
        MinMax2 mm;
        mm.first(raw[0]);
#pragma unroll
        for (int k = 1; k < R; ++k) mm.add(raw[k]);
        mm.finish(lo, hi);
      }
      for (int o = L >> 1; o > 0; o >>= 1) {
        lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
        hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
      }
      if (live && j == 0) {
        const int64_t gi = (int64_t)row * gpr + grp;
        ((T*)mn_out)[gi] = __float2bfloat16_rn(lo);
        ((T*)mx_out)[gi] = __float2bfloat16_rn(hi);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------
// quantise (or fake-quantise) with given parameters; `uniform`: one (scale, zp) per 8-element
// chunk (no g_idx, group / block width a multiple of 8), read once per chunk.
template <int XDT, int SDT, bool GLOBAL, int MODE>
__global__ void __launch_bounds__(kThreads) quant_rows_kernel(
    const void* __restrict__ W, int N, int K, int64_t ldw, int tx_log2, const void* __restrict__ scale,
    const void* __restrict__ zp, int zp_kind, ParamMap pm, bool uniform, const float* __restrict__ gscale,
    QRange qr, void* __restrict__ out, int64_t ldo) {
  using EX = Elem<XDT>;
  using TXT = typename EX::type;
  using ES = Elem<SDT>;
  constexpr bool XB = EX::is_bf16;
  constexpr bool SB = ES::is_bf16 && !GLOBAL;
  constexpr bool CB = XB && SB;
  const float g = GLOBAL ? *gscale : 1.0f;
  const int TX = 1 << tx_log2, rows = kThreads >> tx_log2;
  const int tx = threadIdx.x & (TX - 1), ty = threadIdx.x >> tx_log2;
  const int cpr = K >> 3;
  for (int row = blockIdx.x * rows + ty; row < N; row += gridDim.x * rows) {
    const TXT* wrow = (const TXT*)W + (int64_t)row * ldw;
    for (int c = tx; c < cpr; c += 2 * TX) {
      const int c1 = c + TX;
      const bool l1 = c1 < cpr;
      float v[2][8];
      uint4 raw[2];
      if constexpr (XB) {
        raw[0] = ldg_stream(wrow + (int64_t)c * 8);
        raw[1] = l1 ? ldg_stream(wrow + (int64_t)c1 * 8) : make_uint4(0, 0, 0, 0);
      } else {
        load8s<XDT>(wrow, (int64_t)c * 8, v[0]);
        if (l1) load8s<XDT>(wrow, (int64_t)c1 * 8, v[1]);
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        if (h == 1 && !l1) break;
        const int cc = h ? c1 : c;
        const int col0 = cc * 8;
        float q[8];
        if (uniform) {
          const int64_t pi = pm.index(row, col0);
          float s = ES::load((const typename ES::type*)scale + pi);
          if (GLOBAL) s = __fdiv_rn(s, g);
          const float z = zp ? load_zp(zp, zp_kind, pi) : 0.0f;
          if constexpr (XB && MODE != kFake) {
            uint32_t w0 = 0, w1 = 0;
            const bool p2 = (__float_as_uint(s) & 0x7FFFFFu) == 0u;
            chunk_codes_bf16<MODE, GLOBAL, ES::is_bf16>(raw[h], s, z, p2, qr, w0, w1);
            if (MODE == kInt4 || MODE == kFp4) ((uint32_t*)out)[(int64_t)row * cpr + cc] = w0;
            else reinterpret_cast<uint2*>(out)[(int64_t)row * cpr + cc] = make_uint2(w0, w1);
            continue;
          }
          if constexpr (XB) unpack8_bf16(raw[h], v[h]);
          const float rs = __frcp_rn(s);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            q[i] = quant_code_fast<CB>(v[h][i], s, rs, z, qr);
            if (MODE == kFake) q[i] = dequant_code<SB>(q[i], s, z);
          }
        } else {
          if constexpr (XB) unpack8_bf16(raw[h], v[h]);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int64_t pi = pm.index(row, col0 + i);
            float s = ES::load((const typename ES::type*)scale + pi);
            if (GLOBAL) s = __fdiv_rn(s, g);
            const float z = zp ? load_zp(zp, zp_kind, pi) : 0.0f;
            q[i] = quant_code<CB>(v[h][i], s, z, qr);
            if (MODE == kFake) q[i] = dequant_code<SB>(q[i], s, z);
          }
        }
        store_codes<MODE, XDT>(out, (int64_t)row * cpr + cc, (int64_t)row * ldo + col0, q, qr.kind);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------
// quantise + pack bf16 weights with given per-group parameters (no g_idx, group a power of two
// in 8..256): the lane / chunk split of the fused kernel, parameters read once per R chunks.
template <int SDT, bool GLOBAL, int MODE, int R>
__global__ void __launch_bounds__(kThreads) quant_group_bf16_kernel(
    const void* __restrict__ W, int N, int K, int64_t ldw, int g, int l_log2, int tx_log2,
    const void* __restrict__ scale, const void* __restrict__ zp, int zp_kind, const float* __restrict__ gscale,
    QRange qr, void* __restrict__ out) {
  using T = __nv_bfloat16;
  using ES = Elem<SDT>;
  const float gs = GLOBAL ? *gscale : 1.0f;
  const int TX = 1 << tx_log2, rows = kThreads >> tx_log2;
  const int tx = threadIdx.x & (TX - 1), ty = threadIdx.x >> tx_log2;
  const int L = 1 << l_log2, cpg = g >> 3, cpr = K >> 3, gpr = K / g;
  const int slots = gpr << l_log2;
  for (int row = blockIdx.x * rows + ty; row < N; row += gridDim.x * rows) {
    const T* wrow = (const T*)W + (int64_t)row * ldw;
    for (int t = tx; t < slots; t += TX) {
      const int grp = t >> l_log2, j = t & (L - 1);
      const int c0 = grp * cpg + j;
      uint4 raw[R];
#pragma unroll
      for (int k = 0; k < R; ++k) raw[k] = ldg_stream(wrow + (int64_t)(c0 + k * L) * 8);
      const int64_t pi = (int64_t)row * gpr + grp;
      float s = ES::load((const typename ES::type*)scale + pi);
      if (GLOBAL) s = __fdiv_rn(s, gs);
      const float z = zp ? load_zp(zp, zp_kind, pi) : 0.0f;
      const bool p2 = (__float_as_uint(s) & 0x7FFFFFu) == 0u;
      if (l_log2 == 0) {
        uint32_t a[R], b[R];
#pragma unroll
        for (int k = 0; k < R; ++k) {
          a[k] = 0; b[k] = 0;
          chunk_codes_bf16<MODE, GLOBAL, ES::is_bf16>(raw[k], s, z, p2, qr, a[k], b[k]);
        }
        store_lane_codes<MODE, R>(out, (int64_t)row * cpr + c0, a, b);
        continue;
      }
#pragma unroll
      for (int k = 0; k < R; ++k) {
        uint32_t w0 = 0, w1 = 0;
        chunk_codes_bf16<MODE, GLOBAL, ES::is_bf16>(raw[k], s, z, p2, qr, w0, w1);
        const int64_t wi = (int64_t)row * cpr + c0 + k * L;
        if (MODE == kInt4 || MODE == kFp4) ((uint32_t*)out)[wi] = w0;
        else reinterpret_cast<uint2*>(out)[wi] = make_uint2(w0, w1);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------
// CHANNEL strategy, bf16 weights: one CTA per row, the row held in registers between the
// statistics pass and the quantisation (R chunks of 8 elements per thread, K <= 2048 * R), so the
// row is read from HBM once.  Same packed fast paths as the group kernels.
template <int MODE, int R>
__global__ void __launch_bounds__(kThreads) rtn_channel_bf16_kernel(
    const void* __restrict__ W, int N, int K, int64_t ldw, QParamCfg qc, QRange qr,
    void* __restrict__ scale_out, void* __restrict__ zp_out, void* __restrict__ out) {
  using T = __nv_bfloat16;
  __shared__ float s_lo[2][kThreads / 32], s_hi[2][kThreads / 32];
  const int cpr = K >> 3;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool pow2_scale = qc.scale_kind == B200Q_SCALE_E8M0;
  int par = 0;
  for (int row = blockIdx.x; row < N; row += gridDim.x, par ^= 1) {
    const T* wrow = (const T*)W + (int64_t)row * ldw;
    uint4 raw[R];
#pragma unroll
    for (int k = 0; k < R; ++k) {
      const int c = threadIdx.x + k * kThreads;
      raw[k] = (c < cpr) ? ldg_stream(wrow + (int64_t)c * 8) : make_uint4(0, 0, 0, 0);
    }
    float lo = INFINITY, hi = -INFINITY;
#pragma unroll
    for (int k = 0; k < R; ++k) {
      if (threadIdx.x + k * kThreads < cpr) {
        float a, b;
        minmax8_bf16(raw[k], a, b);
        lo = fminf(lo, a); hi = fmaxf(hi, b);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
      hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
    }
    if (lane == 0) { s_lo[par][warp] = lo; s_hi[par][warp] = hi; }
    __syncthreads();   // one barrier per row: the buffers alternate
#pragma unroll
    for (int w = 0; w < kThreads / 32; ++w) { lo = fminf(lo, s_lo[par][w]); hi = fmaxf(hi, s_hi[par][w]); }
    float s, z;
    qparams_one<true>(lo, hi, qc, 1.0f, s, z);
    if (threadIdx.x == 0) {
      ((T*)scale_out)[row] = __float2bfloat16_rn(s);
      if (zp_out) store_zp(zp_out, qc.zp_kind, row, z);
    }
#pragma unroll
    for (int k = 0; k < R; ++k) {
      const int c = threadIdx.x + k * kThreads;
      if (c < cpr) {
        uint32_t w0 = 0, w1 = 0;
        chunk_codes_bf16<MODE, false, true>(raw[k], s, z, pow2_scale, qr, w0, w1);
        const int64_t wi = (int64_t)row * cpr + c;
        if (MODE == kInt4 || MODE == kFp4) ((uint32_t*)out)[wi] = w0;
        else reinterpret_cast<uint2*>(out)[wi] = make_uint2(w0, w1);
      }
    }
  }
}

}  // namespace stream
}  // namespace b200q
