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
// quant_code<CB> + store_codes produce, in about a quarter of the instructions.
//
// bf16 weight, bf16 scale (CB).  The reference forms q = bf16(float(x) / float(s)).  x and s carry
// 8 significant bits each, so the exact quotient is a ratio of two integers below 256; a bf16
// rounding midpoint has 9 significant bits, so the quotient can neither be a midpoint (that would
// need s to be a multiple of 256) nor come closer to one than 1 / (511 * 255) = 7.7e-6 relative:
// 129 float32 ulps, verified exhaustively over all pairs of mantissas.  x * (1/s) in float32 is
// within 2 ulps of the quotient, therefore bf16(x * (1/s)) is ALWAYS the reference's q and no
// check is needed.  The product is formed two elements at a time (fma.rn.f32x2, with a +0 addend
// where the sign of a zero quotient matters: -0 + 0 = +0 is what the reference's "+ zero_point"
// does), two values are rounded to bf16 with one cvt, the zero point, the clamp and the integer
// rounding run on bf16x2 registers (rounding to an integer is the addition of 192: bf16 has unit
// spacing in [128, 256)), FP8 / FP4 codes come from the hardware converters (round to nearest
// even, saturating: the same ties and the same clamp as the reference).  Power-of-two (MX) scales
// make the product exact in bf16 itself: one packed HFMA2 per pair, no float32 at all.
// Scales outside 2^-100 .. 2^100 (where 1/s leaves the normal range) take the exact path.
__device__ __forceinline__ uint32_t cvt_bf16x2(float hi, float lo) {
  uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}
__device__ __forceinline__ uint32_t bf2_add(uint32_t a, uint32_t b) {
  __nv_bfloat162 r = __hadd2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
  return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t bf2_fma(uint32_t a, uint32_t b, uint32_t c) {
  __nv_bfloat162 r = __hfma2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b),
                             *reinterpret_cast<__nv_bfloat162*>(&c));
  return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t bf2_min(uint32_t a, uint32_t b) {
  __nv_bfloat162 r = __hmin2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
  return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t bf2_max(uint32_t a, uint32_t b) {
  __nv_bfloat162 r = __hmax2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
  return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t bf2_splat(float v) {
  __nv_bfloat162 r = __float2bfloat162_rn(v);
  return *reinterpret_cast<uint32_t*>(&r);
}
// {a0, a1} * r + c on the packed float32 pipe (one instruction for both lanes)
__device__ __forceinline__ void fma2_f32(float a0, float a1, float r, float c, float& q0, float& q1) {
  uint64_t a, b, cc, d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(a) : "f"(a0), "f"(a1));
  asm("mov.b64 %0, {%1, %1};" : "=l"(b) : "f"(r));
  asm("mov.b64 %0, {%1, %1};" : "=l"(cc) : "f"(c));
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(cc));
  asm("mov.b64 {%0, %1}, %2;" : "=f"(q0), "=f"(q1) : "l"(d));
}

// What the 8-element paths need from one (scale, zero point), prepared once per group.
//
// The quotient itself stays in packed bf16 arithmetic: with 1/s (float32) split into two bf16
// parts r_hi = bf16(1/s), r_lo = bf16(1/s - r_hi),
//     t = fma(x, r_lo, +0)        q = fma(x, r_hi, t)            (two HFMA2 per pair)
// gives q = bf16(x / s) for every pair of bf16 significands (checked exhaustively with exact
// rational arithmetic: the error of t, 2^-18 relative to q, is below the 7.7e-6 that separates
// x / s from the nearest rounding midpoint).  A zero x gives +0 whatever its sign, like the
// reference's "+ zero_point".  Power-of-two scales have r_lo = 0 and need one HFMA2.
struct GroupQ {
  float se, rs, z;
  uint32_t z2;           // zero point as a bf16 pair
  uint32_t rhi2, rlo2;   // the two bf16 parts of 1/scale, each as a pair
  bool slow;             // 1/scale leaves the normal range: exact path
};
template <bool CB>
__device__ __forceinline__ GroupQ make_group_q(float se, float z) {
  GroupQ g;
  g.se = se; g.z = z;
  g.rs = __frcp_rn(se);
  g.slow = !(se >= 0x1p-100f && se <= 0x1p100f);
  if (CB) {
    const float rhi = bf16r(g.rs);
    g.rhi2 = bf2_splat(rhi);
    g.rlo2 = bf2_splat(g.rs - rhi);
    g.z2 = bf2_splat(z);
  } else {
    g.rhi2 = g.rlo2 = g.z2 = 0u;
  }
  return g;
}

// q = bf16(x / s) for the 8 elements of a chunk, as 4 bf16 pairs.
template <bool POW2>
__device__ __forceinline__ void quot8_bf16(const uint4& raw, const GroupQ& g, uint32_t (&v)[4]) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    const uint32_t t = POW2 ? 0u : bf2_fma(w[p], g.rlo2, 0u);
    v[p] = bf2_fma(w[p], g.rhi2, t);
  }
}
// int4: 8 nibbles (value + 8) in one word; v holds bf16 pairs already clamped to [-8, 7]
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
// int8: 8 bytes; v holds bf16 pairs already clamped to [-128, 127].  Rounding to an integer is
// the float32 addition of 1.5 * 2^23 (the value is exact in float32, so this is round half to
// even on it), whose low byte is the two's-complement code.
template <bool OFFSET>
__device__ __forceinline__ void tail8_int8(const uint32_t (&v)[4], uint32_t& w0, uint32_t& w1) {
  uint32_t t[8];
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    float a, b;
    fma2_f32(__uint_as_float(v[p] << 16), __uint_as_float(v[p] & 0xFFFF0000u), 1.0f, 12582912.0f, a, b);
    t[2 * p] = __float_as_uint(a); t[2 * p + 1] = __float_as_uint(b);
  }
  w0 = __byte_perm(__byte_perm(t[0], t[1], 0x0040), __byte_perm(t[2], t[3], 0x0040), 0x5410);
  w1 = __byte_perm(__byte_perm(t[4], t[5], 0x0040), __byte_perm(t[6], t[7], 0x0040), 0x5410);
  if (OFFSET) { w0 ^= 0x80808080u; w1 ^= 0x80808080u; }
}
__device__ __forceinline__ void tail8_fp8(const uint32_t (&v)[4], uint32_t& w0, uint32_t& w1) {
  uint32_t h[4];
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(__uint_as_float(v[p] & 0xFFFF0000u)),
        "f"(__uint_as_float(v[p] << 16)));
    h[p] = r;
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
__device__ __forceinline__ uint32_t nvfp4_8(const uint4& raw, float rs, bool& unsafe, float margin = 0x1p-21f) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  // both ends of an interval that holds the exact quotient (reciprocal, its scaling and the
  // product each round by 2^-23 or less; the margin is 2^-21 unless the caller's reciprocal is
  // looser).  The fused "+ 0" turns a -0.0 weight into +0 like the reference's "+ zero_point".
  const float rlo = rs * (1.0f - margin), rhi = rs * (1.0f + margin);
  float lo[8], hi[8];
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    const float x0 = __uint_as_float(w[p] << 16), x1 = __uint_as_float(w[p] & 0xFFFF0000u);
    fma2_f32(x0, x1, rlo, 0.0f, lo[2 * p], lo[2 * p + 1]);
    fma2_f32(x0, x1, rhi, 0.0f, hi[2 * p], hi[2 * p + 1]);
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
// Range of a group for calculate_qparams, which clamps it to contain zero first: bf16 bit
// patterns order like unsigned integers among negative values (the larger pattern is the more
// negative number, and every negative pattern is above every positive one) and like signed
// integers among positive values, so one packed unsigned maximum finds the minimum if it is
// negative and one packed signed maximum finds the maximum if it is positive; whatever they
// return otherwise has the other sign and is replaced by zero by the clamp.  Three inputs per
// instruction (VIMNMX3): 4 instructions per chunk of 8 elements.
struct RangeQ {
  uint32_t umax, smax;
  __device__ __forceinline__ void first(const uint4& raw) {
    umax = __vimax3_u16x2(raw.x, raw.y, raw.z); umax = __vimax3_u16x2(umax, raw.w, raw.w);
    smax = (uint32_t)__vimax3_s16x2(raw.x, raw.y, raw.z); smax = (uint32_t)__vimax3_s16x2(smax, raw.w, raw.w);
  }
  __device__ __forceinline__ void add(const uint4& raw) {
    umax = __vimax3_u16x2(umax, raw.x, raw.y); umax = __vimax3_u16x2(umax, raw.z, raw.w);
    smax = (uint32_t)__vimax3_s16x2(smax, raw.x, raw.y); smax = (uint32_t)__vimax3_s16x2(smax, raw.z, raw.w);
  }
  // (lo, hi): equal to the group's min / max after both are clamped to contain zero
  __device__ __forceinline__ void finish(float& lo, float& hi) const {
    const uint32_t u = max(umax & 0xFFFFu, umax >> 16);
    const int sv = max((int)(short)(smax & 0xFFFFu), (int)(short)(smax >> 16));
    lo = fminf(__uint_as_float(u << 16), 0.0f);
    hi = fmaxf(__uint_as_float((uint32_t)sv << 16), 0.0f);
  }
};
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

// Codes of one chunk with one (scale, zp), exact element-wise path.
// (out of line, arguments and result by value: the packed paths must not be forced onto the stack)
template <int MODE, bool CB>
__device__ __noinline__ uint2 chunk_codes_exact(uint4 raw, float se, float z, QRange qr) {
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
  return make_uint2(a, b);
}

// Codes of one chunk, packed path for a bf16 scale without a global scale (g.slow must be false).
//   POW2    the scale is a power of two (MX formats)
//   HAS_ZP  a zero point has to be added
//   OWN_SYM the scale was derived from this very group's range by a symmetric scheme, so the
//           quotients cannot fall below qmin - 1/2 and only the upper clamp is needed
template <int MODE, bool POW2, bool HAS_ZP, bool OWN_SYM>
__device__ __forceinline__ void chunk_codes_packed(const uint4& raw, const GroupQ& g, const QRange& qr, uint32_t& w0,
                                                   uint32_t& w1) {
  uint32_t v[4];
  quot8_bf16<POW2>(raw, g, v);
  if (HAS_ZP) {
#pragma unroll
    for (int p = 0; p < 4; ++p) v[p] = bf2_add(v[p], g.z2);
  }
  if constexpr (MODE == kFp4) {
    w0 = tail8_fp4(v);             // the converter saturates at +-6
  } else if constexpr (MODE == kInt4) {
    const uint32_t lo2 = bf2_splat(qr.qmin), hi2 = bf2_splat(qr.qmax);
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      if (!OWN_SYM) v[p] = bf2_max(v[p], lo2);
      v[p] = bf2_min(v[p], hi2);
    }
    w0 = tail8_int4(v);
  } else if (qr.kind == kFp8) {
    tail8_fp8(v, w0, w1);          // the converter saturates at +-448
  } else {
    const uint32_t lo2 = bf2_splat(qr.qmin), hi2 = bf2_splat(qr.qmax);
#pragma unroll
    for (int p = 0; p < 4; ++p) v[p] = bf2_min(bf2_max(v[p], lo2), hi2);
    tail8_int8<MODE == kInt8Word>(v, w0, w1);
  }
}

// R chunks of one lane that share (scale, zp) -> codes a[k] (and b[k] for byte codes).
template <int MODE, bool GLOBAL, bool SCALE_BF16, int R, bool POW2, bool HAS_ZP, bool OWN_SYM>
__device__ __forceinline__ void lane_codes(const uint4 (&raw)[R], const GroupQ& g, const QRange& qr, uint32_t (&a)[R],
                                           uint32_t (&b)[R]) {
  constexpr bool CB = SCALE_BF16 && !GLOBAL;
#pragma unroll
  for (int k = 0; k < R; ++k) { a[k] = 0; b[k] = 0; }
  if (g.slow || (!CB && MODE != kFp4)) {
#pragma unroll
    for (int k = 0; k < R; ++k) {
      const uint2 r = chunk_codes_exact<MODE, CB>(raw[k], g.se, g.z, qr);
      a[k] = r.x; b[k] = r.y;
    }
    return;
  }
  if constexpr (!CB) {
    // NVFP4: float32 effective scale, interval test per chunk
#pragma unroll
    for (int k = 0; k < R; ++k) {
      bool unsafe;
      a[k] = nvfp4_8(raw[k], g.rs, unsafe);
      if (unsafe) {
        const uint2 r = chunk_codes_exact<MODE, CB>(raw[k], g.se, g.z, qr);
        a[k] = r.x; b[k] = r.y;
      }
    }
  } else {
#pragma unroll
    for (int k = 0; k < R; ++k) chunk_codes_packed<MODE, POW2, HAS_ZP, OWN_SYM>(raw[k], g, qr, a[k], b[k]);
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
  // group measured 0.41 of the HBM peak against 0.60-0.65).  For 128-element groups 4 lanes x 4
  // chunks measured best (82 us for 8 x 2, 68 for 4 x 4, 75 for 2 x 8, 123 for 1 x 16 on a
  // 16384 x 8192 matrix): a load instruction of 4 lanes covers half a 128-byte line.
  s.R = chunks >= 16 ? 8 : (chunks >= 8 ? 4 : chunks);
  if (s.R > rmax) s.R = rmax;
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

// Stores of a lane's R code words (chunk c0 + k * L of the row) and of its R loads: with L known at
// compile time every address is the slot's base plus an immediate.
template <int MODE, int R, int L>
__device__ __forceinline__ void store_lane_strided(void* out, int64_t wi0, const uint32_t (&a)[R], const uint32_t (&b)[R]) {
  if constexpr (L == 1) {
    store_lane_codes<MODE, R>(out, wi0, a, b);
  } else if constexpr (MODE == kInt4 || MODE == kFp4) {
    uint32_t* o = (uint32_t*)out + wi0;
#pragma unroll
    for (int k = 0; k < R; ++k) o[k * L] = a[k];
  } else {
    uint2* o = reinterpret_cast<uint2*>(out) + wi0;
#pragma unroll
    for (int k = 0; k < R; ++k) o[k * L] = make_uint2(a[k], b[k]);
  }
}

// MODE, GLOBAL as above; R chunks per lane, L lanes per group (compile-time: g = 8 * R * L).
template <int MODE, bool GLOBAL, int R, int L>
__global__ void __launch_bounds__(kThreads) rtn_group_bf16_kernel(
    const void* __restrict__ W, int N, int K, int64_t ldw, int tx_log2, QParamCfg qc, QRange qr,
    const float* __restrict__ gscale, void* __restrict__ scale_out, void* __restrict__ zp_out,
    uint8_t* __restrict__ scale_store, void* __restrict__ out) {
  using T = __nv_bfloat16;
  constexpr int cpg = R * L;                  // chunks per group
  const float gs = GLOBAL ? *gscale : 1.0f;
  const int TX = 1 << tx_log2, rows = kThreads >> tx_log2;
  const int tx = threadIdx.x & (TX - 1), ty = threadIdx.x >> tx_log2;
  const int cpr = K >> 3, gpr = cpr / cpg;
  const int slots = gpr * L;                  // thread slots per row
  const int send = (slots + 31) & ~31;
  const bool mx = qc.scale_kind == B200Q_SCALE_E8M0, sym = qc.symmetric != 0;
  for (int row = blockIdx.x * rows + ty; row < N; row += gridDim.x * rows) {
    const T* wrow = (const T*)W + (int64_t)row * ldw;
    for (int t = tx; t < send; t += TX) {
      const bool live = t < slots;
      const int grp = t / L, j = t % L;
      const int c0 = grp * cpg + j;           // first chunk of this lane
      uint4 raw[R];
      {
        const uint4* src = reinterpret_cast<const uint4*>(wrow) + c0;
#pragma unroll
        for (int k = 0; k < R; ++k) raw[k] = live ? ldg_stream(src + k * L) : make_uint4(0, 0, 0, 0);
      }
      RangeQ mm;
      mm.first(raw[0]);
#pragma unroll
      for (int k = 1; k < R; ++k) mm.add(raw[k]);
      float lo, hi;
      mm.finish(lo, hi);
#pragma unroll
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
      const GroupQ gq = make_group_q<!GLOBAL>(GLOBAL ? __fdiv_rn(s, gs) : s, z);
      uint32_t a[R], b[R];
      if (GLOBAL) lane_codes<MODE, true, true, R, false, false, false>(raw, gq, qr, a, b);
      else if (mx) lane_codes<MODE, false, true, R, true, false, true>(raw, gq, qr, a, b);
      else if (sym) lane_codes<MODE, false, true, R, false, false, true>(raw, gq, qr, a, b);
      else lane_codes<MODE, false, true, R, false, true, false>(raw, gq, qr, a, b);
      store_lane_strided<MODE, R, L>(out, (int64_t)row * cpr + c0, a, b);
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
            {
              const uint4 one[1] = {raw[h]};
              uint32_t a1[1], b1[1];
              const GroupQ gq = make_group_q<ES::is_bf16 && !GLOBAL>(s, z);
              if (zp) lane_codes<MODE, GLOBAL, ES::is_bf16, 1, false, true, false>(one, gq, qr, a1, b1);
              else lane_codes<MODE, GLOBAL, ES::is_bf16, 1, false, false, false>(one, gq, qr, a1, b1);
              w0 = a1[0]; w1 = b1[0];
            }
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
template <int SDT, bool GLOBAL, int MODE, int R, int L>
__global__ void __launch_bounds__(kThreads) quant_group_bf16_kernel(
    const void* __restrict__ W, int N, int K, int64_t ldw, int tx_log2,
    const void* __restrict__ scale, const void* __restrict__ zp, int zp_kind, const float* __restrict__ gscale,
    QRange qr, void* __restrict__ out) {
  using T = __nv_bfloat16;
  using ES = Elem<SDT>;
  constexpr int cpg = R * L;
  const float gs = GLOBAL ? *gscale : 1.0f;
  const int TX = 1 << tx_log2, rows = kThreads >> tx_log2;
  const int tx = threadIdx.x & (TX - 1), ty = threadIdx.x >> tx_log2;
  const int cpr = K >> 3, gpr = cpr / cpg;
  const int slots = gpr * L;
  for (int row = blockIdx.x * rows + ty; row < N; row += gridDim.x * rows) {
    const T* wrow = (const T*)W + (int64_t)row * ldw;
    for (int t = tx; t < slots; t += TX) {
      const int grp = t / L, j = t % L;
      const int c0 = grp * cpg + j;
      uint4 raw[R];
      {
        const uint4* src = reinterpret_cast<const uint4*>(wrow) + c0;
#pragma unroll
        for (int k = 0; k < R; ++k) raw[k] = ldg_stream(src + k * L);
      }
      const int64_t pi = (int64_t)row * gpr + grp;
      float s = ES::load((const typename ES::type*)scale + pi);
      if (GLOBAL) s = __fdiv_rn(s, gs);
      const float z = zp ? load_zp(zp, zp_kind, pi) : 0.0f;
      const GroupQ gq = make_group_q<ES::is_bf16 && !GLOBAL>(s, z);
      uint32_t a[R], b[R];
      if (zp) lane_codes<MODE, GLOBAL, ES::is_bf16, R, false, true, false>(raw, gq, qr, a, b);
      else lane_codes<MODE, GLOBAL, ES::is_bf16, R, false, false, false>(raw, gq, qr, a, b);
      store_lane_strided<MODE, R, L>(out, (int64_t)row * cpr + c0, a, b);
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
  int par = 0;
  for (int row = blockIdx.x; row < N; row += gridDim.x, par ^= 1) {
    const T* wrow = (const T*)W + (int64_t)row * ldw;
    uint4 raw[R];
#pragma unroll
    for (int k = 0; k < R; ++k) {
      const int c = threadIdx.x + k * kThreads;
      raw[k] = (c < cpr) ? ldg_stream(wrow + (int64_t)c * 8) : make_uint4(0, 0, 0, 0);
    }
    // chunks beyond the row are zeros, which the range contains anyway
    float lo, hi;
    {
      RangeQ mm;
      mm.first(raw[0]);
#pragma unroll
      for (int k = 1; k < R; ++k) mm.add(raw[k]);
      mm.finish(lo, hi);
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
    const GroupQ gq = make_group_q<true>(s, z);
    uint32_t a[R], b[R];
    if (qc.symmetric) lane_codes<MODE, false, true, R, false, false, true>(raw, gq, qr, a, b);
    else lane_codes<MODE, false, true, R, false, true, false>(raw, gq, qr, a, b);
#pragma unroll
    for (int k = 0; k < R; ++k) {
      const int c = threadIdx.x + k * kThreads;
      if (c < cpr) {
        const int64_t wi = (int64_t)row * cpr + c;
        if (MODE == kInt4 || MODE == kFp4) ((uint32_t*)out)[wi] = a[k];
        else reinterpret_cast<uint2*>(out)[wi] = make_uint2(a[k], b[k]);
      }
    }
  }
}

}  // namespace stream
}  // namespace b200q
