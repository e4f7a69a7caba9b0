// Shared host/device helpers of the b200q kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "../../include/b200q.h"

namespace b200q {

constexpr int kNumSMs = 148;  // B200: 2 dies x 74 SMs

// ---- host side -------------------------------------------------------------------------
void set_last_error(const char* what, cudaError_t e);
inline int cuda_status(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return B200Q_OK;
  set_last_error(what, e);
  return B200Q_ERR_CUDA;
}
#define B200Q_TRY(expr)                                      \
  do {                                                       \
    int _st = b200q::cuda_status((expr), #expr);             \
    if (_st != B200Q_OK) return _st;                         \
  } while (0)
// every kernel launch is followed by this check; it also feeds b200q_launch_count()
void count_launch();
#define B200Q_LAUNCH_CHECK()          \
  do {                                \
    b200q::count_launch();            \
    B200Q_TRY(cudaGetLastError());    \
  } while (0)

// Grid size for a grid-stride kernel: whole multiples of the SM count, capped by the work.
inline int grid_for(int64_t blocks_needed, int blocks_per_sm) {
  int64_t cap = (int64_t)kNumSMs * blocks_per_sm;
  if (blocks_needed >= cap) return (int)cap;
  return blocks_needed < 1 ? 1 : (int)blocks_needed;
}

// ---- element types ---------------------------------------------------------------------
template <int DT> struct Elem;
template <> struct Elem<B200Q_BF16> {
  using type = __nv_bfloat16;
  static constexpr bool is_bf16 = true;
  __device__ static __forceinline__ float load(const type* p) { return __bfloat162float(*p); }
  __device__ static __forceinline__ void store(type* p, float v) { *p = __float2bfloat16_rn(v); }
  // rounding of an fp32 intermediate to this dtype, kept in a float register
  __device__ static __forceinline__ float rnd(float v) {
    return __bfloat162float(__float2bfloat16_rn(v));
  }
};
template <> struct Elem<B200Q_F32> {
  using type = float;
  static constexpr bool is_bf16 = false;
  __device__ static __forceinline__ float load(const type* p) { return *p; }
  __device__ static __forceinline__ void store(type* p, float v) { *p = v; }
  __device__ static __forceinline__ float rnd(float v) { return v; }
};

__device__ __forceinline__ float bf16r(float v) {
  return __bfloat162float(__float2bfloat16_rn(v));
}
template <bool BF> __device__ __forceinline__ float rnd_if(float v) {
  return BF ? bf16r(v) : v;
}

// ---- rounding rules of the code types ------------------------------------------------------
// FP8 E4M3 (finite, saturating) round-to-nearest-even, value kept as float.
__device__ __forceinline__ uint8_t e4m3_bits(float v) {
  return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}
__device__ __forceinline__ float e4m3_value(uint8_t b) {
  __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
  return __half2float(__half(h));
}
__device__ __forceinline__ float e4m3_round(float v) { return e4m3_value(e4m3_bits(v)); }

// FP4 E2M1 value set {0,.5,1,1.5,2,3,4,6}; ties go to the entry with an even mantissa bit;
// the sign is re-applied by multiplication, so a negative input that rounds to zero gives -0.0
// and a zero input of either sign gives +0.0.
__device__ __forceinline__ float e2m1_round(float v) {
  float a = fabsf(v), r;
  if (a <= 0.25f) r = 0.0f;
  else if (a < 0.75f) r = 0.5f;
  else if (a <= 1.25f) r = 1.0f;
  else if (a < 1.75f) r = 1.5f;
  else if (a <= 2.5f) r = 2.0f;
  else if (a < 3.5f) r = 3.0f;
  else if (a <= 5.0f) r = 4.0f;
  else r = 6.0f;
  float s = (v > 0.0f) ? 1.0f : ((v < 0.0f) ? -1.0f : 0.0f);
  return r * s;
}
// 4-bit storage code of an E2M1 value: table index | sign bit << 3 (-0.0 -> 0x8).
__device__ __forceinline__ uint32_t e2m1_nibble(float q) {
  float a = fabsf(q);
  uint32_t idx = (a < 0.25f) ? 0u : (a < 0.75f) ? 1u : (a < 1.25f) ? 2u : (a < 1.75f) ? 3u
               : (a < 2.5f) ? 4u : (a < 3.5f) ? 5u : (a < 5.0f) ? 6u : 7u;
  return idx | ((__float_as_uint(q) >> 31) << 3);
}

enum CodeKind { kInt = 0, kFp8 = 1, kFp4 = 2 };

struct QRange {
  float qmin, qmax;
  int kind;  // CodeKind
};
inline int make_qrange(const b200q_qargs* qa, QRange* r) {
  if (qa->qtype == B200Q_QINT) {
    if (qa->num_bits < 2 || qa->num_bits > 8) return B200Q_ERR_UNSUPPORTED;
    float half = (float)(1 << (qa->num_bits - 1));
    r->qmin = -half; r->qmax = half - 1.0f; r->kind = kInt;
  } else if (qa->qtype == B200Q_QFLOAT && qa->num_bits == 8) {
    r->qmin = -448.0f; r->qmax = 448.0f; r->kind = kFp8;
  } else if (qa->qtype == B200Q_QFLOAT && qa->num_bits == 4) {
    r->qmin = -6.0f; r->qmax = 6.0f; r->kind = kFp4;
  } else {
    return B200Q_ERR_UNSUPPORTED;
  }
  return B200Q_OK;
}

// x / s + zp -> clamp -> round.  CB: the arithmetic dtype is bf16 (x and effective scale are
// both bf16), otherwise float32; intermediate roundings follow torch's bf16 element-wise ops.
// The zero point is always added (0 for symmetric schemes), as the reference does: that turns
// a -0.0 quotient into +0.0.
__device__ __forceinline__ float round_code(float v, QRange r) {
  v = fminf(fmaxf(v, r.qmin), r.qmax);
  if (r.kind == kInt) return rintf(v);
  if (r.kind == kFp8) return e4m3_round(v);
  return e2m1_round(v);
}
template <bool CB>
__device__ __forceinline__ float quant_code(float x, float s, float zp, QRange r) {
  float v = rnd_if<CB>(__fdiv_rn(x, s));
  v = rnd_if<CB>(v + zp);
  return round_code(v, r);
}
// Same result as quant_code<CB>(x, s, zp, r) given rs = 1/s to within an ulp.  The quotient is
// formed as x*rs (a few ulp off); the IEEE division is redone only when that product lies so
// close to a rounding boundary that those ulps could change the outcome (a few times in 1e4).
template <bool CB>
__device__ __forceinline__ float quant_code_fast(float x, float s, float rs, float zp, QRange r) {
  const float qa = x * rs;
  const float aq = fabsf(qa);
  bool safe = (aq < 1e30f) && (aq > 1e-30f || aq == 0.0f);
  if (CB) {
    // bf16 rounding midpoints sit at low half-word 0x8000; keep 16 float ulps away from them
    const uint32_t low = __float_as_uint(qa) & 0xFFFFu;
    safe = safe && ((low - 0x7FF0u) > 0x20u);
    if (safe) return round_code(bf16r(bf16r(qa) + zp), r);
  } else if (safe) {
    // the code is a monotone function of the quotient: equal codes at both ends of an
    // interval that contains the exact quotient settle it
    const float a = round_code(qa * (1.0f - 0x1p-20f) + zp, r);
    const float b = round_code(qa * (1.0f + 0x1p-20f) + zp, r);
    if (a == b) return a;   // both ends have the sign of qa, so this is also the code's sign of zero
  }
  return quant_code<CB>(x, s, zp, r);
}
// round_code with the code type known at compile time
template <int KIND>
__device__ __forceinline__ float round_code_k(float v, float qmin, float qmax) {
  v = fminf(fmaxf(v, qmin), qmax);
  if constexpr (KIND == kInt) return rintf(v);
  else if constexpr (KIND == kFp8) return e4m3_round(v);
  else return e2m1_round(v);
}
// (q - zp) * s in the scale's dtype (SB: bf16).
template <bool SB>
__device__ __forceinline__ float dequant_code(float q, float s, float zp) {
  float d = rnd_if<SB>(q - zp);
  return rnd_if<SB>(d * s);
}

// Fake-quantised value of a float32 weight, as the GPTQ sweep needs it once per column on its
// critical path: the same result as dequant_code<SB>(quant_code<false>(x, s, zp, r), s, zp), with
// the code type a compile-time constant and the division replaced by the product with rs = 1/s
// whenever both ends of a 2^-20 interval around it give the same code (else the division is redone).
template <int KIND, bool SB>
__device__ __forceinline__ float fake_quant_f32(float x, float s, float rs, float zp, float qmin, float qmax) {
  const float qa = x * rs;
  const float aq = fabsf(qa);
  const float a = round_code_k<KIND>(fmaf(qa, 1.0f - 0x1p-20f, zp), qmin, qmax);
  const float b = round_code_k<KIND>(fmaf(qa, 1.0f + 0x1p-20f, zp), qmin, qmax);
  float q = a;   // both ends have the sign of qa, so this is also the code's sign of zero
  if (!((aq < 1e30f) && (aq > 1e-30f || aq == 0.0f) && (a == b)))
    q = round_code_k<KIND>(__fdiv_rn(x, s) + zp, qmin, qmax);
  if constexpr (KIND == kInt) {
    // an integer code minus an integer zero point is at most 255 in magnitude: exact in bf16 too,
    // so only the product with the scale is rounded
    return rnd_if<SB>((q - zp) * s);
  }
  return dequant_code<SB>(q, s, zp);
}

__device__ __forceinline__ float load_zp(const void* zp, int zp_kind, int64_t i) {
  if (zp_kind == B200Q_ZP_INT8) return (float)((const int8_t*)zp)[i];
  if (zp_kind == B200Q_ZP_UINT8) return (float)((const uint8_t*)zp)[i];
  return e4m3_value(((const uint8_t*)zp)[i]);
}

// Index of the scale / zero point that governs element (row, col).
struct ParamMap {
  int strategy;
  int group_size;
  int block_h, block_w;
  int64_t groups_per_row;   // GROUP: K/g ; BLOCK: number of block columns
  const int32_t* g_idx;     // optional column -> group map
  __device__ __forceinline__ int64_t index(int64_t row, int64_t col) const {
    switch (strategy) {
      case B200Q_TENSOR: return 0;
      case B200Q_CHANNEL: return row;
      case B200Q_BLOCK: return (int64_t)((int)row / block_h) * groups_per_row + (int)col / block_w;
      default: {
        int64_t g = g_idx ? (int64_t)g_idx[col] : (int64_t)((int)col / group_size);
        return row * groups_per_row + g;
      }
    }
  }
};
inline int make_param_map(const b200q_qargs* qa, int64_t N, int64_t K, const int32_t* g_idx,
                          ParamMap* m) {
  m->strategy = qa->strategy; m->group_size = qa->group_size;
  m->block_h = qa->block_h; m->block_w = qa->block_w; m->g_idx = g_idx; m->groups_per_row = 1;
  switch (qa->strategy) {
    case B200Q_TENSOR: case B200Q_CHANNEL: break;
    case B200Q_GROUP: case B200Q_TENSOR_GROUP:
      if (qa->group_size <= 0) return B200Q_ERR_ARG;
      m->groups_per_row = (K + qa->group_size - 1) / qa->group_size; break;
    case B200Q_BLOCK:
      if (qa->block_h <= 0 || qa->block_w <= 0) return B200Q_ERR_ARG;
      m->groups_per_row = (K + qa->block_w - 1) / qa->block_w; break;
    default: return B200Q_ERR_ARG;
  }
  return B200Q_OK;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

}  // namespace b200q
