// MSE shrink-grid observer: all shrink candidates evaluated in one pass over the weight.
//
// For each group the elements stay in registers (GROUP strategies) or shared memory
// (CHANNEL) while every candidate p = 1 - i/grid is tried: qparams from (p*min, p*max),
// fake-quantise, sum |q - x|^norm, keep the strictly smallest.  Arithmetic is done in the
// weight's dtype step by step (bf16 weights: every elementwise result is rounded to bf16,
// sums are accumulated in float32 and rounded once), like the element-wise torch ops of the
// reference.  The reference stops the whole search once `patience` consecutive candidates
// improved no group anywhere; pass 1 records per candidate whether any group improved, a
// one-thread kernel derives the stopping step, and pass 2 (a no-op unless the search stops
// early) repeats the search up to that step.
#include "common.cuh"

#include <string.h>

#include <mutex>

namespace b200q {
namespace mse {

struct Cfg {
  int symmetric, scale_kind, zp_kind, mx_offset;
  float qmin, qmax, half_range, range, eps;
  int kind;
  int steps, patience;
  double grid;
  float norm, expand;
};

// qparams of calculate_qparams without a global scale, in dtype T (TB: bf16).
template <bool TB>
__device__ __forceinline__ void qparams_local(float mn, float mx, const Cfg& c, float& s, float& zp) {
  mn = fminf(mn, 0.0f);
  mx = fmaxf(mx, 0.0f);
  if (c.symmetric) {
    float amax = fmaxf(fabsf(mn), fabsf(mx));
    if (c.scale_kind == B200Q_SCALE_E8M0) {
      int biased;
      if (TB) { uint32_t b = __float_as_uint(amax) >> 16; b = (b + 32u) & 0xFF80u; biased = (int)((b >> 7) & 0xFFu); }
      else { uint32_t b = __float_as_uint(amax); b = (b + (1u << 21)) & 0xFF800000u; biased = (int)((b >> 23) & 0xFFu); }
      float e = (biased == 0) ? 0.0f : fminf(fmaxf((float)(biased - c.mx_offset), 0.0f), 255.0f);
      s = __uint_as_float(e >= 1.0f ? ((uint32_t)e << 23) : 0x00400000u);
    } else {
      s = rnd_if<TB>(__fdiv_rn(amax, c.half_range));
      if (c.scale_kind == B200Q_SCALE_FP8) s = e4m3_round(fminf(fmaxf(s, -448.0f), 448.0f));
    }
    zp = 0.0f;
  } else {
    float d = rnd_if<TB>(mx - mn);
    s = rnd_if<TB>(__fdiv_rn(d, c.range));
    float z = rnd_if<TB>(__fdiv_rn(mn, s));
    z = rnd_if<TB>(c.qmin - z);
    // 0/0 for an all-zero group: torch's clamp keeps the NaN and the integer cast makes it 0
    zp = (z != z) ? 0.0f : fminf(fmaxf(z, c.qmin), c.qmax);
  }
  if (s == 0.0f) s = c.eps;
  if (c.zp_kind == B200Q_ZP_INT8) zp = rintf(fminf(fmaxf(zp, -128.0f), 127.0f));
  else if (c.zp_kind == B200Q_ZP_UINT8) zp = rintf(fminf(fmaxf(zp, 0.0f), 255.0f));
  else zp = e4m3_round(fminf(fmaxf(zp, -448.0f), 448.0f));
}

template <bool TB>
__device__ __forceinline__ float elem_error(float x, float s, float z, const Cfg& c) {
  QRange qr{c.qmin, c.qmax, c.kind};
  float q = quant_code<TB>(x, s, z, qr);
  float fq = dequant_code<TB>(q, s, z);
  float d = rnd_if<TB>(fabsf(rnd_if<TB>(fq - x)));
  float e = (d == 0.0f) ? 0.0f : powf(d, c.norm);
  return rnd_if<TB>(e);
}

__device__ __forceinline__ float shrink_factor(int i, double grid) {
  return (float)(1.0 - (double)i / grid);
}

// ctl[0] = number of steps to run, ctl[1..] = per-step "some group improved" flags
template <int DT>
__global__ void __launch_bounds__(256) mse_group_kernel(const void* __restrict__ W, int64_t N, int64_t K,
                                                        int64_t ldw, int g, Cfg c, int* __restrict__ ctl,
                                                        int pass, void* __restrict__ mn_out,
                                                        void* __restrict__ mx_out) {
  using E = Elem<DT>;
  using T = typename E::type;
  constexpr bool TB = E::is_bf16;
  const int limit = (pass == 0) ? c.steps : ctl[0];
  if (pass == 1 && limit >= c.steps) return;  // the search never stopped early
  const int lanes = g >> 3;
  const int64_t cpr = K >> 3, total = N * cpr, gpr = K / g;
  for (int64_t ch = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; ch < ((total + 31) & ~31LL);
       ch += (int64_t)gridDim.x * blockDim.x) {
    const bool live = ch < total;
    float v[8];
    float lo = INFINITY, hi = -INFINITY;
    int64_t row = 0, cc = 0;
    if (live) {
      row = ch / cpr; cc = ch - row * cpr;
      const T* src = (const T*)W + row * ldw + cc * 8;
#pragma unroll
      for (int i = 0; i < 8; ++i) { v[i] = E::load(src + i); lo = fminf(lo, v[i]); hi = fmaxf(hi, v[i]); }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = 0.0f;
    }
    for (int o = lanes >> 1; o > 0; o >>= 1) {
      lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
      hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
    }
    const float mn = rnd_if<TB>(lo * c.expand), mx = rnd_if<TB>(hi * c.expand);
    float best_err = TB ? 3.3895313892515355e38f : 3.402823466e38f;  // finfo(dtype).max
    float best_mn = mn, best_mx = mx;
    for (int i = 0; i < limit; ++i) {
      const float p = shrink_factor(i, c.grid);
      const float smn = rnd_if<TB>(mn * p), smx = rnd_if<TB>(mx * p);
      float s, z;
      qparams_local<TB>(smn, smx, c, s, z);
      float err = 0.0f;
#pragma unroll
      for (int e = 0; e < 8; ++e) err += elem_error<TB>(v[e], s, z, c);
      for (int o = lanes >> 1; o > 0; o >>= 1) err += __shfl_xor_sync(0xffffffffu, err, o);
      err = rnd_if<TB>(err);
      if (live && err < best_err) {
        best_err = err; best_mn = smn; best_mx = smx;
        if (pass == 0 && (cc % lanes) == 0 && ((volatile int*)ctl)[1 + i] == 0) atomicOr(&ctl[1 + i], 1);
      }
    }
    if (live && (cc % lanes) == 0) {
      int64_t gi = row * gpr + (cc * 8) / g;
      E::store((T*)mn_out + gi, best_mn);
      E::store((T*)mx_out + gi, best_mx);
    }
  }
}

// ---------------------------------------------------------------------------------------
// bf16 weights, integer codes, GROUP strategies: the same search with packed bf16x2 arithmetic.
// torch evaluates the candidate with element-wise bf16 ops; for bf16 operands a packed
// HADD2 / HMUL2 gives exactly the rounded result of the float32 operation followed by a
// rounding to bf16 (the _rn forms of the intrinsics: the plain ones let the compiler fuse the
// product and the subtraction into one FMA with a single rounding), so add-zero-point, clamp, round-to-integer (magic number 192 for 4 bits,
// h2rint otherwise), dequantise, subtract and abs run two elements per instruction.  The two
// places where float32 is needed keep an exact fallback: the quotient x/s is formed as x*(1/s)
// and the power as exp2(norm*log2 d); a lane whose value lies within a few float ulps of a bf16
// rounding midpoint (3 ulps for the quotient, 192 for the power, twice the error bound of the
// MUFU functions at these magnitudes) recomputes that element with the IEEE division / powf.
__device__ __forceinline__ uint32_t bf2_of(float v) {
  __nv_bfloat162 r = __float2bfloat162_rn(v);
  return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t bf2_pack(float hi, float lo) {
  uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}
#define B200Q_BF2(op, a, b) ([&] { __nv_bfloat162 r_ = op(*reinterpret_cast<const __nv_bfloat162*>(&(a)), \
                                                         *reinterpret_cast<const __nv_bfloat162*>(&(b)));   \
                                   return *reinterpret_cast<uint32_t*>(&r_); }())

template <bool FOUR_BIT>
__global__ void __launch_bounds__(256) mse_group_bf16_int_kernel(const void* __restrict__ W, int64_t N, int64_t K,
                                                                 int64_t ldw, int g, Cfg c, int* __restrict__ ctl,
                                                                 int pass, void* __restrict__ mn_out,
                                                                 void* __restrict__ mx_out) {
  using T = __nv_bfloat16;
  __shared__ float s_shrink[1024];
  const int limit = (pass == 0) ? c.steps : ctl[0];
  if (pass == 1 && limit >= c.steps) return;  // the search never stopped early
  for (int i = threadIdx.x; i < limit; i += blockDim.x) s_shrink[i] = shrink_factor(i, c.grid);
  __syncthreads();
  const int lanes = g >> 3;
  const int64_t cpr = K >> 3, total = N * cpr, gpr = K / g;
  const QRange qr{c.qmin, c.qmax, c.kind};
  const uint32_t qmin2 = bf2_of(c.qmin), qmax2 = bf2_of(c.qmax), magic = 0x43404340u;  // {192, 192}
  for (int64_t ch = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; ch < ((total + 31) & ~31LL);
       ch += (int64_t)gridDim.x * blockDim.x) {
    const bool live = ch < total;
    uint32_t w[4] = {0u, 0u, 0u, 0u};
    float lo = INFINITY, hi = -INFINITY;
    int64_t row = 0, cc = 0;
    if (live) {
      row = ch / cpr; cc = ch - row * cpr;
      const uint4 raw = *reinterpret_cast<const uint4*>((const T*)W + row * ldw + cc * 8);
      w[0] = raw.x; w[1] = raw.y; w[2] = raw.z; w[3] = raw.w;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float a = __uint_as_float(w[k] << 16), b = __uint_as_float(w[k] & 0xFFFF0000u);
        lo = fminf(lo, fminf(a, b)); hi = fmaxf(hi, fmaxf(a, b));
      }
    }
    for (int o = lanes >> 1; o > 0; o >>= 1) {
      lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
      hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
    }
    const float mn = bf16r(lo * c.expand), mx = bf16r(hi * c.expand);
    float best_err = 3.3895313892515355e38f;  // finfo(bfloat16).max
    float best_mn = mn, best_mx = mx;
    for (int i = 0; i < limit; ++i) {
      const float p = s_shrink[i];
      const float smn = bf16r(mn * p), smx = bf16r(mx * p);
      float s, z;
      qparams_local<true>(smn, smx, c, s, z);
      const float rs = __frcp_rn(s);
      const uint32_t s2 = bf2_of(s), z2 = bf2_of(z);
      float err = 0.0f;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float x0 = __uint_as_float(w[k] << 16), x1 = __uint_as_float(w[k] & 0xFFFF0000u);
        const float q0 = x0 * rs, q1 = x1 * rs;
        // quotients within 3 ulps of a bf16 midpoint (half-word 0x8000) take the IEEE division
        const uint32_t mq = (__byte_perm(__float_as_uint(q0), __float_as_uint(q1), 0x5410) + 0x80048004u) & 0xFFF0FFF0u;
        uint32_t cq = bf2_pack(q1, q0);
        if (((mq & 0xFFFFu) == 0u) || ((mq >> 16) == 0u))
          cq = bf2_pack(bf16r(__fdiv_rn(x1, s)), bf16r(__fdiv_rn(x0, s)));
        uint32_t v = c.symmetric ? cq : B200Q_BF2(__hadd2_rn, cq, z2);
        v = B200Q_BF2(__hmax2, v, qmin2);
        v = B200Q_BF2(__hmin2, v, qmax2);
        if (FOUR_BIT) {
          v = B200Q_BF2(__hadd2_rn, v, magic);   // integers are 1 apart in [128, 256): rounds to nearest even
          v = B200Q_BF2(__hsub2_rn, v, magic);
        } else {
          __nv_bfloat162 r_ = h2rint(*reinterpret_cast<const __nv_bfloat162*>(&v));
          v = *reinterpret_cast<uint32_t*>(&r_);
        }
        if (!c.symmetric) v = B200Q_BF2(__hsub2_rn, v, z2);
        v = B200Q_BF2(__hmul2_rn, v, s2);
        v = B200Q_BF2(__hsub2_rn, v, w[k]);
        v &= 0x7FFF7FFFu;   // |.|
        const float d0 = __uint_as_float(v << 16), d1 = __uint_as_float(v & 0xFFFF0000u);
        float e0 = exp2f(c.norm * __log2f(d0)), e1 = exp2f(c.norm * __log2f(d1));
        e0 = (d0 == 0.0f) ? 0.0f : e0;
        e1 = (d1 == 0.0f) ? 0.0f : e1;
        // powers within 192 ulps of a bf16 midpoint, or outside the range where the MUFU error
        // bounds hold, are recomputed with powf
        const uint32_t l0 = __float_as_uint(e0) & 0xFFFFu, l1 = __float_as_uint(e1) & 0xFFFFu;
        // (|log2 d| <= 20 keeps the error of norm * log2 d below 80 ulps of the result)
        if ((d0 != 0.0f) && (((l0 - 0x7F40u) & 0xFFFFu) <= 0x180u || !(d0 > 9.6e-7f && d0 < 1.0e6f))) e0 = powf(d0, c.norm);
        if ((d1 != 0.0f) && (((l1 - 0x7F40u) & 0xFFFFu) <= 0x180u || !(d1 > 9.6e-7f && d1 < 1.0e6f))) e1 = powf(d1, c.norm);
        const uint32_t eb = bf2_pack(e1, e0);
        err += __uint_as_float(eb << 16);
        err += __uint_as_float(eb & 0xFFFF0000u);
      }
      for (int o = lanes >> 1; o > 0; o >>= 1) err += __shfl_xor_sync(0xffffffffu, err, o);
      err = bf16r(err);
      if (live && err < best_err) {
        best_err = err; best_mn = smn; best_mx = smx;
        if (pass == 0 && (cc % lanes) == 0 && ((volatile int*)ctl)[1 + i] == 0) atomicOr(&ctl[1 + i], 1);
      }
    }
    if (live && (cc % lanes) == 0) {
      int64_t gi = row * gpr + (cc * 8) / g;
      ((T*)mn_out)[gi] = __float2bfloat16_rn(best_mn);
      ((T*)mx_out)[gi] = __float2bfloat16_rn(best_mx);
    }
  }
}
#undef B200Q_BF2

// One CTA per group held in shared memory: a row (CHANNEL, bh = 1, bw = K) or a bh x bw block
// (BLOCK; blocks that stick out of the matrix are completed with zeros, which take part in the
// statistics like the reference's padding).  The per-candidate error is summed in a fixed order
// (thread-strided partial sums, warp tree, warps in order), so results do not depend on timing.
template <int DT>
__global__ void __launch_bounds__(256) mse_tile_kernel(const void* __restrict__ W, int64_t N, int64_t K,
                                                       int64_t ldw, int bh, int bw, Cfg c, int* __restrict__ ctl,
                                                       int pass, void* __restrict__ mn_out, void* __restrict__ mx_out) {
  using E = Elem<DT>;
  using T = typename E::type;
  constexpr bool TB = E::is_bf16;
  extern __shared__ float srow[];
  __shared__ float s_a[8], s_b[8];
  __shared__ float s_bc[2];
  const int limit = (pass == 0) ? c.steps : ctl[0];
  if (pass == 1 && limit >= c.steps) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int64_t gpr = (K + bw - 1) / bw, groups = ((N + bh - 1) / bh) * gpr;
  const int elems = bh * bw;
  for (int64_t grp = blockIdx.x; grp < groups; grp += gridDim.x) {
    const int64_t r0 = (grp / gpr) * bh, c0 = (grp % gpr) * bw;
    float lo = INFINITY, hi = -INFINITY;
    for (int x = threadIdx.x; x < elems; x += blockDim.x) {
      const int64_t r = r0 + x / bw, cc = c0 + x % bw;
      const float v = (r < N && cc < K) ? E::load((const T*)W + r * ldw + cc) : 0.0f;
      srow[x] = v; lo = fminf(lo, v); hi = fmaxf(hi, v);
    }
    lo = warp_min(lo); hi = warp_max(hi);
    if (lane == 0) { s_a[warp] = lo; s_b[warp] = hi; }
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int w = 1; w < nw; ++w) { lo = fminf(lo, s_a[w]); hi = fmaxf(hi, s_b[w]); }
      s_bc[0] = lo; s_bc[1] = hi;
    }
    __syncthreads();
    const float mn = rnd_if<TB>(s_bc[0] * c.expand), mx = rnd_if<TB>(s_bc[1] * c.expand);
    float best_err = TB ? 3.3895313892515355e38f : 3.402823466e38f;
    float best_mn = mn, best_mx = mx;
    for (int i = 0; i < limit; ++i) {
      const float p = shrink_factor(i, c.grid);
      const float smn = rnd_if<TB>(mn * p), smx = rnd_if<TB>(mx * p);
      float s, z;
      qparams_local<TB>(smn, smx, c, s, z);
      float err = 0.0f;
      for (int x = threadIdx.x; x < elems; x += blockDim.x) err += elem_error<TB>(srow[x], s, z, c);
      err = warp_sum(err);
      __syncthreads();
      if (lane == 0) s_a[warp] = err;
      __syncthreads();
      float tot = 0.0f;
      for (int w = 0; w < nw; ++w) tot += s_a[w];
      tot = rnd_if<TB>(tot);
      if (tot < best_err) {
        best_err = tot; best_mn = smn; best_mx = smx;
        if (pass == 0 && threadIdx.x == 0 && ((volatile int*)ctl)[1 + i] == 0) atomicOr(&ctl[1 + i], 1);
      }
    }
    if (threadIdx.x == 0) {
      E::store((T*)mn_out + grp, best_mn);
      E::store((T*)mx_out + grp, best_mx);
    }
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------------------
// TENSOR strategy: the whole matrix is one group.  One launch per shrink candidate sums the
// element errors into per-CTA partials (grid-stride, fixed order inside a CTA); a one-warp kernel
// folds the partials in index order, compares with the best so far and keeps the reference's
// patience counter, all on the device.  After the search has stopped the remaining launches return
// at once.  state: [0] min, [1] max (expanded), [2] best error, [3] best min, [4] best max,
// [5] stale count, [6] stopped flag (both as int bit patterns), then the partials.
constexpr int kSpanState = 8;

template <int DT>
__global__ void __launch_bounds__(256) mse_span_range_kernel(const void* __restrict__ W, int64_t N, int64_t K,
                                                             int64_t ldw, float* __restrict__ partial) {
  using E = Elem<DT>;
  using T = typename E::type;
  __shared__ float s_a[8], s_b[8];
  float lo = INFINITY, hi = -INFINITY;
  const int64_t total = N * K;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / K, cc = i - r * K;
    const float v = E::load((const T*)W + r * ldw + cc);
    lo = fminf(lo, v); hi = fmaxf(hi, v);
  }
  lo = warp_min(lo); hi = warp_max(hi);
  if ((threadIdx.x & 31) == 0) { s_a[threadIdx.x >> 5] = lo; s_b[threadIdx.x >> 5] = hi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) { lo = fminf(lo, s_a[w]); hi = fmaxf(hi, s_b[w]); }
    partial[2 * blockIdx.x] = lo; partial[2 * blockIdx.x + 1] = hi;
  }
}
template <bool TB>
__global__ void mse_span_init_kernel(float* __restrict__ state, const float* __restrict__ partial, int nblocks, Cfg c) {
  float lo = INFINITY, hi = -INFINITY;
  for (int i = 0; i < nblocks; ++i) { lo = fminf(lo, partial[2 * i]); hi = fmaxf(hi, partial[2 * i + 1]); }
  const float mn = rnd_if<TB>(lo * c.expand), mx = rnd_if<TB>(hi * c.expand);
  state[0] = mn; state[1] = mx;
  state[2] = TB ? 3.3895313892515355e38f : 3.402823466e38f;
  state[3] = mn; state[4] = mx;
  ((int*)state)[5] = 0; ((int*)state)[6] = 0;
}
template <int DT>
__global__ void __launch_bounds__(256) mse_span_error_kernel(const void* __restrict__ W, int64_t N, int64_t K,
                                                             int64_t ldw, Cfg c, int step,
                                                             const float* __restrict__ state,
                                                             float* __restrict__ partial) {
  using E = Elem<DT>;
  using T = typename E::type;
  constexpr bool TB = E::is_bf16;
  __shared__ float s_a[8];
  if (((const int*)state)[6]) return;
  const float p = shrink_factor(step, c.grid);
  const float smn = rnd_if<TB>(state[0] * p), smx = rnd_if<TB>(state[1] * p);
  float s, z;
  qparams_local<TB>(smn, smx, c, s, z);
  float err = 0.0f;
  const int64_t total = N * K;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / K, cc = i - r * K;
    err += elem_error<TB>(E::load((const T*)W + r * ldw + cc), s, z, c);
  }
  err = warp_sum(err);
  if ((threadIdx.x & 31) == 0) s_a[threadIdx.x >> 5] = err;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.0f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += s_a[w];
    partial[blockIdx.x] = tot;
  }
}
template <bool TB>
__global__ void mse_span_fold_kernel(float* __restrict__ state, const float* __restrict__ partial, int nblocks, Cfg c,
                                     int step) {
  int* istate = (int*)state;
  if (istate[6]) return;
  float tot = 0.0f;
  for (int i = 0; i < nblocks; ++i) tot += partial[i];
  tot = rnd_if<TB>(tot);
  if (tot < state[2]) {
    const float p = shrink_factor(step, c.grid);
    state[2] = tot; state[3] = rnd_if<TB>(state[0] * p); state[4] = rnd_if<TB>(state[1] * p);
    istate[5] = 0;
  } else if (++istate[5] >= c.patience) {
    istate[6] = 1;
  }
}
template <int DT>
__global__ void mse_span_store_kernel(const float* __restrict__ state, void* __restrict__ mn_out,
                                      void* __restrict__ mx_out) {
  using E = Elem<DT>;
  using T = typename E::type;
  E::store((T*)mn_out, state[3]);
  E::store((T*)mx_out, state[4]);
}

// ctl[0] <- number of candidates the reference's loop evaluates before it breaks
__global__ void stop_step_kernel(int* ctl, int steps, int patience) {
  int stale = 0, run = steps;
  for (int i = 0; i < steps; ++i) {
    if (ctl[1 + i]) stale = 0;
    else if (++stale >= patience) { run = i + 1; break; }
  }
  ctl[0] = run;
}
__global__ void clear_ctl_kernel(int* ctl, int n) {
  for (int i = threadIdx.x; i < n; i += blockDim.x) ctl[i] = 0;
}

}  // namespace mse
}  // namespace b200q

using namespace b200q;

extern "C" {

// int(maxshrink * grid) in double precision, as the reference's Python evaluates it
int b200q_observe_mse_steps(double maxshrink, double grid) {
  const double v = maxshrink * grid;
  if (!(v >= 0.0)) return -1;
  return v > 2147483647.0 ? 2147483647 : (int)v;
}

size_t b200q_observe_mse_workspace_bytes(int64_t, int64_t, const b200q_qargs* qa, int steps) {
  const size_t flags = sizeof(int) * (size_t)(steps + 1 > 1 ? steps + 1 : 1);
  if (qa && qa->strategy == B200Q_TENSOR)   // search state and per-CTA partials
    return flags + sizeof(float) * (size_t)(b200q::mse::kSpanState + 2 * 4 * b200q::kNumSMs);
  return flags;
}

int b200q_observe_mse(const void* W, int wdtype, int64_t N, int64_t K, int64_t ldw, const b200q_qargs* qa,
                      double maxshrink, int patience, double grid, float norm, float expand, void* mn_out,
                      void* mx_out, void* scratch, void* stream) {
  using namespace b200q::mse;
  if (!W || !qa || !mn_out || !mx_out || !scratch || N <= 0 || K <= 0 || ldw < K) return B200Q_ERR_ARG;
  if (wdtype != B200Q_BF16 && wdtype != B200Q_F32) return B200Q_ERR_UNSUPPORTED;
  QRange qr;
  int rc = make_qrange(qa, &qr); if (rc) return rc;
  Cfg c;
  c.symmetric = qa->symmetric; c.scale_kind = qa->scale_kind; c.zp_kind = qa->zp_kind;
  c.mx_offset = (qa->num_bits == 4) ? 2 : 8;
  c.qmin = qr.qmin; c.qmax = qr.qmax; c.range = qr.qmax - qr.qmin; c.half_range = c.range / 2.0f; c.kind = qr.kind;
  if (!qa->symmetric && qr.kind == kFp4) return B200Q_ERR_UNSUPPORTED;
  if (qa->scale_kind == B200Q_SCALE_FP8) c.eps = 0.125f;
  else if (qa->scale_kind == B200Q_SCALE_E8M0) c.eps = 1.0f;
  else c.eps = (wdtype == B200Q_BF16) ? 0.0078125f : 1.1920928955078125e-07f;
  c.steps = b200q_observe_mse_steps(maxshrink, grid);
  c.patience = patience; c.grid = grid; c.norm = norm; c.expand = expand;
  if (wdtype == B200Q_BF16) {
    // torch casts the python exponent to the tensor's dtype: |e|.pow(2.4) on bf16 uses 2.40625
    uint32_t b;
    memcpy(&b, &norm, 4);
    b = (b + 0x7FFFu + ((b >> 16) & 1u)) & 0xFFFF0000u;
    memcpy(&c.norm, &b, 4);
  }
  if (c.steps < 0) return B200Q_ERR_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  int* ctl = (int*)scratch;
  clear_ctl_kernel<<<1, 128, 0, st>>>(ctl, c.steps + 1);
  B200Q_LAUNCH_CHECK();
  const bool grp = qa->strategy == B200Q_GROUP || qa->strategy == B200Q_TENSOR_GROUP;
  for (int pass = 0; pass < 2; ++pass) {
    if (grp) {
      int g = qa->group_size;
      if (!(g >= 8 && g <= 256 && (g & (g - 1)) == 0 && K % g == 0)) return B200Q_ERR_UNSUPPORTED;
      int grid_sz = grid_for((N * (K >> 3) + 255) / 256, 4);
      const bool fast = wdtype == B200Q_BF16 && qr.kind == kInt && qa->scale_kind != B200Q_SCALE_FP8 &&
                        qa->scale_kind != B200Q_SCALE_E8M0 && c.steps <= 1024 && (K & 7) == 0 && (ldw & 7) == 0 &&
                        (((uintptr_t)W) & 15) == 0;
      if (fast && qa->num_bits == 4) mse_group_bf16_int_kernel<true><<<grid_sz, 256, 0, st>>>(W, N, K, ldw, g, c, ctl, pass, mn_out, mx_out);
      else if (fast) mse_group_bf16_int_kernel<false><<<grid_sz, 256, 0, st>>>(W, N, K, ldw, g, c, ctl, pass, mn_out, mx_out);
      else if (wdtype == B200Q_BF16) mse_group_kernel<B200Q_BF16><<<grid_sz, 256, 0, st>>>(W, N, K, ldw, g, c, ctl, pass, mn_out, mx_out);
      else mse_group_kernel<B200Q_F32><<<grid_sz, 256, 0, st>>>(W, N, K, ldw, g, c, ctl, pass, mn_out, mx_out);
    } else if (qa->strategy == B200Q_CHANNEL || qa->strategy == B200Q_BLOCK) {
      const bool blk = qa->strategy == B200Q_BLOCK;
      if (blk && (qa->block_h <= 0 || qa->block_w <= 0)) return B200Q_ERR_ARG;
      const int64_t bh = blk ? qa->block_h : 1, bw = blk ? qa->block_w : K;
      const size_t smem = (size_t)(bh * bw) * sizeof(float);
      if (bh * bw > (int64_t)50 * 1024) return B200Q_ERR_UNSUPPORTED;   // group does not fit in shared memory
      const int64_t groups = ((N + bh - 1) / bh) * ((K + bw - 1) / bw);
      int grid_sz = grid_for(groups, smem > 100 * 1024 ? 1 : 2);
      if (wdtype == B200Q_BF16) {
        B200Q_TRY(cudaFuncSetAttribute(mse_tile_kernel<B200Q_BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        mse_tile_kernel<B200Q_BF16><<<grid_sz, 256, smem, st>>>(W, N, K, ldw, (int)bh, (int)bw, c, ctl, pass, mn_out, mx_out);
      } else {
        B200Q_TRY(cudaFuncSetAttribute(mse_tile_kernel<B200Q_F32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        mse_tile_kernel<B200Q_F32><<<grid_sz, 256, smem, st>>>(W, N, K, ldw, (int)bh, (int)bw, c, ctl, pass, mn_out, mx_out);
      }
    } else if (qa->strategy == B200Q_TENSOR) {
      // one group: the search runs candidate by candidate, with its state on the device
      if (pass == 1) break;
      float* state = (float*)(ctl + c.steps + 1);
      float* partial = state + kSpanState;
      const int nblk = grid_for((N * K + 255) / 256, 4);
      const bool tb = wdtype == B200Q_BF16;
      if (tb) mse_span_range_kernel<B200Q_BF16><<<nblk, 256, 0, st>>>(W, N, K, ldw, partial);
      else mse_span_range_kernel<B200Q_F32><<<nblk, 256, 0, st>>>(W, N, K, ldw, partial);
      B200Q_LAUNCH_CHECK();
      if (tb) mse_span_init_kernel<true><<<1, 1, 0, st>>>(state, partial, nblk, c);
      else mse_span_init_kernel<false><<<1, 1, 0, st>>>(state, partial, nblk, c);
      B200Q_LAUNCH_CHECK();
      for (int i = 0; i < c.steps; ++i) {
        if (tb) mse_span_error_kernel<B200Q_BF16><<<nblk, 256, 0, st>>>(W, N, K, ldw, c, i, state, partial);
        else mse_span_error_kernel<B200Q_F32><<<nblk, 256, 0, st>>>(W, N, K, ldw, c, i, state, partial);
        B200Q_LAUNCH_CHECK();
        if (tb) mse_span_fold_kernel<true><<<1, 1, 0, st>>>(state, partial, nblk, c, i);
        else mse_span_fold_kernel<false><<<1, 1, 0, st>>>(state, partial, nblk, c, i);
        B200Q_LAUNCH_CHECK();
      }
      if (tb) mse_span_store_kernel<B200Q_BF16><<<1, 1, 0, st>>>(state, mn_out, mx_out);
      else mse_span_store_kernel<B200Q_F32><<<1, 1, 0, st>>>(state, mn_out, mx_out);
      B200Q_LAUNCH_CHECK();
      return B200Q_OK;
    } else {
      return B200Q_ERR_UNSUPPORTED;
    }
    B200Q_LAUNCH_CHECK();
    if (pass == 0) {
      stop_step_kernel<<<1, 1, 0, st>>>(ctl, c.steps, c.patience);
      B200Q_LAUNCH_CHECK();
    }
  }
  return B200Q_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------
// Allocation-free variant of b200q_observe_mse.
//
// Some callers cannot obtain device memory at the moment they need an MSE observation: a
// serving process that has handed its whole memory budget to a KV-cache pool and re-calibrates
// a layer in place, code running inside a framework callback where the caching allocator must
// not be re-entered, or a C program that links this library without any allocator of its own.
// For them the search's scratch (one flag per shrink candidate plus the stop step) lives in a
// fixed array inside the library image instead of a caller-supplied buffer.
namespace b200q {
namespace mse {

constexpr int kStaticMaxSteps = 1023;  // candidates; the array holds kStaticMaxSteps + 1 ints (4 KiB)
static __device__ __align__(256) int g_static_ctl[kStaticMaxSteps + 1];

constexpr int kMaxDevices = 64;
static int* g_static_ctl_ptr[kMaxDevices] = {nullptr};
static std::mutex g_static_mutex;

// Device address of the array on the current device.  In host code the symbol's name is only a
// handle, not an address, so it is resolved once per device with cudaGetSymbolAddress.
static int static_ctl_address(int** out) {
  int dev = -1;
  B200Q_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return B200Q_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (g_static_ctl_ptr[dev] == nullptr) {
    void* p = nullptr;
    B200Q_TRY(cudaGetSymbolAddress(&p, g_static_ctl));
    if (p == nullptr) return B200Q_ERR_CUDA;
    g_static_ctl_ptr[dev] = static_cast<int*>(p);
  }
  *out = g_static_ctl_ptr[dev];
  return B200Q_OK;
}

}  // namespace mse
}  // namespace b200q

extern "C" int b200q_observe_mse_noalloc(const void* W, int wdtype, int64_t N, int64_t K, int64_t ldw,
                                         const b200q_qargs* qa, double maxshrink, int patience, double grid,
                                         float norm, float expand, void* mn_out, void* mx_out, void* stream) {
  using namespace b200q::mse;
  const int steps = b200q_observe_mse_steps(maxshrink, grid);
  if (steps < 0 || steps > kStaticMaxSteps) {
    b200q::set_last_error("b200q_observe_mse_noalloc: int(maxshrink*grid) exceeds the built-in scratch (1023 candidates)",
                          cudaErrorInvalidValue);
    return B200Q_ERR_ARG;
  }
  if (qa && qa->strategy == B200Q_TENSOR) {
    // the whole-tensor search keeps per-CTA partial sums in its scratch, more than the array holds
    b200q::set_last_error("b200q_observe_mse_noalloc: the TENSOR strategy needs more scratch than the built-in array",
                          cudaErrorInvalidValue);
    return B200Q_ERR_UNSUPPORTED;
  }
  int* ctl = nullptr;
  int rc = static_ctl_address(&ctl);
  if (rc != B200Q_OK) return rc;
  // the search clears the flags it uses before its first pass, so the contents left by the
  // previous call do not matter
  return b200q_observe_mse(W, wdtype, N, K, ldw, qa, maxshrink, patience, grid, norm, expand, mn_out, mx_out,
                           ctl, stream);
}
