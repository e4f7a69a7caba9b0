// HBM-bound kernels of the observer / qparams / quantize / pack path (sm_100a).
//
// All kernels stream the weight matrix once with 16-byte loads, keep the group
// statistics in registers (warp shuffles between the lanes that share a group) and
// write packed codes with 4..16-byte stores.  Grids are whole multiples of the SM count.
#include "common.cuh"

#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <mutex>
#include <string>

namespace b200q {

static thread_local std::string g_last_error;
static std::atomic<long long> g_launches{0};
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
void set_last_error(const char* what, cudaError_t e) {
  g_last_error = std::string(what) + ": " + cudaGetErrorString(e);
}

// ----------------------------------------------------------------------------------------
// qparams of one group, in the statistics' dtype (TB: bf16), following calculate_qparams.
struct QParamCfg {
  int symmetric, scale_kind, zp_kind, mx_offset, has_global;
  float qmin, qmax, half_range, range, eps;
  float inv_half_range, inv_range;   // float32 reciprocals, used for bf16 statistics (see qparams_one)
};

static int make_qparam_cfg(const b200q_qargs* qa, bool stat_bf16, bool has_global, QParamCfg* c) {
  QRange r;
  int st = make_qrange(qa, &r);
  if (st) return st;
  c->symmetric = qa->symmetric; c->scale_kind = qa->scale_kind; c->zp_kind = qa->zp_kind;
  c->has_global = has_global ? 1 : 0;
  c->qmin = r.qmin; c->qmax = r.qmax; c->range = r.qmax - r.qmin; c->half_range = c->range / 2.0f;
  c->inv_half_range = 1.0f / c->half_range; c->inv_range = 1.0f / c->range;
  c->mx_offset = (qa->num_bits == 4) ? 2 : 8;
  if (qa->scale_kind == B200Q_SCALE_E8M0 &&
      !(qa->qtype == B200Q_QFLOAT && qa->group_size == 32 && qa->symmetric))
    return B200Q_ERR_UNSUPPORTED;
  if (!qa->symmetric && r.kind == kFp4) return B200Q_ERR_UNSUPPORTED;
  if (qa->scale_kind == B200Q_SCALE_FP8) c->eps = 0.125f;
  else if (qa->scale_kind == B200Q_SCALE_E8M0) c->eps = 1.0f;
  else c->eps = (stat_bf16 && !has_global) ? 0.0078125f : 1.1920928955078125e-07f;
  return B200Q_OK;
}

template <bool TB>
__device__ __forceinline__ void qparams_one(float mn, float mx, const QParamCfg& c, float g,
                                            float& scale, float& zp) {
  mn = fminf(mn, 0.0f);
  mx = fmaxf(mx, 0.0f);
  float s;
  if (c.symmetric) {
    float amax = fmaxf(fabsf(mn), fabsf(mx));
    if (c.scale_kind == B200Q_SCALE_E8M0) {
      // keep sign+exponent after adding a quarter exponent step to the mantissa
      int biased;
      if (TB) {
        uint32_t b = __float_as_uint(amax) >> 16;
        b = (b + 32u) & 0xFF80u;
        biased = (int)((b >> 7) & 0xFFu);
      } else {
        uint32_t b = __float_as_uint(amax);
        b = (b + (1u << 21)) & 0xFF800000u;
        biased = (int)((b >> 23) & 0xFFu);
      }
      s = (biased == 0) ? -INFINITY : (float)(biased - c.mx_offset);
    } else {
      // bf16 statistics: the quotient of an 8-bit significand by 7.5, 127.5, 448 or 6 stays at least
      // 129 float32 ulps away from every bf16 rounding midpoint (checked over all significands), so
      // the product with the float32 reciprocal rounds to the same bf16 value as the division
      s = TB ? bf16r(amax * c.inv_half_range) : __fdiv_rn(amax, c.half_range);
    }
    zp = 0.0f;
  } else {
    float d = rnd_if<TB>(mx - mn);
    s = TB ? bf16r(d * c.inv_range) : __fdiv_rn(d, c.range);
    float z = rnd_if<TB>(__fdiv_rn(mn, s));
    z = rnd_if<TB>(c.qmin - z);
    // 0/0 for an all-zero group: torch's clamp keeps the NaN and the integer cast makes it 0
    zp = (z != z) ? 0.0f : fminf(fmaxf(z, c.qmin), c.qmax);
  }
  if (c.has_global) s = g * s;
  if (c.scale_kind == B200Q_SCALE_FP8) {
    s = e4m3_round(fminf(fmaxf(s, -448.0f), 448.0f));
  } else if (c.scale_kind == B200Q_SCALE_E8M0) {
    float e = rintf(fminf(fmaxf(s, 0.0f), 255.0f));
    s = __uint_as_float(e >= 1.0f ? ((uint32_t)e << 23) : 0x00400000u);  // 2^(e-127)
  }
  if (s == 0.0f) s = c.eps;
  if (!c.symmetric) {   // a symmetric zero point is exactly 0 in every storage type
    if (c.zp_kind == B200Q_ZP_INT8) zp = rintf(fminf(fmaxf(zp, -128.0f), 127.0f));
    else if (c.zp_kind == B200Q_ZP_UINT8) zp = rintf(fminf(fmaxf(zp, 0.0f), 255.0f));
    else zp = e4m3_round(fminf(fmaxf(zp, -448.0f), 448.0f));
  }
  scale = s;
}

__device__ __forceinline__ void store_zp(void* out, int zp_kind, int64_t i, float zp) {
  if (zp_kind == B200Q_ZP_INT8) ((int8_t*)out)[i] = (int8_t)zp;
  else if (zp_kind == B200Q_ZP_UINT8) ((uint8_t*)out)[i] = (uint8_t)zp;
  else ((uint8_t*)out)[i] = e4m3_bits(zp);
}

// 127 + floor(log2 s) of a positive power-of-two scale (also right for any positive float).
__device__ __forceinline__ uint8_t e8m0_of(float s) {
  uint32_t b = __float_as_uint(s);
  uint32_t e = (b >> 23) & 0xFFu;
  if (e == 0) {  // subnormal float: 2^-127 has mantissa 0x400000
    uint32_t m = b & 0x7FFFFFu;
    if (m == 0) return 0;
    int lz = __clz(m) - 9;  // leading zeros inside the 23-bit mantissa
    int v = 127 + (-127 - lz);
    return (uint8_t)(v < 0 ? 0 : v);
  }
  return (uint8_t)e;
}

// ----------------------------------------------------------------------------------------
// 8 consecutive elements of a row as floats
template <int DT>
__device__ __forceinline__ void load8(const void* base, int64_t off, float (&v)[8]) {
  if constexpr (DT == B200Q_BF16) {
    uint4 u = __ldg(reinterpret_cast<const uint4*>((const __nv_bfloat16*)base + off));
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
  } else {
    const float4* p = reinterpret_cast<const float4*>((const float*)base + off);
    float4 a = __ldg(p), b = __ldg(p + 1);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
}
template <int DT>
__device__ __forceinline__ void store8(void* base, int64_t off, const float (&v)[8]) {
  if constexpr (DT == B200Q_BF16) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>((__nv_bfloat16*)base + off) = make_uint4(w[0], w[1], w[2], w[3]);
  } else {
    float4* p = reinterpret_cast<float4*>((float*)base + off);
    p[0] = make_float4(v[0], v[1], v[2], v[3]);
    p[1] = make_float4(v[4], v[5], v[6], v[7]);
  }
}

}  // namespace b200q
#include "stream_kernels.cuh"
#include "stream_tma.cuh"
namespace b200q {

// ---- tensor map of a bf16 weight for the TMA-fed kernels: rows cut into 128-byte pieces -------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn tensor_map_encoder() {
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
// dims (64 elements, K/64 pieces, N rows), box (64, 32, 1) = one 4 KiB tile, 128-byte swizzle
static bool make_weight_tile_map(CUtensorMap* m, const void* W, int64_t N, int64_t K, int64_t ldw) {
  EncodeTiledFn enc = tensor_map_encoder();
  if (!enc) return false;
  cuuint64_t dims[3] = {64u, (cuuint64_t)(K / 64), (cuuint64_t)N};
  cuuint64_t strides[2] = {128u, (cuuint64_t)ldw * 2u};
  cuuint32_t box[3] = {64u, 32u, 1u};
  cuuint32_t estr[3] = {1, 1, 1};
  return enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(W), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
static bool tma_path_enabled() {
  static const bool on = [] { const char* e = getenv("B200Q_STREAM_TMA"); return !(e && e[0] == '0'); }();
  return on;
}

static bool vec_ok(const void* p, int64_t K, int64_t ld, int elem_bytes) {
  return (K % 8 == 0) && (ld % 8 == 0) && (((uintptr_t)p) % 16 == 0) && elem_bytes > 0;
}
static bool pow2(int v) { return v > 0 && (v & (v - 1)) == 0; }

// ========================================================================================
// observe_minmax (the streaming group kernels are in stream_kernels.cuh)
// ========================================================================================
// generic: one thread per qparam entry (group / block), any sizes
template <int DT>
__global__ void minmax_generic_kernel(const void* __restrict__ W, int64_t N, int64_t K, int64_t ldw,
                                      int strategy, int g, int bh, int bw,
                                      void* __restrict__ mn_out, void* __restrict__ mx_out) {
  using E = Elem<DT>;
  using T = typename E::type;
  int64_t gpr = (strategy == B200Q_BLOCK) ? (K + bw - 1) / bw : (K + g - 1) / g;
  int64_t rows = (strategy == B200Q_BLOCK) ? (N + bh - 1) / bh : N;
  int64_t total = rows * gpr;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    int64_t r = i / gpr, c = i - r * gpr;
    float lo = INFINITY, hi = -INFINITY;
    if (strategy == B200Q_BLOCK) {
      // zero padding of ragged blocks takes part in the statistics
      bool ragged = (r * bh + bh > N) || (c * bw + bw > K);
      if (ragged) { lo = 0.0f; hi = 0.0f; }
      for (int64_t y = r * bh; y < min((int64_t)(r * bh + bh), N); ++y)
        for (int64_t x = c * bw; x < min((int64_t)(c * bw + bw), K); ++x) {
          float v = E::load((const T*)W + y * ldw + x);
          lo = fminf(lo, v); hi = fmaxf(hi, v);
        }
    } else {
      for (int64_t x = c * g; x < min((int64_t)(c * g + g), K); ++x) {
        float v = E::load((const T*)W + r * ldw + x);
        lo = fminf(lo, v); hi = fmaxf(hi, v);
      }
    }
    E::store((T*)mn_out + i, lo);
    E::store((T*)mx_out + i, hi);
  }
}

// CHANNEL: one CTA per row
template <int DT>
__global__ void __launch_bounds__(256) minmax_channel_kernel(const void* __restrict__ W, int64_t N,
                                                             int64_t K, int64_t ldw, bool vec,
                                                             void* __restrict__ mn_out,
                                                             void* __restrict__ mx_out) {
  using E = Elem<DT>;
  using T = typename E::type;
  __shared__ float s_lo[8], s_hi[8];
  for (int64_t row = blockIdx.x; row < N; row += gridDim.x) {
    float lo = INFINITY, hi = -INFINITY;
    if (vec) {
      for (int64_t c = threadIdx.x; c < (K >> 3); c += blockDim.x) {
        float v[8];
        load8<DT>(W, row * ldw + c * 8, v);
#pragma unroll
        for (int i = 0; i < 8; ++i) { lo = fminf(lo, v[i]); hi = fmaxf(hi, v[i]); }
      }
    } else {
      for (int64_t x = threadIdx.x; x < K; x += blockDim.x) {
        float v = E::load((const T*)W + row * ldw + x);
        lo = fminf(lo, v); hi = fmaxf(hi, v);
      }
    }
    lo = warp_min(lo); hi = warp_max(hi);
    if ((threadIdx.x & 31) == 0) { s_lo[threadIdx.x >> 5] = lo; s_hi[threadIdx.x >> 5] = hi; }
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int w = 1; w < (blockDim.x >> 5); ++w) { lo = fminf(lo, s_lo[w]); hi = fmaxf(hi, s_hi[w]); }
      E::store((T*)mn_out + row, lo);
      E::store((T*)mx_out + row, hi);
    }
    __syncthreads();
  }
}

// TENSOR: per-CTA partials, then one CTA folds them
template <int DT>
__global__ void __launch_bounds__(256) minmax_tensor_partial_kernel(const void* __restrict__ W,
                                                                    int64_t N, int64_t K,
                                                                    int64_t ldw, bool vec,
                                                                    float* __restrict__ partial) {
  using E = Elem<DT>;
  using T = typename E::type;
  __shared__ float s_lo[8], s_hi[8];
  float lo = INFINITY, hi = -INFINITY;
  if (vec) {
    int64_t cpr = K >> 3, total = N * cpr;
    for (int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; c < total;
         c += (int64_t)gridDim.x * blockDim.x) {
      int64_t row = c / cpr, cc = c - row * cpr;
      float v[8];
      load8<DT>(W, row * ldw + cc * 8, v);
#pragma unroll
      for (int i = 0; i < 8; ++i) { lo = fminf(lo, v[i]); hi = fmaxf(hi, v[i]); }
    }
  } else {
    int64_t total = N * K;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
      int64_t row = i / K, x = i - row * K;
      float v = E::load((const T*)W + row * ldw + x);
      lo = fminf(lo, v); hi = fmaxf(hi, v);
    }
  }
  lo = warp_min(lo); hi = warp_max(hi);
  if ((threadIdx.x & 31) == 0) { s_lo[threadIdx.x >> 5] = lo; s_hi[threadIdx.x >> 5] = hi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (blockDim.x >> 5); ++w) { lo = fminf(lo, s_lo[w]); hi = fmaxf(hi, s_hi[w]); }
    partial[2 * blockIdx.x] = lo;
    partial[2 * blockIdx.x + 1] = hi;
  }
}
template <int DT>
__global__ void minmax_tensor_final_kernel(const float* __restrict__ partial, int n,
                                           void* __restrict__ mn_out, void* __restrict__ mx_out) {
  using E = Elem<DT>;
  using T = typename E::type;
  float lo = INFINITY, hi = -INFINITY;
  for (int i = threadIdx.x; i < n; i += 32) { lo = fminf(lo, partial[2 * i]); hi = fmaxf(hi, partial[2 * i + 1]); }
  lo = warp_min(lo); hi = warp_max(hi);
  if (threadIdx.x == 0) { E::store((T*)mn_out, lo); E::store((T*)mx_out, hi); }
}

constexpr int kTensorPartialBlocks = kNumSMs * 4;

template <int DT>
static int observe_minmax_impl(const void* W, int64_t N, int64_t K, int64_t ldw,
                               const b200q_qargs* qa, void* mn, void* mx, void* scratch,
                               cudaStream_t st) {
  const bool vec = vec_ok(W, K, ldw, 2);
  switch (qa->strategy) {
    case B200Q_GROUP:
    case B200Q_TENSOR_GROUP: {
      int g = qa->group_size;
      if (g <= 0) return B200Q_ERR_ARG;
      if (vec && pow2(g) && g >= 8 && g <= 256 && K % g == 0) {
        if constexpr (DT == B200Q_BF16) {
          const stream::GroupSplit gsp = stream::make_group_split(g);
          const int64_t slots = (K / g) * gsp.L;
          int tx2 = 32;
          while (tx2 < 256 && tx2 < slots) tx2 <<= 1;
          const int rows2 = stream::kThreads / tx2;
          const int grid2 = grid_for((N + rows2 - 1) / rows2, 8);
          const int txl2 = __builtin_ctz(tx2), ll2 = __builtin_ctz(gsp.L);
          if (gsp.R == 8) stream::minmax_group_bf16_kernel<8><<<grid2, stream::kThreads, 0, st>>>(W, (int)N, (int)K, ldw, g, ll2, txl2, mn, mx);
          else if (gsp.R == 4) stream::minmax_group_bf16_kernel<4><<<grid2, stream::kThreads, 0, st>>>(W, (int)N, (int)K, ldw, g, ll2, txl2, mn, mx);
          else if (gsp.R == 2) stream::minmax_group_bf16_kernel<2><<<grid2, stream::kThreads, 0, st>>>(W, (int)N, (int)K, ldw, g, ll2, txl2, mn, mx);
          else stream::minmax_group_bf16_kernel<1><<<grid2, stream::kThreads, 0, st>>>(W, (int)N, (int)K, ldw, g, ll2, txl2, mn, mx);
        } else {
          stream::RowTiling t = stream::make_tiling(N, K, 8);
          stream::minmax_group_kernel<DT><<<t.grid, stream::kThreads, 0, st>>>(W, (int)N, (int)K, ldw, g, __builtin_ctz(t.tx), mn, mx);
        }
      } else {
        int64_t total = N * ((K + g - 1) / g);
        minmax_generic_kernel<DT><<<grid_for((total + 127) / 128, 8), 128, 0, st>>>(
            W, N, K, ldw, qa->strategy, g, 1, 1, mn, mx);
      }
      break;
    }
    case B200Q_BLOCK: {
      if (qa->block_h <= 0 || qa->block_w <= 0) return B200Q_ERR_ARG;
      int64_t total = ((N + qa->block_h - 1) / qa->block_h) * ((K + qa->block_w - 1) / qa->block_w);
      minmax_generic_kernel<DT><<<grid_for((total + 127) / 128, 8), 128, 0, st>>>(
          W, N, K, ldw, qa->strategy, 1, qa->block_h, qa->block_w, mn, mx);
      break;
    }
    case B200Q_CHANNEL:
      minmax_channel_kernel<DT><<<grid_for(N, 8), 256, 0, st>>>(W, N, K, ldw, vec, mn, mx);
      break;
    case B200Q_TENSOR: {
      if (!scratch) return B200Q_ERR_ARG;
      int blocks = grid_for((N * K / 8 + 255) / 256, 4);
      minmax_tensor_partial_kernel<DT><<<blocks, 256, 0, st>>>(W, N, K, ldw, vec, (float*)scratch);
      minmax_tensor_final_kernel<DT><<<1, 32, 0, st>>>((const float*)scratch, blocks, mn, mx);
      break;
    }
    default: return B200Q_ERR_ARG;
  }
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

// ========================================================================================
// global scale
// ========================================================================================
template <int DT>
__global__ void absmax_kernel(const void* __restrict__ mn, const void* __restrict__ mx, int64_t n,
                              float* __restrict__ absmax) {
  using E = Elem<DT>;
  using T = typename E::type;
  float a = 0.0f;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    a = fmaxf(a, fmaxf(fabsf(E::load((const T*)mn + i)), fabsf(E::load((const T*)mx + i))));
  }
  a = warp_max(a);
  // non-negative floats order like their bit patterns
  if ((threadIdx.x & 31) == 0) atomicMax(reinterpret_cast<int*>(absmax), __float_as_int(a));
}
// largest magnitude of a whole bf16 matrix, folded into *absmax: 16-byte loads, four in flight,
// sign bits cleared and a packed unsigned 16-bit maximum (bf16 magnitudes order like integers)
__global__ void __launch_bounds__(256) absmax_weight_bf16_kernel(const void* __restrict__ W, int64_t N, int64_t K,
                                                                 int64_t ldw, float* __restrict__ absmax) {
  const int64_t cpr = K >> 3, total = N * cpr;
  const int64_t step = (int64_t)gridDim.x * blockDim.x;
  uint32_t m = 0;
  int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  auto chunk = [&](int64_t i) {
    const int64_t row = i / cpr, cc = i - row * cpr;
    return stream::ldg_stream((const __nv_bfloat16*)W + row * ldw + cc * 8);
  };
  for (; c + 3 * step < total; c += 4 * step) {
    const uint4 a = chunk(c), b = chunk(c + step), d = chunk(c + 2 * step), e = chunk(c + 3 * step);
    const uint4 v[4] = {a, b, d, e};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      m = __vimax3_u16x2(m, v[k].x & 0x7FFF7FFFu, v[k].y & 0x7FFF7FFFu);
      m = __vimax3_u16x2(m, v[k].z & 0x7FFF7FFFu, v[k].w & 0x7FFF7FFFu);
    }
  }
  for (; c < total; c += step) {
    const uint4 a = chunk(c);
    m = __vimax3_u16x2(m, a.x & 0x7FFF7FFFu, a.y & 0x7FFF7FFFu);
    m = __vimax3_u16x2(m, a.z & 0x7FFF7FFFu, a.w & 0x7FFF7FFFu);
  }
  uint32_t h = max(m & 0xFFFFu, m >> 16);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) h = max(h, __shfl_xor_sync(0xffffffffu, h, o));
  __shared__ uint32_t s_m[8];
  if ((threadIdx.x & 31) == 0) s_m[threadIdx.x >> 5] = h;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) h = max(h, s_m[w]);
    // non-negative floats order like their bit patterns
    atomicMax(reinterpret_cast<int*>(absmax), (int)(h << 16));
  }
}

__global__ void global_scale_kernel(const float* __restrict__ absmax, int stat_bf16,
                                    float* __restrict__ out) {
  float a = *absmax;
  float tiny = 1.17549435e-38f;  // smallest normal of both bf16 and float32
  a = fmaxf(a, tiny);
  // "scalar / tensor" in torch is tensor.reciprocal() * scalar: two roundings in the statistics' dtype
  float r = __frcp_rn(a);
  if (stat_bf16) r = bf16r(r);
  float g = __fmul_rn(r, 448.0f * 6.0f);
  if (stat_bf16) g = bf16r(g);
  if (!(fabsf(g) <= 3.402823466e38f)) g = 1.0f;  // NaN / Inf -> 1
  *out = g;
}

// ========================================================================================
// qparams
// ========================================================================================
template <int DT, bool GLOBAL>
__global__ void qparams_kernel(const void* __restrict__ mn, const void* __restrict__ mx, int64_t n,
                               QParamCfg c, const float* __restrict__ gscale,
                               void* __restrict__ scale_out, void* __restrict__ zp_out) {
  using E = Elem<DT>;
  using T = typename E::type;
  float g = GLOBAL ? *gscale : 1.0f;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    float s, z;
    qparams_one<E::is_bf16>(E::load((const T*)mn + i), E::load((const T*)mx + i), c, g, s, z);
    if (GLOBAL) ((float*)scale_out)[i] = s;
    else E::store((T*)scale_out + i, s);
    if (zp_out) store_zp(zp_out, c.zp_kind, i, z);
  }
}

// ========================================================================================
// fake_quantize / quantize_pack with given parameters
// ========================================================================================
enum PackMode { kPackFake = 0, kPackInt4 = 1, kPackByte = 2, kPackFp4 = 3, kPackInt8Word = 4 };

template <int SDT>
__device__ __forceinline__ float load_scale(const void* scale, int64_t i) {
  return Elem<SDT>::load((const typename Elem<SDT>::type*)scale + i);
}

// Scalar path for ragged shapes: one thread per output unit (word / byte / element).
template <int XDT, int SDT, bool GLOBAL, int MODE>
__global__ void quant_scalar_kernel(const void* __restrict__ W, int64_t N, int64_t K, int64_t ldw,
                                    const void* __restrict__ scale, const void* __restrict__ zp,
                                    int zp_kind, ParamMap pm, const float* __restrict__ gscale,
                                    QRange qr, void* __restrict__ out, int64_t ldo) {
  using EX = Elem<XDT>;
  constexpr bool XB = EX::is_bf16;
  constexpr bool SB = Elem<SDT>::is_bf16 && !GLOBAL;
  constexpr bool CB = XB && SB;
  constexpr int per = (MODE == kPackInt4) ? 8 : (MODE == kPackInt8Word) ? 4 : (MODE == kPackFp4) ? 2 : 1;
  const float g = GLOBAL ? *gscale : 1.0f;
  const int64_t upr = (K + per - 1) / per, total = N * upr;
  for (int64_t u = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; u < total;
       u += (int64_t)gridDim.x * blockDim.x) {
    int64_t row = u / upr, uc = u - row * upr;
    uint32_t word = 0;
    for (int i = 0; i < per; ++i) {
      int64_t col = uc * per + i;
      if (col >= K) break;  // zero padding of the last word
      int64_t pi = pm.index(row, col);
      float s = load_scale<SDT>(scale, pi);
      if (GLOBAL) s = __fdiv_rn(s, g);
      float z = zp ? load_zp(zp, zp_kind, pi) : 0.0f;
      float x = EX::load((const typename EX::type*)W + row * ldw + col);
      float q = quant_code<CB>(x, s, z, qr);
      if constexpr (MODE == kPackFake) {
        EX::store((typename EX::type*)out + row * ldo + col, dequant_code<SB>(q, s, z));
      } else if constexpr (MODE == kPackInt4) {
        word |= ((uint32_t)((int)q + 8) & 0xFu) << (4 * i);
      } else if constexpr (MODE == kPackInt8Word) {
        word |= ((uint32_t)((int)q + 128) & 0xFFu) << (8 * i);
      } else if constexpr (MODE == kPackFp4) {
        word |= e2m1_nibble(q) << (4 * i);
      } else {
        word = (qr.kind == kFp8) ? e4m3_bits(q) : ((uint32_t)(int)q & 0xFFu);
      }
    }
    if constexpr (MODE == kPackInt4 || MODE == kPackInt8Word) ((uint32_t*)out)[u] = word;
    else if constexpr (MODE == kPackFp4 || MODE == kPackByte) ((uint8_t*)out)[u] = (uint8_t)word;
  }
}

template <int XDT, int SDT, bool GLOBAL, int MODE>
static int quant_launch(const void* W, int64_t N, int64_t K, int64_t ldw, const void* scale,
                        const void* zp, int zp_kind, const ParamMap& pm, const float* gscale,
                        const QRange& qr, void* out, int64_t ldo, cudaStream_t st) {
  bool vec = vec_ok(W, K, ldw, 2) && (((uintptr_t)out) % 16 == 0) &&
             (MODE != kPackFake || ldo % 8 == 0);
  if (vec && N < (1LL << 31) && K < (1LL << 31)) {
    const bool uniform = (pm.strategy == B200Q_TENSOR) || (pm.strategy == B200Q_CHANNEL) ||
                         ((pm.strategy == B200Q_GROUP || pm.strategy == B200Q_TENSOR_GROUP) &&
                          pm.g_idx == nullptr && (pm.group_size & 7) == 0) ||
                         (pm.strategy == B200Q_BLOCK && (pm.block_w & 7) == 0);
    // bf16 weights with per-group parameters in column order: lane / chunk split kernels.  The
    // combinations that occur: a bf16 scale without a global scale, or a float32 scale with one
    // (FP4 only); everything else takes the row kernel below.
    if constexpr (XDT == B200Q_BF16 && MODE != kPackFake &&
                  ((SDT == B200Q_BF16 && !GLOBAL) || (SDT == B200Q_F32 && GLOBAL && MODE == kPackFp4))) {
      const int g = pm.group_size;
      if ((pm.strategy == B200Q_GROUP || pm.strategy == B200Q_TENSOR_GROUP) && pm.g_idx == nullptr && g >= 8 &&
          g <= 256 && (g & (g - 1)) == 0 && K % g == 0) {
        const stream::GroupSplit gsp = stream::make_group_split(g, 4);
        const int64_t slots = (K / g) * gsp.L;
        int tx2 = 32;
        while (tx2 < 256 && tx2 < slots) tx2 <<= 1;
        const int rows2 = stream::kThreads / tx2;
        const int grid2 = grid_for((N + rows2 - 1) / rows2, 6);
        const int txl2 = __builtin_ctz(tx2);
#define B200Q_QG(RR, LL) stream::quant_group_bf16_kernel<SDT, GLOBAL, MODE, RR, LL><<<grid2, stream::kThreads, 0, st>>>(W, (int)N, (int)K, ldw, txl2, scale, zp, zp_kind, gscale, qr, out)
        switch (g) {
          case 8: B200Q_QG(1, 1); break;
          case 16: B200Q_QG(2, 1); break;
          case 32: B200Q_QG(4, 1); break;
          case 64: B200Q_QG(4, 2); break;
          case 128: B200Q_QG(4, 4); break;
          default: B200Q_QG(4, 8); break;
        }
#undef B200Q_QG
        B200Q_LAUNCH_CHECK();
        return B200Q_OK;
      }
    }
    stream::RowTiling t = stream::make_tiling(N, K, 6);
    stream::quant_rows_kernel<XDT, SDT, GLOBAL, MODE><<<t.grid, stream::kThreads, 0, st>>>(
        W, (int)N, (int)K, ldw, __builtin_ctz(t.tx), scale, zp, zp_kind, pm, uniform, gscale, qr, out, ldo);
  } else {
    int64_t blocks = (N * K + 255) / 256;
    quant_scalar_kernel<XDT, SDT, GLOBAL, MODE><<<grid_for(blocks, 8), 256, 0, st>>>(
        W, N, K, ldw, scale, zp, zp_kind, pm, gscale, qr, out, ldo);
  }
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

template <int MODE>
static int quant_dispatch(const void* W, int wdtype, int64_t N, int64_t K, int64_t ldw,
                          const void* scale, int sdtype, const void* zp, const int32_t* g_idx,
                          const float* gscale, const b200q_qargs* qa, void* out, int64_t ldo,
                          cudaStream_t st) {
  if (!W || !scale || !out || !qa || N <= 0 || K <= 0) return B200Q_ERR_ARG;
  QRange qr; ParamMap pm;
  int rc = make_qrange(qa, &qr); if (rc) return rc;
  rc = make_param_map(qa, N, K, g_idx, &pm); if (rc) return rc;
  int zk = qa->zp_kind;
#define B200Q_Q(X, S, G) return quant_launch<X, S, G, MODE>(W, N, K, ldw, scale, zp, zk, pm, gscale, qr, out, ldo, st)
  if (wdtype == B200Q_BF16 && sdtype == B200Q_BF16) { if (gscale) B200Q_Q(B200Q_BF16, B200Q_BF16, true); else B200Q_Q(B200Q_BF16, B200Q_BF16, false); }
  if (wdtype == B200Q_BF16 && sdtype == B200Q_F32)  { if (gscale) B200Q_Q(B200Q_BF16, B200Q_F32, true);  else B200Q_Q(B200Q_BF16, B200Q_F32, false); }
  if (wdtype == B200Q_F32 && sdtype == B200Q_BF16)  { if (gscale) B200Q_Q(B200Q_F32, B200Q_BF16, true);  else B200Q_Q(B200Q_F32, B200Q_BF16, false); }
  if (wdtype == B200Q_F32 && sdtype == B200Q_F32)   { if (gscale) B200Q_Q(B200Q_F32, B200Q_F32, true);   else B200Q_Q(B200Q_F32, B200Q_F32, false); }
#undef B200Q_Q
  return B200Q_ERR_UNSUPPORTED;
}

// ========================================================================================
// zero-point packing along dim 0 and scale compression
// ========================================================================================
__global__ void pack_zp_kernel(const int8_t* __restrict__ zp, int64_t N, int64_t G, int bits,
                               int32_t* __restrict__ out) {
  const int pf = 32 / bits;
  const int64_t rows_out = (N + pf - 1) / pf, total = rows_out * G;
  const int off = 1 << (bits - 1);
  const uint32_t mask = (bits == 32) ? 0xFFFFFFFFu : ((1u << bits) - 1u);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    int64_t ro = i / G, c = i - ro * G;
    uint32_t w = 0;
    for (int j = 0; j < pf; ++j) {
      int64_t r = ro * pf + j;
      if (r >= N) break;
      w |= (((uint32_t)((int)zp[r * G + c] + off)) & mask) << (bits * j);
    }
    out[i] = (int32_t)w;
  }
}

template <int DT>
__global__ void compress_scale_kernel(const void* __restrict__ scale, int64_t n, int kind,
                                      uint8_t* __restrict__ out) {
  using E = Elem<DT>;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    float s = E::load((const typename E::type*)scale + i);
    out[i] = (kind == B200Q_SCALE_FP8) ? e4m3_bits(s) : e8m0_of(s);
  }
}

// ========================================================================================
// fused round-to-nearest: statistics -> qparams -> codes -> packed, one read of W
// ========================================================================================
// GROUP strategies (g power of two, 8..256): thread = 8 elements, lanes of a group shuffle.
template <int DT, int MODE, bool GLOBAL>
__global__ void __launch_bounds__(256) rtn_group_kernel(
    const void* __restrict__ W, int64_t N, int64_t K, int64_t ldw, int g, QParamCfg qc, QRange qr,
    const float* __restrict__ gscale, void* __restrict__ scale_out, void* __restrict__ zp_out,
    uint8_t* __restrict__ scale_store, void* __restrict__ out) {
  using E = Elem<DT>;
  using T = typename E::type;
  constexpr bool XB = E::is_bf16;
  constexpr bool SB = XB && !GLOBAL;  // scale dtype: stats dtype unless a global scale promotes it
  constexpr bool CB = XB && SB;
  const float gs = GLOBAL ? *gscale : 1.0f;
  const int lanes = g >> 3;
  const int64_t cpr = K >> 3, total = N * cpr, gpr = K / g;
  for (int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; c < ((total + 31) & ~31LL);
       c += (int64_t)gridDim.x * blockDim.x) {
    const bool live = c < total;
    float v[8];
    float lo = INFINITY, hi = -INFINITY;
    int64_t row = 0, cc = 0;
    if (live) {
      row = c / cpr; cc = c - row * cpr;
      load8<DT>(W, row * ldw + cc * 8, v);
#pragma unroll
      for (int i = 0; i < 8; ++i) { lo = fminf(lo, v[i]); hi = fmaxf(hi, v[i]); }
    }
    for (int o = lanes >> 1; o > 0; o >>= 1) {
      lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
      hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
    }
    if (!live) continue;
    float s, z;
    qparams_one<XB>(lo, hi, qc, gs, s, z);
    if ((cc % lanes) == 0) {
      int64_t gi = row * gpr + (cc * 8) / g;
      // the module keeps the scale in the weight dtype (exact: FP8-grid and power-of-two
      // scales are bf16 values; plain scales already are bf16 when the statistics are)
      E::store((T*)scale_out + gi, s);
      if (zp_out) store_zp(zp_out, qc.zp_kind, gi, z);
      if (scale_store) scale_store[gi] = (qc.scale_kind == B200Q_SCALE_FP8) ? e4m3_bits(s) : e8m0_of(s);
    }
    float se = GLOBAL ? __fdiv_rn(s, gs) : s;
    uint32_t w0 = 0, w1 = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float q = quant_code<CB>(v[i], se, z, qr);
      if (MODE == kPackInt4) w0 |= ((uint32_t)((int)q + 8) & 0xFu) << (4 * i);
      else if (MODE == kPackFp4) w0 |= e2m1_nibble(q) << (4 * i);
      else {
        uint32_t b = (qr.kind == kFp8) ? e4m3_bits(q)
                   : (MODE == kPackInt8Word) ? ((uint32_t)((int)q + 128) & 0xFFu)
                                             : ((uint32_t)(int)q & 0xFFu);
        if (i < 4) w0 |= b << (8 * i); else w1 |= b << (8 * (i - 4));
      }
    }
    if (MODE == kPackInt4 || MODE == kPackFp4) ((uint32_t*)out)[row * cpr + cc] = w0;
    else reinterpret_cast<uint2*>(out)[row * cpr + cc] = make_uint2(w0, w1);
  }
}

// CHANNEL strategy: one CTA per row, the row staged in shared memory between the two passes.
template <int DT, int MODE>
__global__ void __launch_bounds__(256) rtn_channel_kernel(
    const void* __restrict__ W, int64_t N, int64_t K, int64_t ldw, QParamCfg qc, QRange qr,
    void* __restrict__ scale_out, void* __restrict__ zp_out, void* __restrict__ out) {
  using E = Elem<DT>;
  using T = typename E::type;
  constexpr bool XB = E::is_bf16;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* srow = reinterpret_cast<T*>(smem_raw);
  __shared__ float s_lo[8], s_hi[8], s_par[2];
  const int64_t cpr = K >> 3;
  for (int64_t row = blockIdx.x; row < N; row += gridDim.x) {
    float lo = INFINITY, hi = -INFINITY;
    for (int64_t c = threadIdx.x; c < cpr; c += blockDim.x) {
      float v[8];
      load8<DT>(W, row * ldw + c * 8, v);
      store8<DT>(srow, c * 8, v);
#pragma unroll
      for (int i = 0; i < 8; ++i) { lo = fminf(lo, v[i]); hi = fmaxf(hi, v[i]); }
    }
    lo = warp_min(lo); hi = warp_max(hi);
    if ((threadIdx.x & 31) == 0) { s_lo[threadIdx.x >> 5] = lo; s_hi[threadIdx.x >> 5] = hi; }
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int w = 1; w < (blockDim.x >> 5); ++w) { lo = fminf(lo, s_lo[w]); hi = fmaxf(hi, s_hi[w]); }
      float s, z;
      qparams_one<XB>(lo, hi, qc, 1.0f, s, z);
      s_par[0] = s; s_par[1] = z;
      E::store((T*)scale_out + row, s);
      if (zp_out) store_zp(zp_out, qc.zp_kind, row, z);
    }
    __syncthreads();
    const float s = s_par[0], z = s_par[1];
    for (int64_t c = threadIdx.x; c < cpr; c += blockDim.x) {
      float v[8];
      if constexpr (XB) {
        uint4 u = *reinterpret_cast<const uint4*>(srow + c * 8);
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) { v[2 * i] = __uint_as_float(w[i] << 16); v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u); }
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = ((const float*)srow)[c * 8 + i];
      }
      uint32_t w0 = 0, w1 = 0;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float q = quant_code<XB>(v[i], s, z, qr);
        if (MODE == kPackInt4) w0 |= ((uint32_t)((int)q + 8) & 0xFu) << (4 * i);
        else {
          uint32_t b = (qr.kind == kFp8) ? e4m3_bits(q)
                     : (MODE == kPackInt8Word) ? ((uint32_t)((int)q + 128) & 0xFFu)
                                               : ((uint32_t)(int)q & 0xFFu);
          if (i < 4) w0 |= b << (8 * i); else w1 |= b << (8 * (i - 4));
        }
      }
      if (MODE == kPackInt4) ((uint32_t*)out)[row * cpr + c] = w0;
      else reinterpret_cast<uint2*>(out)[row * cpr + c] = make_uint2(w0, w1);
    }
    __syncthreads();
  }
}

}  // namespace b200q

using namespace b200q;

// ========================================================================================
// C ABI
// ========================================================================================
extern "C" {

const char* b200q_version(void) { return "b200q 0.1 (sm_100a)"; }
const char* b200q_last_error(void) { return g_last_error.c_str(); }
long long b200q_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int b200q_take_wait_status(void) {
  int v = 0;
  B200Q_TRY(cudaMemcpyFromSymbol(&v, tma::g_wait_expired, sizeof(int)));
  if (v == 0) return B200Q_OK;
  v = 0;
  B200Q_TRY(cudaMemcpyToSymbol(tma::g_wait_expired, &v, sizeof(int)));
  return B200Q_ERR_DEVICE;
}

size_t b200q_observe_minmax_workspace_bytes(int64_t, int64_t, const b200q_qargs* qa) {
  return (qa && qa->strategy == B200Q_TENSOR) ? sizeof(float) * 2 * kTensorPartialBlocks : 0;
}

int b200q_observe_minmax(const void* W, int wdtype, int64_t N, int64_t K, int64_t ldw,
                         const b200q_qargs* qa, void* mn, void* mx, void* scratch, void* stream) {
  if (!W || !qa || !mn || !mx || N <= 0 || K <= 0 || ldw < K) return B200Q_ERR_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  if (wdtype == B200Q_BF16) return observe_minmax_impl<B200Q_BF16>(W, N, K, ldw, qa, mn, mx, scratch, st);
  if (wdtype == B200Q_F32) return observe_minmax_impl<B200Q_F32>(W, N, K, ldw, qa, mn, mx, scratch, st);
  return B200Q_ERR_UNSUPPORTED;
}

int b200q_absmax_accumulate(const void* mn, const void* mx, int dtype, int64_t count, float* absmax,
                            void* stream) {
  if (!mn || !mx || !absmax || count <= 0) return B200Q_ERR_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  int grid = grid_for((count + 255) / 256, 2);
  if (dtype == B200Q_BF16) absmax_kernel<B200Q_BF16><<<grid, 256, 0, st>>>(mn, mx, count, absmax);
  else if (dtype == B200Q_F32) absmax_kernel<B200Q_F32><<<grid, 256, 0, st>>>(mn, mx, count, absmax);
  else return B200Q_ERR_UNSUPPORTED;
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_absmax_accumulate_weight(const void* W, int wdtype, int64_t N, int64_t K, int64_t ldw, float* absmax,
                                   void* stream) {
  if (!W || !absmax || N <= 0 || K <= 0 || ldw < K) return B200Q_ERR_ARG;
  if (wdtype != B200Q_BF16 || !vec_ok(W, K, ldw, 2)) return B200Q_ERR_UNSUPPORTED;
  const int grid = grid_for((N * (K >> 3) + 1023) / 1024, 8);
  absmax_weight_bf16_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(W, N, K, ldw, absmax);
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_global_scale_finalize(const float* absmax, int stat_dtype, float* global_scale, void* stream) {
  if (!absmax || !global_scale) return B200Q_ERR_ARG;
  global_scale_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(absmax, stat_dtype == B200Q_BF16, global_scale);
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_qparams(const void* mn, const void* mx, int stat_dtype, int64_t count, const b200q_qargs* qa,
                  const float* gscale, void* scale_out, void* zp_out, void* stream) {
  if (!mn || !mx || !qa || !scale_out || count <= 0) return B200Q_ERR_ARG;
  QParamCfg c;
  int rc = make_qparam_cfg(qa, stat_dtype == B200Q_BF16, gscale != nullptr, &c);
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  int grid = grid_for((count + 255) / 256, 4);
  if (stat_dtype == B200Q_BF16) {
    if (gscale) qparams_kernel<B200Q_BF16, true><<<grid, 256, 0, st>>>(mn, mx, count, c, gscale, scale_out, zp_out);
    else qparams_kernel<B200Q_BF16, false><<<grid, 256, 0, st>>>(mn, mx, count, c, gscale, scale_out, zp_out);
  } else if (stat_dtype == B200Q_F32) {
    if (gscale) qparams_kernel<B200Q_F32, true><<<grid, 256, 0, st>>>(mn, mx, count, c, gscale, scale_out, zp_out);
    else qparams_kernel<B200Q_F32, false><<<grid, 256, 0, st>>>(mn, mx, count, c, gscale, scale_out, zp_out);
  } else return B200Q_ERR_UNSUPPORTED;
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_fake_quantize(const void* W, int wdtype, int64_t N, int64_t K, int64_t ldw, const void* scale,
                        int sdtype, const void* zp, const int32_t* g_idx, const float* gscale,
                        const b200q_qargs* qa, void* out, int64_t ldo, void* stream) {
  if (ldw < K || ldo < K) return B200Q_ERR_ARG;
  return quant_dispatch<kPackFake>(W, wdtype, N, K, ldw, scale, sdtype, zp, g_idx, gscale, qa, out, ldo,
                                   (cudaStream_t)stream);
}

int b200q_quantize_pack(const void* W, int wdtype, int64_t N, int64_t K, int64_t ldw, const void* scale,
                        int sdtype, const void* zp, const int32_t* g_idx, const float* gscale,
                        const b200q_qargs* qa, int pack_int8, void* out, void* stream) {
  if (!qa || ldw < K) return B200Q_ERR_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  if (qa->qtype == B200Q_QINT && qa->num_bits == 4)
    return quant_dispatch<kPackInt4>(W, wdtype, N, K, ldw, scale, sdtype, zp, g_idx, gscale, qa, out, 0, st);
  if (qa->qtype == B200Q_QINT && qa->num_bits == 8) {
    if (pack_int8)
      return quant_dispatch<kPackInt8Word>(W, wdtype, N, K, ldw, scale, sdtype, zp, g_idx, gscale, qa, out, 0, st);
    return quant_dispatch<kPackByte>(W, wdtype, N, K, ldw, scale, sdtype, zp, g_idx, gscale, qa, out, 0, st);
  }
  if (qa->qtype == B200Q_QFLOAT && qa->num_bits == 8)
    return quant_dispatch<kPackByte>(W, wdtype, N, K, ldw, scale, sdtype, zp, g_idx, gscale, qa, out, 0, st);
  if (qa->qtype == B200Q_QFLOAT && qa->num_bits == 4) {
    if (K % 2) return B200Q_ERR_ARG;
    return quant_dispatch<kPackFp4>(W, wdtype, N, K, ldw, scale, sdtype, zp, g_idx, gscale, qa, out, 0, st);
  }
  return B200Q_ERR_UNSUPPORTED;
}

int b200q_pack_zero_points(const int8_t* zp, int64_t N, int64_t G, int num_bits, int32_t* out, void* stream) {
  if (!zp || !out || N <= 0 || G <= 0 || num_bits < 1 || num_bits > 8) return B200Q_ERR_ARG;
  int64_t total = ((N + 32 / num_bits - 1) / (32 / num_bits)) * G;
  pack_zp_kernel<<<grid_for((total + 255) / 256, 4), 256, 0, (cudaStream_t)stream>>>(zp, N, G, num_bits, out);
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_compress_scale(const void* scale, int sdtype, int64_t count, int scale_kind, uint8_t* out, void* stream) {
  if (!scale || !out || count <= 0) return B200Q_ERR_ARG;
  if (scale_kind != B200Q_SCALE_FP8 && scale_kind != B200Q_SCALE_E8M0) return B200Q_ERR_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  int grid = grid_for((count + 255) / 256, 4);
  if (sdtype == B200Q_BF16) compress_scale_kernel<B200Q_BF16><<<grid, 256, 0, st>>>(scale, count, scale_kind, out);
  else if (sdtype == B200Q_F32) compress_scale_kernel<B200Q_F32><<<grid, 256, 0, st>>>(scale, count, scale_kind, out);
  else return B200Q_ERR_UNSUPPORTED;
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

}  // extern "C"

template <int DT>
static int rtn_impl(const void* W, int64_t N, int64_t K, int64_t ldw, const b200q_qargs* qa,
                    const float* gscale, void* scale_out, void* zp_out, uint8_t* scale_store, void* out,
                    cudaStream_t st) {
  QParamCfg qc; QRange qr;
  int rc = make_qparam_cfg(qa, DT == B200Q_BF16, gscale != nullptr, &qc); if (rc) return rc;
  rc = make_qrange(qa, &qr); if (rc) return rc;
  if (!vec_ok(W, K, ldw, 2) || (((uintptr_t)out) % 16)) return B200Q_ERR_UNSUPPORTED;
  if (!qa->symmetric && !zp_out) return B200Q_ERR_ARG;
  const bool grp = qa->strategy == B200Q_GROUP || qa->strategy == B200Q_TENSOR_GROUP;
  if (grp) {
    int g = qa->group_size;
    if (!(pow2(g) && g >= 8 && g <= 256 && K % g == 0)) return B200Q_ERR_UNSUPPORTED;
    stream::RowTiling t = stream::make_tiling(N, K, 6);
    const int txl = __builtin_ctz(t.tx);
    // bf16 weights whose rows are whole 2048-element tiles: the TMA-fed kernel
    if constexpr (DT == B200Q_BF16) {
      const bool aligned = (((uintptr_t)scale_out) % 16 == 0) && (!zp_out || ((uintptr_t)zp_out) % 4 == 0) &&
                           (!scale_store || ((uintptr_t)scale_store) % 4 == 0) && (((uintptr_t)out) % 16 == 0);
      if (tma_path_enabled() && aligned && K % tma::kTileElems == 0 && (g == 16 || g == 32 || g == 128) &&
          N < (1 << 30) && (!gscale || (g == 16 && qr.kind == kFp4))) {
        CUtensorMap wm;
        if (make_weight_tile_map(&wm, W, N, K, ldw)) {
          const int64_t tiles = N * (K / tma::kTileElems);
          const int gridt = (int)std::min<int64_t>((tiles + tma::kWarps - 1) / tma::kWarps, 2 * kNumSMs);
          // test hook: B200Q_TEST_DROP_TILE=n makes one warp skip its n-th tile request (see the kernel)
          const char* drop_env = getenv("B200Q_TEST_DROP_TILE");
          const int drop_request = drop_env ? atoi(drop_env) : -1;
#define B200Q_T3(MODE, GL, GG)                                                                                   \
  do {                                                                                                           \
    B200Q_TRY(cudaFuncSetAttribute(tma::rtn_group_tma_kernel<stream::MODE, GL, GG>,                              \
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, tma::kSmemBytes));               \
    tma::rtn_group_tma_kernel<stream::MODE, GL, GG><<<gridt, tma::kWarps * 32, tma::kSmemBytes, st>>>(           \
        wm, (int)N, (int)K, qc, qr, gscale, scale_out, zp_out, scale_store, out, drop_request);                  \
  } while (0)
#define B200Q_T2(MODE)                                     \
  do {                                                     \
    if (g == 16) B200Q_T3(MODE, false, 16);                \
    else if (g == 32) B200Q_T3(MODE, false, 32);           \
    else B200Q_T3(MODE, false, 128);                       \
  } while (0)
          if (gscale) B200Q_T3(kFp4, true, 16);
          else if (qr.kind == kInt && qa->num_bits == 4) B200Q_T2(kInt4);
          else if (qr.kind == kInt && qa->num_bits == 8) B200Q_T2(kInt8Word);
          else if (qr.kind == kFp8) B200Q_T2(kByte);
          else if (qr.kind == kFp4) B200Q_T2(kFp4);
          else return B200Q_ERR_UNSUPPORTED;
#undef B200Q_T2
#undef B200Q_T3
          B200Q_LAUNCH_CHECK();
          return B200Q_OK;
        }
      }
    }
    // bf16 weights: R chunks per lane, L lanes per group (both compile-time)
    const stream::GroupSplit gsp = stream::make_group_split(g, 4);
    const int64_t slots = (K / g) * gsp.L;
    int tx2 = 32;
    while (tx2 < 256 && tx2 < slots) tx2 <<= 1;
    const int rows2 = stream::kThreads / tx2;
    const int grid2 = grid_for((N + rows2 - 1) / rows2, 6);
    const int txl2 = __builtin_ctz(tx2);
#define B200Q_RB3(MODE, GL, RR, LL) stream::rtn_group_bf16_kernel<stream::MODE, GL, RR, LL><<<grid2, stream::kThreads, 0, st>>>(W, (int)N, (int)K, ldw, txl2, qc, qr, gscale, scale_out, zp_out, scale_store, out)
#define B200Q_RB2(MODE, GL)                          \
  do {                                               \
    switch (g) {                                     \
      case 8: B200Q_RB3(MODE, GL, 1, 1); break;      \
      case 16: B200Q_RB3(MODE, GL, 2, 1); break;     \
      case 32: B200Q_RB3(MODE, GL, 4, 1); break;     \
      case 64: B200Q_RB3(MODE, GL, 4, 2); break;     \
      case 128: B200Q_RB3(MODE, GL, 4, 4); break;    \
      default: B200Q_RB3(MODE, GL, 4, 8); break;     \
    }                                                \
  } while (0)
#define B200Q_RB(MODE)                                                            \
  do {                                                                            \
    if (gscale) {                                                                 \
      if constexpr (stream::MODE == stream::kFp4) {                               \
        if (g != 16) return B200Q_ERR_UNSUPPORTED;                                \
        B200Q_RB3(MODE, true, 2, 1);                                              \
      } else {                                                                    \
        return B200Q_ERR_UNSUPPORTED;                                             \
      }                                                                           \
    } else {                                                                      \
      B200Q_RB2(MODE, false);                                                     \
    }                                                                             \
  } while (0)
#define B200Q_R(MODE)                                                                              \
  do {                                                                                             \
    if constexpr (DT == B200Q_BF16) {                                                              \
      B200Q_RB(MODE);                                                                               \
    } else if (gscale) stream::rtn_group_kernel<DT, stream::MODE, true><<<t.grid, stream::kThreads, 0, st>>>(W, (int)N, (int)K, ldw, g, txl, qc, qr, gscale, scale_out, zp_out, scale_store, out); \
    else stream::rtn_group_kernel<DT, stream::MODE, false><<<t.grid, stream::kThreads, 0, st>>>(W, (int)N, (int)K, ldw, g, txl, qc, qr, gscale, scale_out, zp_out, scale_store, out);      \
  } while (0)
    if (qr.kind == kInt && qa->num_bits == 4) B200Q_R(kInt4);
    else if (qr.kind == kInt && qa->num_bits == 8) B200Q_R(kInt8Word);
    else if (qr.kind == kFp8) B200Q_R(kByte);
    else if (qr.kind == kFp4) B200Q_R(kFp4);
    else return B200Q_ERR_UNSUPPORTED;
#undef B200Q_R
#undef B200Q_RB
#undef B200Q_RB2
#undef B200Q_RB3
  } else if (qa->strategy == B200Q_CHANNEL) {
    if (gscale) return B200Q_ERR_UNSUPPORTED;
    if constexpr (DT == B200Q_BF16) {
      const int64_t cpr = K >> 3;
      if ((K & 7) == 0 && cpr <= 16 * stream::kThreads && N < (1 << 30)) {
        const int r = cpr <= 2 * stream::kThreads ? 2 : cpr <= 4 * stream::kThreads ? 4
                    : cpr <= 8 * stream::kThreads ? 8 : 16;
        const int gridc = grid_for(N, r <= 4 ? 4 : 2);
#define B200Q_CB2(MODE, RR) stream::rtn_channel_bf16_kernel<stream::MODE, RR><<<gridc, stream::kThreads, 0, st>>>(W, (int)N, (int)K, ldw, qc, qr, scale_out, zp_out, out)
#define B200Q_CB(MODE)                       \
  do {                                       \
    if (r == 2) B200Q_CB2(MODE, 2);          \
    else if (r == 4) B200Q_CB2(MODE, 4);     \
    else if (r == 8) B200Q_CB2(MODE, 8);     \
    else B200Q_CB2(MODE, 16);                \
  } while (0)
        if (qr.kind == kInt && qa->num_bits == 4) B200Q_CB(kInt4);
        else if (qr.kind == kInt && qa->num_bits == 8) B200Q_CB(kInt8Word);
        else if (qr.kind == kFp8) B200Q_CB(kByte);
        else return B200Q_ERR_UNSUPPORTED;
#undef B200Q_CB
#undef B200Q_CB2
        B200Q_LAUNCH_CHECK();
        return B200Q_OK;
      }
    }
    size_t smem = (size_t)K * (DT == B200Q_BF16 ? 2 : 4);
    if (smem > 200 * 1024) return B200Q_ERR_UNSUPPORTED;
    int grid = grid_for(N, smem > 100 * 1024 ? 1 : 2);
#define B200Q_C(MODE)                                                                               \
  do {                                                                                              \
    B200Q_TRY(cudaFuncSetAttribute(rtn_channel_kernel<DT, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    rtn_channel_kernel<DT, MODE><<<grid, 256, smem, st>>>(W, N, K, ldw, qc, qr, scale_out, zp_out, out); \
  } while (0)
    if (qr.kind == kInt && qa->num_bits == 4) B200Q_C(kPackInt4);
    else if (qr.kind == kInt && qa->num_bits == 8) B200Q_C(kPackInt8Word);
    else if (qr.kind == kFp8) B200Q_C(kPackByte);
    else return B200Q_ERR_UNSUPPORTED;
#undef B200Q_C
  } else {
    return B200Q_ERR_UNSUPPORTED;
  }
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

extern "C" {

int b200q_rtn_quantize_pack(const void* W, int wdtype, int64_t N, int64_t K, int64_t ldw,
                            const b200q_qargs* qa, void* scale_out, void* zp_out, uint8_t* scale_store,
                            void* out, void* stream) {
  if (!W || !qa || !scale_out || !out || N <= 0 || K <= 0 || ldw < K) return B200Q_ERR_ARG;
  if (qa->strategy == B200Q_TENSOR_GROUP) return B200Q_ERR_UNSUPPORTED;  // needs the global scale
  cudaStream_t st = (cudaStream_t)stream;
  if (wdtype == B200Q_BF16) return rtn_impl<B200Q_BF16>(W, N, K, ldw, qa, nullptr, scale_out, zp_out, scale_store, out, st);
  if (wdtype == B200Q_F32) return rtn_impl<B200Q_F32>(W, N, K, ldw, qa, nullptr, scale_out, zp_out, scale_store, out, st);
  return B200Q_ERR_UNSUPPORTED;
}

int b200q_nvfp4_quantize_pack(const void* W, int wdtype, int64_t N, int64_t K, int64_t ldw,
                              const float* global_scale, void* scale_out, uint8_t* scale_store, void* out,
                              void* stream) {
  if (!W || !global_scale || !scale_out || !out || N <= 0 || K <= 0 || ldw < K) return B200Q_ERR_ARG;
  b200q_qargs qa = {4, B200Q_QFLOAT, 1, B200Q_TENSOR_GROUP, 16, 0, 0, B200Q_SCALE_FP8, B200Q_ZP_FP8};
  cudaStream_t st = (cudaStream_t)stream;
  if (wdtype == B200Q_BF16) return rtn_impl<B200Q_BF16>(W, N, K, ldw, &qa, global_scale, scale_out, nullptr, scale_store, out, st);
  if (wdtype == B200Q_F32) return rtn_impl<B200Q_F32>(W, N, K, ldw, &qa, global_scale, scale_out, nullptr, scale_store, out, st);
  return B200Q_ERR_UNSUPPORTED;
}

}  // extern "C"
