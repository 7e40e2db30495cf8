// Dynamic activation quantisation (per token / per 1xG group, e4m3 or int8) and
// the row gather into the expert-sorted layout.  Both are HBM-bound: 128-bit
// loads/stores, one pass over the data.
#include "common.cuh"

namespace bolt {
namespace {

template <int QT>
struct QTraits;
template <>
struct QTraits<BOLT_FP8_E4M3> {
  using type = uint8_t;
  static constexpr float kMax = 448.0f;
  __device__ static __forceinline__ uint8_t cvt(float v) { return f32_to_e4m3(v); }
};
template <>
struct QTraits<BOLT_INT8> {
  using type = int8_t;
  static constexpr float kMax = 127.0f;
  __device__ static __forceinline__ int8_t cvt(float v) { return f32_to_i8(v); }
};

// scale and its reciprocal from the group absmax.
template <int QT, bool POW2>
__device__ __forceinline__ void scale_from_amax(float amax, float& scale, float& inv) {
  if (POW2) {
    const float raw = fmaxf(amax, 1.0e-10f) * (float)(1.0 / 448.0);
    const float lg = ceilf((float)log2((double)raw));
    scale = ldexpf(1.0f, (int)lg);
    inv = ldexpf(1.0f, -(int)lg);
  } else {
    scale = __fdiv_rn(fmaxf(amax, 1.0e-10f), QTraits<QT>::kMax);
    inv = __frcp_rn(scale);
  }
}

template <int QT, bool POW2>
__device__ __forceinline__ typename QTraits<QT>::type quant_one(float x, float inv) {
  float y = x * inv;
  if (POW2) y = fminf(fmaxf(y, -448.0f), 448.0f);
  return QTraits<QT>::cvt(y);
}

// ---- small groups: TPG threads (a power of two <= 32) share one group ----------
// A thread owns W input vectors = EPT consecutive elements (EPT = 16: 16-byte stores).
// Where the scale of group `grp` (= row * groups_per_row + g) goes: row-major [rows, groups]
// (ld == 0) or group-major [groups, ld] (the layout the grouped GEMM reads per K block).
struct ScaleOut {
  float* p;
  int groups_per_row;
  int64_t ld;
  __device__ __forceinline__ void put(int64_t grp, float v) const {
    if (ld == 0) p[grp] = v;
    else p[(grp % groups_per_row) * ld + grp / groups_per_row] = v;
  }
};

template <typename TIn, int QT, bool POW2, int W>
__global__ void __launch_bounds__(256) k_quant_group(const TIn* __restrict__ x,
                                                     typename QTraits<QT>::type* __restrict__ q,
                                                     const ScaleOut scales,
                                                     int64_t num_groups, int tpg) {
  constexpr int VEC = 16 / sizeof(TIn);
  constexpr int EPT = VEC * W;
  using VIn = Vec<TIn, VEC>;
  using VOut = Vec<typename QTraits<QT>::type, EPT>;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t grp = tid / tpg;
  const bool live = grp < num_groups;
  VIn v[W];
  float amax = 0.f;
  if (live) {
#pragma unroll
    for (int w = 0; w < W; ++w) {
      v[w] = reinterpret_cast<const VIn*>(x)[tid * W + w];
#pragma unroll
      for (int i = 0; i < VEC; ++i) amax = fmaxf(amax, fabsf(to_f32(v[w].v[i])));
    }
  }
  for (int o = tpg >> 1; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if (!live) return;
  float scale, inv;
  scale_from_amax<QT, POW2>(amax, scale, inv);
  VOut o;
#pragma unroll
  for (int w = 0; w < W; ++w)
#pragma unroll
    for (int i = 0; i < VEC; ++i) o.v[w * VEC + i] = quant_one<QT, POW2>(to_f32(v[w].v[i]), inv);
  reinterpret_cast<VOut*>(q)[tid] = o;
  if ((tid % tpg) == 0) scales.put(grp, scale);
}

// ---- one CTA per group (large or oddly sized groups) ---------------------------
template <typename TIn, int QT, bool POW2>
__global__ void __launch_bounds__(256) k_quant_row(const TIn* __restrict__ x,
                                                   typename QTraits<QT>::type* __restrict__ q,
                                                   const ScaleOut scales, int group) {
  const int64_t g = blockIdx.x;
  const TIn* xr = x + g * (int64_t)group;
  typename QTraits<QT>::type* qr = q + g * (int64_t)group;
  float amax = 0.f;
  for (int i = threadIdx.x; i < group; i += blockDim.x) amax = fmaxf(amax, fabsf(to_f32(xr[i])));
  __shared__ float red[8];
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) amax = fmaxf(amax, red[w]);
  float scale, inv;
  scale_from_amax<QT, POW2>(amax, scale, inv);
  for (int i = threadIdx.x; i < group; i += blockDim.x)
    qr[i] = quant_one<QT, POW2>(to_f32(xr[i]), inv);
  if (threadIdx.x == 0) scales.put(g, scale);
}

// vectorised variant of the above: group % VEC == 0 and 16-byte aligned rows.
template <typename TIn, int QT, bool POW2, int NV>
__global__ void __launch_bounds__(256) k_quant_row_vec(const TIn* __restrict__ x,
                                                       typename QTraits<QT>::type* __restrict__ q,
                                                       const ScaleOut scales, int group) {
  constexpr int VEC = 16 / sizeof(TIn);
  using VIn = Vec<TIn, VEC>;
  using VOut = Vec<typename QTraits<QT>::type, VEC>;
  const int64_t g = blockIdx.x;
  const VIn* xr = reinterpret_cast<const VIn*>(x + g * (int64_t)group);
  VOut* qr = reinterpret_cast<VOut*>(q + g * (int64_t)group);
  const int nvec = group / VEC;
  VIn cache[NV];
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int i = threadIdx.x + j * 256;
    if (i < nvec) {
      cache[j] = xr[i];
#pragma unroll
      for (int e = 0; e < VEC; ++e) amax = fmaxf(amax, fabsf(to_f32(cache[j].v[e])));
    }
  }
  for (int i = threadIdx.x + NV * 256; i < nvec; i += 256) {
    VIn v = xr[i];
#pragma unroll
    for (int e = 0; e < VEC; ++e) amax = fmaxf(amax, fabsf(to_f32(v.v[e])));
  }
  __shared__ float red[8];
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) amax = fmaxf(amax, red[w]);
  float scale, inv;
  scale_from_amax<QT, POW2>(amax, scale, inv);
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int i = threadIdx.x + j * 256;
    if (i < nvec) {
      VOut o;
#pragma unroll
      for (int e = 0; e < VEC; ++e) o.v[e] = quant_one<QT, POW2>(to_f32(cache[j].v[e]), inv);
      qr[i] = o;
    }
  }
  for (int i = threadIdx.x + NV * 256; i < nvec; i += 256) {
    VIn v = xr[i];
    VOut o;
#pragma unroll
    for (int e = 0; e < VEC; ++e) o.v[e] = quant_one<QT, POW2>(to_f32(v.v[e]), inv);
    qr[i] = o;
  }
  if (threadIdx.x == 0) scales.put(g, scale);
}

// ---- one warp per group (mid-sized rows: the row lives in the warp's registers) -----
// A lane owns units of W input vectors = EPT consecutive elements; with EPT = 16 every store is
// 16 bytes wide.
template <typename TIn, int QT, bool POW2, int NV, int W>
__global__ void __launch_bounds__(256) k_quant_row_warp(const TIn* __restrict__ x,
                                                        typename QTraits<QT>::type* __restrict__ q,
                                                        const ScaleOut scales,
                                                        int64_t num_groups, int group) {
  constexpr int VEC = 16 / sizeof(TIn);
  constexpr int EPT = VEC * W;
  using VIn = Vec<TIn, VEC>;
  using VOut = Vec<typename QTraits<QT>::type, EPT>;
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int nunits = group / EPT;
  for (int64_t g = warp0; g < num_groups; g += nwarps) {
    const VIn* xr = reinterpret_cast<const VIn*>(x + g * (int64_t)group);
    VOut* qr = reinterpret_cast<VOut*>(q + g * (int64_t)group);
    VIn cache[NV][W];
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int i = lane + j * 32;
      if (i < nunits) {
#pragma unroll
        for (int w = 0; w < W; ++w) {
          cache[j][w] = xr[i * W + w];
#pragma unroll
          for (int e = 0; e < VEC; ++e) amax = fmaxf(amax, fabsf(to_f32(cache[j][w].v[e])));
        }
      }
    }
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    float scale, inv;
    scale_from_amax<QT, POW2>(amax, scale, inv);
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int i = lane + j * 32;
      if (i < nunits) {
        VOut o;
#pragma unroll
        for (int w = 0; w < W; ++w)
#pragma unroll
          for (int e = 0; e < VEC; ++e)
            o.v[w * VEC + e] = quant_one<QT, POW2>(to_f32(cache[j][w].v[e]), inv);
        qr[i] = o;
      }
    }
    if (lane == 0) scales.put(g, scale);
  }
}

template <typename TIn, int QT, bool POW2>
int launch_quant(const void* x, int64_t rows, int cols, int group, void* q, ScaleOut scales,
                 cudaStream_t st) {
  using QTy = typename QTraits<QT>::type;
  constexpr int VEC = 16 / sizeof(TIn);
  const int64_t num_groups = rows * (int64_t)(cols / group);
  if (num_groups == 0) return BOLT_OK;
  BOLT_REQUIRE(num_groups < (1ll << 31), "quant: too many groups");
  const bool aligned = (reinterpret_cast<uintptr_t>(x) % 16 == 0) &&
                       (reinterpret_cast<uintptr_t>(q) % (VEC * sizeof(QTy)) == 0) &&
                       (group % VEC == 0);
  const int tpg = aligned ? group / VEC : 0;
  const int tpg16 = group / 16;
  if (aligned && group % 16 == 0 && reinterpret_cast<uintptr_t>(q) % 16 == 0 && tpg16 <= 32 &&
      (tpg16 & (tpg16 - 1)) == 0) {
    // 16 elements per thread: 16-byte stores
    const int64_t threads = num_groups * tpg16;
    const int64_t blocks = (threads + 255) / 256;
    k_quant_group<TIn, QT, POW2, 16 / VEC><<<(unsigned)blocks, 256, 0, st>>>(
        static_cast<const TIn*>(x), static_cast<QTy*>(q), scales, num_groups, tpg16);
  } else if (aligned && tpg <= 32 && (tpg & (tpg - 1)) == 0) {
    const int64_t threads = num_groups * tpg;
    const int64_t blocks = (threads + 255) / 256;
    k_quant_group<TIn, QT, POW2, 1><<<(unsigned)blocks, 256, 0, st>>>(
        static_cast<const TIn*>(x), static_cast<QTy*>(q), scales, num_groups, tpg);
  } else if (aligned && group / VEC <= 8 * 32) {
    // up to 8 vectors per lane: one warp per row, rows strided over a capped grid
    int64_t blocks = (num_groups + 7) / 8;
    const int64_t cap = (int64_t)sm_count_of_current_device() * 32;
    if (blocks > cap) blocks = cap;
    // (16-element units per lane were measured slower here: 0.153 vs 0.122 ms at 147456 x 768)
    k_quant_row_warp<TIn, QT, POW2, 8, 1><<<(unsigned)blocks, 256, 0, st>>>(
        static_cast<const TIn*>(x), static_cast<QTy*>(q), scales, num_groups, group);
  } else if (aligned) {
    k_quant_row_vec<TIn, QT, POW2, 4><<<(unsigned)num_groups, 256, 0, st>>>(
        static_cast<const TIn*>(x), static_cast<QTy*>(q), scales, group);
  } else {
    k_quant_row<TIn, QT, POW2><<<(unsigned)num_groups, 256, 0, st>>>(
        static_cast<const TIn*>(x), static_cast<QTy*>(q), scales, group);
  }
  BOLT_LAUNCH_CHECK();
  return BOLT_OK;
}

template <typename TIn>
int dispatch_quant(const void* x, int64_t rows, int cols, int group, int q_dtype, int power2,
                   void* q, ScaleOut scales, cudaStream_t st) {
  if (q_dtype == BOLT_FP8_E4M3) {
    return power2 ? launch_quant<TIn, BOLT_FP8_E4M3, true>(x, rows, cols, group, q, scales, st)
                  : launch_quant<TIn, BOLT_FP8_E4M3, false>(x, rows, cols, group, q, scales, st);
  }
  return launch_quant<TIn, BOLT_INT8, false>(x, rows, cols, group, q, scales, st);
}

// ---- gather into expert-sorted rows ----------------------------------------------
__global__ void __launch_bounds__(256) k_gather_rows(const uint4* __restrict__ src,
                                                     int num_tokens, int row_vecs,
                                                     int64_t src_stride_vecs,
                                                     const float* __restrict__ src_scale,
                                                     int64_t scale_stride, int groups,
                                                     const int32_t* __restrict__ sorted_ids,
                                                     const int32_t* __restrict__ num_valid,
                                                     int capacity, uint4* __restrict__ dst,
                                                     float* __restrict__ dst_scale,
                                                     int64_t dst_scale_ld) {
  const int valid = min(*num_valid, capacity);
  for (int row = blockIdx.x; row < valid; row += gridDim.x) {
    const int token = sorted_ids[row] & 0xFFFFFF;
    uint4* d = dst + (int64_t)row * row_vecs;
    if (token >= num_tokens) {
      // pad row inside a tile: its results are never consumed, but the GEMM streams it through
      // the tensor cores, and zeros cost less power there than stale memory does
      for (int i = threadIdx.x; i < row_vecs; i += blockDim.x) d[i] = make_uint4(0u, 0u, 0u, 0u);
      if (src_scale != nullptr) {
        if (groups == 1) {
          if (threadIdx.x == 0) dst_scale[row] = 0.f;
        } else {
          for (int g = threadIdx.x; g < groups; g += blockDim.x)
            dst_scale[(int64_t)g * dst_scale_ld + row] = 0.f;
        }
      }
      continue;
    }
    const uint4* s = src + (int64_t)token * src_stride_vecs;
    for (int i = threadIdx.x; i < row_vecs; i += blockDim.x) d[i] = __ldg(s + i);
    if (src_scale != nullptr) {
      if (groups == 1) {
        if (threadIdx.x == 0) dst_scale[row] = src_scale[(int64_t)token * scale_stride];
      } else {
        for (int g = threadIdx.x; g < groups; g += blockDim.x)
          dst_scale[(int64_t)g * dst_scale_ld + row] = src_scale[(int64_t)token * scale_stride + g];
      }
    }
  }
}

// Zero-fill the rows below num_valid that hold no token (tile padding).  Warp-granular: every
// lane tests one row of a 32-row window, the warp then clears the rows that were flagged, so no
// thread walks the id list serially.  `pad_warp` / `pad_warps` = this warp's index / count among
// the warps doing this job.
template <typename QTy, int VEC>
__device__ __forceinline__ void zero_pad_rows(const int32_t* __restrict__ sorted_ids,
                                              int64_t num_tokens, int valid, int row_vecs,
                                              int groups, QTy* __restrict__ dst,
                                              float* __restrict__ dst_scale, int64_t dst_scale_ld,
                                              int pad_warp, int pad_warps, bool token_order) {
  using VOut = Vec<QTy, VEC>;
  const int lane = threadIdx.x & 31;
  VOut zero;
#pragma unroll
  for (int i = 0; i < VEC; ++i) zero.v[i] = 0;
  // token_order: the codes live in token order and the GEMM fills padding positions with zeros
  // itself; only the padding positions' scales are written here
  for (int row0 = pad_warp * 32; row0 < valid; row0 += pad_warps * 32) {
    const int row = row0 + lane;
    const bool is_pad = row < valid && (sorted_ids[row] & 0xFFFFFF) >= num_tokens;
    unsigned mask = __ballot_sync(0xffffffffu, is_pad);
    while (mask) {
      const int r = row0 + __ffs(mask) - 1;
      mask &= mask - 1;
      if (!token_order) {
        VOut* d = reinterpret_cast<VOut*>(dst) + (int64_t)r * row_vecs;
        for (int i = lane; i < row_vecs; i += 32) d[i] = zero;
      }
      for (int g = lane; g < groups; g += 32) dst_scale[(int64_t)g * dst_scale_ld + r] = 0.f;
    }
  }
}

// ---- quantise a token once, write it to every sorted row that holds one of its routes -----
// Same arithmetic as k_quant_group (TPG threads share a 1 x group block of one token row); the
// 8-bit codes and the scale then go straight to rows route_pos[token][k] >= 0 of the
// expert-sorted layout (scales group-major, [groups, dst_scale_ld]), so the quantised
// activations never exist in token order.  The tail of the kernel zero-fills the rows below
// num_valid that hold no token (tile padding).
template <typename TIn, int QT, bool POW2, int W>
__global__ void __launch_bounds__(256) k_quant_scatter(
    const TIn* __restrict__ x, int64_t num_tokens, int cols, int tpg,
    const int32_t* __restrict__ route_pos, int slots, const int32_t* __restrict__ sorted_ids,
    const int32_t* __restrict__ num_valid, int capacity,
    typename QTraits<QT>::type* __restrict__ dst, float* __restrict__ dst_scale,
    int64_t dst_scale_ld, int64_t quant_blocks, int token_order) {
  // a thread owns W input vectors = EPT consecutive elements (EPT = 16: one 16-byte store per
  // route); tpg threads share a group
  constexpr int VEC = 16 / sizeof(TIn);
  constexpr int EPT = VEC * W;
  using VIn = Vec<TIn, VEC>;
  using VOut = Vec<typename QTraits<QT>::type, EPT>;
  const int row_units = cols / EPT;
  if (blockIdx.x < quant_blocks) {
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t token = tid / row_units;
    const int unit_in_row = (int)(tid - token * row_units);
    const bool live = token < num_tokens;
    VIn v[W];
    float amax = 0.f;
    if (live) {
#pragma unroll
      for (int w = 0; w < W; ++w) {
        v[w] = reinterpret_cast<const VIn*>(x)[tid * W + w];
#pragma unroll
        for (int i = 0; i < VEC; ++i) amax = fmaxf(amax, fabsf(to_f32(v[w].v[i])));
      }
    }
    for (int o = tpg >> 1; o > 0; o >>= 1)
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (!live) return;
    float scale, inv;
    scale_from_amax<QT, POW2>(amax, scale, inv);
    VOut o;
#pragma unroll
    for (int w = 0; w < W; ++w)
#pragma unroll
      for (int i = 0; i < VEC; ++i)
        o.v[w * VEC + i] = quant_one<QT, POW2>(to_f32(v[w].v[i]), inv);
    const bool leader = (unit_in_row % tpg) == 0;
    const int grp = unit_in_row / tpg;
    if (token_order) {
      // codes once, in token order (the GEMM gathers rows itself); only scales go to the routes
      reinterpret_cast<VOut*>(dst)[token * row_units + unit_in_row] = o;
      if (!leader) return;
    }
    // eight routes at a time: all positions first, then the independent stores
    for (int k0 = 0; k0 < slots; k0 += 8) {
      int pos[8];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        pos[j] = (k0 + j < slots) ? __ldg(route_pos + token * slots + k0 + j) : -1;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (pos[j] < 0 || pos[j] >= capacity) continue;
        if (!token_order)
          reinterpret_cast<VOut*>(dst)[(int64_t)pos[j] * row_units + unit_in_row] = o;
        if (leader) dst_scale[(int64_t)grp * dst_scale_ld + pos[j]] = scale;
      }
    }
    return;
  }
  // padding rows
  const int pad_blocks = gridDim.x - (int)quant_blocks;
  zero_pad_rows<typename QTraits<QT>::type, EPT>(
      sorted_ids, num_tokens, min(*num_valid, capacity), row_units, row_units / tpg, dst,
      dst_scale, dst_scale_ld, (int)(blockIdx.x - quant_blocks) * 8 + (threadIdx.x >> 5),
      pad_blocks * 8, token_order != 0);
}

// Same for groups that span up to 8 x 32 vectors (per-token quantisation of mid-sized rows): one
// warp owns a group, keeps it in registers between the absmax pass and the stores.
template <typename TIn, int QT, bool POW2, int NV>
__global__ void __launch_bounds__(256) k_quant_scatter_warp(
    const TIn* __restrict__ x, int64_t num_tokens, int cols, int group,
    const int32_t* __restrict__ route_pos, int slots, const int32_t* __restrict__ sorted_ids,
    const int32_t* __restrict__ num_valid, int capacity,
    typename QTraits<QT>::type* __restrict__ dst, float* __restrict__ dst_scale,
    int64_t dst_scale_ld, int quant_blocks, int token_order) {
  constexpr int VEC = 16 / sizeof(TIn);
  using VIn = Vec<TIn, VEC>;
  using VOut = Vec<typename QTraits<QT>::type, VEC>;
  const int lane = threadIdx.x & 31;
  const int groups = cols / group;
  const int nvec = group / VEC;
  const int row_vecs = cols / VEC;
  if ((int)blockIdx.x < quant_blocks) {
    const int64_t warp0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)quant_blocks * blockDim.x) >> 5;
    const int64_t num_groups = num_tokens * groups;
    for (int64_t g = warp0; g < num_groups; g += nwarps) {
      const int64_t token = g / groups;
      const int grp = (int)(g - token * groups);
      const VIn* xr = reinterpret_cast<const VIn*>(x + g * (int64_t)group);
      VIn cache[NV];
      float amax = 0.f;
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        const int i = lane + j * 32;
        if (i < nvec) {
          cache[j] = xr[i];
#pragma unroll
          for (int e = 0; e < VEC; ++e) amax = fmaxf(amax, fabsf(to_f32(cache[j].v[e])));
        }
      }
      for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      float scale, inv;
      scale_from_amax<QT, POW2>(amax, scale, inv);
      VOut out[NV];
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        if (lane + j * 32 < nvec) {
#pragma unroll
          for (int e = 0; e < VEC; ++e)
            out[j].v[e] = quant_one<QT, POW2>(to_f32(cache[j].v[e]), inv);
        }
      }
      if (token_order) {
        VOut* d = reinterpret_cast<VOut*>(dst) + token * row_vecs + grp * nvec;
#pragma unroll
        for (int j = 0; j < NV; ++j)
          if (lane + j * 32 < nvec) d[lane + j * 32] = out[j];
      }
      // lane k holds the position of route k (slots <= 32 per pass)
      for (int k0 = 0; k0 < slots; k0 += 32) {
        const int mine = (k0 + lane < slots) ? __ldg(route_pos + token * slots + k0 + lane) : -1;
        const int nk = min(32, slots - k0);
        for (int k = 0; k < nk; ++k) {
        const int pos = __shfl_sync(0xffffffffu, mine, k);
        if (pos < 0 || pos >= capacity) continue;
        if (!token_order) {
          VOut* d = reinterpret_cast<VOut*>(dst) + (int64_t)pos * row_vecs + grp * nvec;
#pragma unroll
          for (int j = 0; j < NV; ++j)
            if (lane + j * 32 < nvec) d[lane + j * 32] = out[j];
        }
        if (lane == 0) dst_scale[(int64_t)grp * dst_scale_ld + pos] = scale;
        }
      }
    }
    return;
  }
  const int pad_blocks = gridDim.x - quant_blocks;
  zero_pad_rows<typename QTraits<QT>::type, VEC>(
      sorted_ids, num_tokens, min(*num_valid, capacity), row_vecs, groups, dst, dst_scale,
      dst_scale_ld, ((int)blockIdx.x - quant_blocks) * 8 + (threadIdx.x >> 5), pad_blocks * 8,
      token_order != 0);
}

template <typename TIn, int QT, bool POW2>
int launch_quant_scatter(const void* x, int64_t num_tokens, int cols, int group,
                         const int32_t* route_pos, int slots, const int32_t* sorted_ids,
                         const int32_t* num_valid, int capacity, void* dst, float* dst_scale,
                         int64_t dst_scale_ld, int token_order, cudaStream_t st) {
  constexpr int VEC = 16 / sizeof(TIn);
  const int tpg = group / VEC;
  // (with codes in token order the padding job is a few scale words per row: fewer blocks)
  const int pad_blocks = token_order ? sm_count_of_current_device() / 2
                                     : sm_count_of_current_device() * 4;
  if (tpg > 32 || (tpg & (tpg - 1)) != 0) {
    // a warp per group, groups strided over a capped grid
    const int64_t num_groups = num_tokens * (cols / group);
    int64_t qb = (num_groups + 7) / 8;
    const int64_t cap = (int64_t)sm_count_of_current_device() * 32;
    if (qb > cap) qb = cap;
    if (qb < 1) qb = 1;
    k_quant_scatter_warp<TIn, QT, POW2, 8><<<(unsigned)(qb + pad_blocks), 256, 0, st>>>(
        static_cast<const TIn*>(x), num_tokens, cols, group, route_pos, slots, sorted_ids,
        num_valid, capacity, static_cast<typename QTraits<QT>::type*>(dst), dst_scale,
        dst_scale_ld, (int)qb, token_order);
    BOLT_LAUNCH_CHECK();
    return BOLT_OK;
  }
  // 16 output bytes per thread when the group allows it (at least two threads per group stay)
  constexpr int W16 = 16 / VEC;
  const bool wide = (group % 16 == 0) && (group / 16) >= 1 && ((group / 16) & (group / 16 - 1)) == 0;
  const int ept = wide ? 16 : VEC;
  const int64_t threads = num_tokens * (cols / ept);
  const int64_t quant_blocks = (threads + 255) / 256;
  BOLT_REQUIRE(quant_blocks + pad_blocks < (int64_t)1 << 31, "quant_scatter: too many elements");
  if (wide) {
    k_quant_scatter<TIn, QT, POW2, W16><<<(unsigned)(quant_blocks + pad_blocks), 256, 0, st>>>(
        static_cast<const TIn*>(x), num_tokens, cols, group / 16, route_pos, slots, sorted_ids,
        num_valid, capacity, static_cast<typename QTraits<QT>::type*>(dst), dst_scale,
        dst_scale_ld, quant_blocks, token_order);
  } else {
    k_quant_scatter<TIn, QT, POW2, 1><<<(unsigned)(quant_blocks + pad_blocks), 256, 0, st>>>(
        static_cast<const TIn*>(x), num_tokens, cols, tpg, route_pos, slots, sorted_ids,
        num_valid, capacity, static_cast<typename QTraits<QT>::type*>(dst), dst_scale,
        dst_scale_ld, quant_blocks, token_order);
  }
  BOLT_LAUNCH_CHECK();
  return BOLT_OK;
}

template <typename TIn>
int dispatch_quant_scatter(const void* x, int64_t num_tokens, int cols, int group, int q_dtype,
                           int power2, const int32_t* route_pos, int slots,
                           const int32_t* sorted_ids, const int32_t* num_valid, int capacity,
                           void* dst, float* dst_scale, int64_t dst_scale_ld, int token_order,
                           cudaStream_t st) {
  constexpr int VEC = 16 / sizeof(TIn);
  const int tpg = group / VEC;
  BOLT_REQUIRE(group % VEC == 0 && tpg >= 1 && tpg <= 8 * 32,
               "quant_scatter: group %d must be a multiple of %d elements, at most %d", group,
               VEC, 8 * 32 * VEC);
#define BOLT_QS(QT, P2)                                                                         \
  return launch_quant_scatter<TIn, QT, P2>(x, num_tokens, cols, group, route_pos, slots,        \
                                           sorted_ids, num_valid, capacity, dst, dst_scale,     \
                                           dst_scale_ld, token_order, st)
  if (q_dtype == BOLT_FP8_E4M3) {
    if (power2) BOLT_QS(BOLT_FP8_E4M3, true);
    BOLT_QS(BOLT_FP8_E4M3, false);
  }
  BOLT_QS(BOLT_INT8, false);
#undef BOLT_QS
}

// ---- MX (OCP microscaling) e4m3: 1 x 32 groups, power-of-two E8M0 scales ---------------------
// exponent byte = clamp(ceil(log2(amax / 448)) + 127, 0, 254), q = e4m3(v * 2^(127 - byte)),
// optionally after a split gated activation  min(g, L) * sigmoid(alpha g) * (clamp(u, +-L) + beta)
// computed in fp32 from [rows, 2 cols] = [gate | up].  Four lanes share a group (8 elements each).
// Outputs (each optional): codes, exponent bytes, and the dequantised values q * 2^(byte - 127)
// in a 16- or 32-bit float type (exact: an e4m3 value times a power of two).
template <typename TIn, typename TDeq>
__global__ void __launch_bounds__(256) k_mx_quant(const TIn* __restrict__ x, int64_t rows, int cols,
                                                  int gated, float alpha, float beta,
                                                  int has_limit, float limit,
                                                  uint8_t* __restrict__ q,
                                                  uint8_t* __restrict__ scales,
                                                  TDeq* __restrict__ deq) {
  const int units = cols / 8;                       // 8-element units per output row
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t row = tid / units;
  const int unit = (int)(tid - row * units);
  const bool live = row < rows;
  const int in_cols = gated ? 2 * cols : cols;
  float v[8];
  float amax = 0.f;
  if (live) {
    const TIn* src = x + row * (int64_t)in_cols + unit * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = to_f32(src[i]);
    if (gated) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float g = v[i], u = to_f32(src[cols + i]);
        if (has_limit) {
          g = fminf(g, limit);
          u = fminf(fmaxf(u, -limit), limit);
        }
        v[i] = g * __frcp_rn(1.0f + expf(-alpha * g)) * (u + beta);
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
  }
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  if (!live) return;
  amax = fmaxf(amax, 1.1754943508222875e-38f);
  const float e = fminf(fmaxf(ceilf(log2f(__fdiv_rn(amax, 448.0f))) + 127.0f, 0.0f), 254.0f);
  const int byte = (int)e;
  const float down = exp2f(127.0f - e);             // exact powers of two
  const float up2 = exp2f(e - 127.0f);
  uint8_t code[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) code[i] = f32_to_e4m3(v[i] * down);
  const int64_t o = row * (int64_t)cols + unit * 8;
  if (q != nullptr) {
    uint2 w;
    w.x = code[0] | (code[1] << 8) | (code[2] << 16) | ((uint32_t)code[3] << 24);
    w.y = code[4] | (code[5] << 8) | (code[6] << 16) | ((uint32_t)code[7] << 24);
    *reinterpret_cast<uint2*>(q + o) = w;
  }
  if (scales != nullptr && (unit & 3) == 0) scales[row * (int64_t)(cols / 32) + unit / 4] = (uint8_t)byte;
  if (deq != nullptr) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const __nv_fp8_e4m3 c = *reinterpret_cast<const __nv_fp8_e4m3*>(&code[i]);
      deq[o + i] = from_f32<TDeq>(float(c) * up2);
    }
  }
}

// codes [rows, cols] e4m3 + exponent bytes [rows, cols/32] -> floats (checkpoint weights)
template <typename TDeq>
__global__ void __launch_bounds__(256) k_mx_dequant(const uint8_t* __restrict__ q,
                                                    const uint8_t* __restrict__ scales,
                                                    int64_t rows, int cols,
                                                    TDeq* __restrict__ out) {
  const int units = cols / 8;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t row = tid / units;
  if (row >= rows) return;
  const int unit = (int)(tid - row * units);
  const int64_t o = row * (int64_t)cols + unit * 8;
  const float s = exp2f((float)scales[row * (int64_t)(cols / 32) + unit / 4] - 127.0f);
  const uint2 w = *reinterpret_cast<const uint2*>(q + o);
  const uint8_t* c = reinterpret_cast<const uint8_t*>(&w);
#pragma unroll
  for (int i = 0; i < 8; ++i)
    out[o + i] = from_f32<TDeq>(float(*reinterpret_cast<const __nv_fp8_e4m3*>(&c[i])) * s);
}

// E8M0 bytes [rows, sf_cols] (one per 32 K elements) -> the tiled layout the block-scaled MMA
// reads through TMEM: tiles of 128 rows x 4 K groups = 512 bytes, [row tile][K block][512], byte
// (r % 32) * 16 + (r / 32) * 4 + g.  With row_ids the rows are gathered (sorted layout, token in
// the low 24 bits); rows without a source get byte 0, a valid tiny scale.
__global__ void __launch_bounds__(256) k_mx_sf_layout(const uint8_t* __restrict__ src,
                                                      int64_t src_rows, int sf_cols,
                                                      const int32_t* __restrict__ row_ids,
                                                      const int32_t* __restrict__ num_valid,
                                                      int64_t dst_rows,
                                                      uint8_t* __restrict__ dst) {
  const int num_kb = sf_cols / 4;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t r = tid / num_kb;
  if (r >= dst_rows) return;
  const int kb = (int)(tid - r * num_kb);
  int64_t s = r;
  bool ok = r < src_rows;
  if (row_ids != nullptr) {
    const int64_t valid = num_valid != nullptr ? *num_valid : dst_rows;
    s = row_ids[r] & 0xFFFFFF;
    ok = r < valid && s < src_rows;
  }
  uint32_t w = 0;
  if (ok) w = *reinterpret_cast<const uint32_t*>(src + s * (int64_t)sf_cols + kb * 4);
  const int rr = (int)(r & 127);
  const int64_t off = ((r >> 7) * num_kb + kb) * 512 + (rr & 31) * 16 + (rr >> 5) * 4;
  *reinterpret_cast<uint32_t*>(dst + off) = w;
}

}  // namespace
}  // namespace bolt

extern "C" int bolt_quant_rows(const void* x, int x_dtype, int64_t rows, int cols, int group,
                               int q_dtype, int power2, void* q, float* scales_ptr,
                               int64_t scales_ld, void* stream) {
  using namespace bolt;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  BOLT_REQUIRE(scales_ld == 0 || scales_ld >= rows, "quant: scales_ld %lld below the row count",
               (long long)scales_ld);
  const ScaleOut scales{scales_ptr, group > 0 ? cols / group : 1, scales_ld};
  BOLT_REQUIRE(rows >= 0 && cols > 0, "quant: bad shape");
  BOLT_REQUIRE(group > 0 && cols % group == 0, "quant: group %d does not divide cols %d", group,
               cols);
  BOLT_REQUIRE(q_dtype == BOLT_FP8_E4M3 || q_dtype == BOLT_INT8, "quant: bad q_dtype %d", q_dtype);
  BOLT_REQUIRE(!power2 || q_dtype == BOLT_FP8_E4M3, "quant: power-of-two scales need e4m3");
  BOLT_REQUIRE(rows == 0 || (x && q && scales_ptr), "quant: null pointer");
  switch (x_dtype) {
    case BOLT_BF16:
      return dispatch_quant<__nv_bfloat16>(x, rows, cols, group, q_dtype, power2, q, scales, st);
    case BOLT_F16:
      return dispatch_quant<__half>(x, rows, cols, group, q_dtype, power2, q, scales, st);
    case BOLT_F32:
      return dispatch_quant<float>(x, rows, cols, group, q_dtype, power2, q, scales, st);
    default:
      set_error("quant: unsupported input dtype %d", x_dtype);
      return BOLT_ERR_INVALID;
  }
}

extern "C" int bolt_gather_rows(const void* src, int num_tokens, int row_bytes,
                                int64_t src_stride_bytes, const float* src_scale,
                                int64_t src_scale_stride, int groups, const int32_t* sorted_ids,
                                const int32_t* num_valid_ids, int capacity, void* dst,
                                float* dst_scale, int64_t dst_scale_ld, void* stream) {
  using namespace bolt;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  BOLT_REQUIRE(row_bytes > 0 && row_bytes % 16 == 0, "gather: row_bytes must be a multiple of 16");
  if (src_stride_bytes == 0) src_stride_bytes = row_bytes;
  if (src_scale_stride == 0) src_scale_stride = groups;
  BOLT_REQUIRE(src_stride_bytes >= row_bytes && src_stride_bytes % 16 == 0,
               "gather: source row stride must be a multiple of 16 bytes, at least one row");
  BOLT_REQUIRE(src_scale == nullptr || src_scale_stride >= groups,
               "gather: scale row stride below the group count");
  BOLT_REQUIRE(capacity >= 0 && num_tokens >= 0, "gather: bad sizes");
  if (capacity == 0 || num_tokens == 0) return BOLT_OK;
  BOLT_REQUIRE(src && dst && sorted_ids && num_valid_ids, "gather: null pointer");
  BOLT_REQUIRE((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) % 16 == 0,
               "gather: buffers must be 16-byte aligned");
  BOLT_REQUIRE(src_scale == nullptr || (dst_scale != nullptr && groups >= 1),
               "gather: scale arguments inconsistent");
  const int max_grid = sm_count_of_current_device() * 16;
  const int grid = capacity < max_grid ? capacity : max_grid;
  k_gather_rows<<<grid, 256, 0, st>>>(static_cast<const uint4*>(src), num_tokens, row_bytes / 16,
                                      src_stride_bytes / 16, src_scale, src_scale_stride, groups,
                                      sorted_ids, num_valid_ids, capacity,
                                      static_cast<uint4*>(dst), dst_scale, dst_scale_ld);
  BOLT_LAUNCH_CHECK();
  return BOLT_OK;
}

extern "C" int bolt_quant_scatter_rows(const void* x, int x_dtype, int64_t num_tokens, int cols,
                                       int group, int q_dtype, int power2,
                                       const int32_t* route_pos, int slots,
                                       const int32_t* sorted_ids, const int32_t* num_valid_ids,
                                       int capacity, void* dst, float* dst_scale,
                                       int64_t dst_scale_ld, int codes_in_token_order,
                                       void* stream) {
  using namespace bolt;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  BOLT_REQUIRE(num_tokens >= 0 && cols > 0 && capacity >= 0 && slots > 0,
               "quant_scatter: bad shape");
  BOLT_REQUIRE(group > 0 && cols % group == 0, "quant_scatter: group %d does not divide cols %d",
               group, cols);
  BOLT_REQUIRE(q_dtype == BOLT_FP8_E4M3 || q_dtype == BOLT_INT8, "quant_scatter: bad q_dtype %d",
               q_dtype);
  BOLT_REQUIRE(!power2 || q_dtype == BOLT_FP8_E4M3,
               "quant_scatter: power-of-two scales need e4m3");
  BOLT_REQUIRE(dst_scale_ld >= capacity, "quant_scatter: dst_scale_ld too small");
  if (capacity == 0) return BOLT_OK;
  BOLT_REQUIRE(dst && dst_scale && sorted_ids && num_valid_ids &&
                   (num_tokens == 0 || (x && route_pos)),
               "quant_scatter: null pointer");
  BOLT_REQUIRE((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dst)) % 16 == 0,
               "quant_scatter: buffers must be 16-byte aligned");
  switch (x_dtype) {
    case BOLT_BF16:
      return dispatch_quant_scatter<__nv_bfloat16>(x, num_tokens, cols, group, q_dtype, power2,
                                                   route_pos, slots, sorted_ids, num_valid_ids,
                                                   capacity, dst, dst_scale, dst_scale_ld,
                                                   codes_in_token_order, st);
    case BOLT_F16:
      return dispatch_quant_scatter<__half>(x, num_tokens, cols, group, q_dtype, power2,
                                            route_pos, slots, sorted_ids, num_valid_ids, capacity,
                                            dst, dst_scale, dst_scale_ld, codes_in_token_order, st);
    case BOLT_F32:
      return dispatch_quant_scatter<float>(x, num_tokens, cols, group, q_dtype, power2, route_pos,
                                           slots, sorted_ids, num_valid_ids, capacity, dst,
                                           dst_scale, dst_scale_ld, codes_in_token_order, st);
    default:
      set_error("quant_scatter: unsupported input dtype %d", x_dtype);
      return BOLT_ERR_INVALID;
  }
}

extern "C" int bolt_mx_quant_rows(const void* x, int x_dtype, int64_t rows, int cols, int gated,
                                  float alpha, float beta, int has_limit, float limit, void* q,
                                  uint8_t* scales, void* deq, int deq_dtype, void* stream) {
  using namespace bolt;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  BOLT_REQUIRE(rows >= 0 && cols > 0 && cols % 32 == 0, "mx_quant: cols %d must be a multiple of 32",
               cols);
  BOLT_REQUIRE(q != nullptr || deq != nullptr, "mx_quant: no output requested");
  if (rows == 0) return BOLT_OK;
  BOLT_REQUIRE(x != nullptr, "mx_quant: null input");
  BOLT_REQUIRE(q == nullptr || reinterpret_cast<uintptr_t>(q) % 8 == 0, "mx_quant: q misaligned");
  const int64_t threads = rows * (cols / 8);
  const int64_t blocks = (threads + 255) / 256;
  BOLT_REQUIRE(blocks < ((int64_t)1 << 31), "mx_quant: too many elements");
#define BOLT_MXQ(TIn, TDeq)                                                                    \
  k_mx_quant<TIn, TDeq><<<(unsigned)blocks, 256, 0, st>>>(                                     \
      static_cast<const TIn*>(x), rows, cols, gated, alpha, beta, has_limit, limit,            \
      static_cast<uint8_t*>(q), scales, static_cast<TDeq*>(deq))
#define BOLT_MXQ_IN(TDeq)                                                                      \
  switch (x_dtype) {                                                                           \
    case BOLT_BF16: BOLT_MXQ(__nv_bfloat16, TDeq); break;                                      \
    case BOLT_F16: BOLT_MXQ(__half, TDeq); break;                                              \
    case BOLT_F32: BOLT_MXQ(float, TDeq); break;                                               \
    default: set_error("mx_quant: unsupported input dtype %d", x_dtype); return BOLT_ERR_INVALID; \
  }
  switch (deq == nullptr ? BOLT_BF16 : deq_dtype) {
    case BOLT_BF16: BOLT_MXQ_IN(__nv_bfloat16); break;
    case BOLT_F16: BOLT_MXQ_IN(__half); break;
    case BOLT_F32: BOLT_MXQ_IN(float); break;
    default: set_error("mx_quant: unsupported output dtype %d", deq_dtype); return BOLT_ERR_INVALID;
  }
#undef BOLT_MXQ_IN
#undef BOLT_MXQ
  BOLT_LAUNCH_CHECK();
  return BOLT_OK;
}

extern "C" int bolt_mx_dequant_rows(const void* q, const uint8_t* scales, int64_t rows, int cols,
                                    void* out, int out_dtype, void* stream) {
  using namespace bolt;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  BOLT_REQUIRE(rows >= 0 && cols > 0 && cols % 32 == 0,
               "mx_dequant: cols %d must be a multiple of 32", cols);
  if (rows == 0) return BOLT_OK;
  BOLT_REQUIRE(q && scales && out, "mx_dequant: null pointer");
  BOLT_REQUIRE(reinterpret_cast<uintptr_t>(q) % 8 == 0, "mx_dequant: codes misaligned");
  const int64_t threads = rows * (cols / 8);
  const int64_t blocks = (threads + 255) / 256;
  BOLT_REQUIRE(blocks < ((int64_t)1 << 31), "mx_dequant: too many elements");
  switch (out_dtype) {
    case BOLT_BF16:
      k_mx_dequant<__nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>(
          static_cast<const uint8_t*>(q), scales, rows, cols, static_cast<__nv_bfloat16*>(out));
      break;
    case BOLT_F16:
      k_mx_dequant<__half><<<(unsigned)blocks, 256, 0, st>>>(
          static_cast<const uint8_t*>(q), scales, rows, cols, static_cast<__half*>(out));
      break;
    case BOLT_F32:
      k_mx_dequant<float><<<(unsigned)blocks, 256, 0, st>>>(
          static_cast<const uint8_t*>(q), scales, rows, cols, static_cast<float*>(out));
      break;
    default: set_error("mx_dequant: unsupported output dtype %d", out_dtype); return BOLT_ERR_INVALID;
  }
  BOLT_LAUNCH_CHECK();
  return BOLT_OK;
}

extern "C" int bolt_mx_sf_layout(const uint8_t* src, int64_t src_rows, int sf_cols,
                                 const int32_t* row_ids, const int32_t* num_valid_ids,
                                 int64_t dst_rows, uint8_t* dst, void* stream) {
  using namespace bolt;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  BOLT_REQUIRE(src_rows >= 0 && dst_rows >= 0 && dst_rows % 128 == 0,
               "mx_sf_layout: dst_rows must be a multiple of 128");
  BOLT_REQUIRE(sf_cols > 0 && sf_cols % 4 == 0, "mx_sf_layout: sf_cols %d must be a multiple of 4",
               sf_cols);
  if (dst_rows == 0) return BOLT_OK;
  BOLT_REQUIRE(dst != nullptr && (src != nullptr || src_rows == 0), "mx_sf_layout: null pointer");
  BOLT_REQUIRE((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) % 4 == 0,
               "mx_sf_layout: buffers must be 4-byte aligned");
  const int64_t threads = dst_rows * (sf_cols / 4);
  const int64_t blocks = (threads + 255) / 256;
  BOLT_REQUIRE(blocks < ((int64_t)1 << 31), "mx_sf_layout: too many elements");
  k_mx_sf_layout<<<(unsigned)blocks, 256, 0, st>>>(src, src_rows, sf_cols, row_ids, num_valid_ids,
                                                   dst_rows, dst);
  BOLT_LAUNCH_CHECK();
  return BOLT_OK;
}
