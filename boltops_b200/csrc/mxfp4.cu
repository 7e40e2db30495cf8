// MXFP4 (w4a8) experts: packed e2m1 weights with one E8M0 byte per 32 K elements, e4m3
// activations (dynamic 1 x 128 groups with power-of-two scales, or one static fp32 scale).
//
// Everything an e2m1 or e4m3 code stands for, times a power of two, is exactly representable in
// bf16, and products of two such values are exact in fp32.  The expert GEMMs therefore run on the
// 16-bit tensor-core kind over DECODED operands with fp32 accumulation -- the same contraction as
// the reference's K-grouped scaled dot (boltops/fused_moe/triton/mxfp4.py:61-157) -- and the
// kernels here do the decoding and the quantise-then-decode steps around them:
//   k_mxfp4_decode        weights      packed nibbles + E8M0 bytes  -> bf16 / f16 / f32
//   k_mx4_act_quant       activations  [optional SiLU(gate)*up] -> 1 x 128 power-of-two quantiser
//                                      (or one static scale) -> e4m3 -> decoded values
//   k_fp8_group_decode    pre-quantised activations: codes * fp32 group scale -> decoded values
//   k_mx4_swiglu_static   static recipe between the GEMMs: * a1_scale, + bias, SwiGLU-OAI,
//                                      [* router weight], e4m3(. / a2_scale)
//   k_mx4_affine_rows     static recipe after GEMM2: * a2_scale, + bias, [* router weight], cast
// Arithmetic follows boltops/fused_moe/triton/mxfp4_quant.py:38-56 and the CPU statement in
// test/fused_moe/test_fused_moe.py:1411-1563 of the reference project.
#include "common.cuh"

namespace bolt {
namespace {

__device__ __forceinline__ float e2m1_value(uint32_t code) {
  // magnitudes 0, .5, 1, 1.5, 2, 3, 4, 6; bit 3 = sign
  const uint32_t m = code & 7u;
  float v = m < 2 ? 0.5f * (float)m : ldexpf(1.0f + 0.5f * (float)(m & 1u), (int)(m >> 1) - 1);
  return (code & 8u) ? -v : v;
}

template <typename T>
__device__ __forceinline__ void store_as(T* p, float v);
template <>
__device__ __forceinline__ void store_as<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void store_as<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ void store_as<__half>(__half* p, float v) { *p = __float2half_rn(v); }

__device__ __forceinline__ float e4m3_to_f32(uint8_t code) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw(code, __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}

template <typename TOut>
__global__ void __launch_bounds__(256) k_mxfp4_decode(const uint8_t* __restrict__ packed,
                                                      const uint8_t* __restrict__ scales,
                                                      int64_t rows, int cols,
                                                      TOut* __restrict__ out) {
  // one thread per 8 packed bytes = 16 values (half of an E8M0 group)
  const int units = cols / 16;
  const int64_t total = rows * units;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / units;
    const int u = (int)(i - row * units);
    const float s = exp2f((float)scales[row * (cols / 32) + u / 2] - 127.0f);
    const uint2 raw = *reinterpret_cast<const uint2*>(packed + row * (cols / 2) + u * 8);
    TOut* o = out + row * cols + u * 16;
#pragma unroll
    for (int b = 0; b < 8; ++b) {
      const uint32_t byte = ((b < 4 ? raw.x : raw.y) >> (8 * (b & 3))) & 0xFFu;
      store_as<TOut>(o + 2 * b, e2m1_value(byte & 15u) * s);        // low nibble first
      store_as<TOut>(o + 2 * b + 1, e2m1_value(byte >> 4) * s);
    }
  }
}

template <typename T>
__device__ __forceinline__ float load_as(const T* p) { return to_f32(*p); }

// One warp per (row, 128-wide group); a lane owns 4 consecutive elements.
//   gated  : x is [rows, 2 * cols] = [gate | up]; v = up * gate / (1 + exp(-gate)) with the
//            optional clamp (gate <= limit, |up| <= limit), rounded through bf16
//   mode 0 : dynamic -- scale = the power of two at or above max(amax, 1e-10) / 448 (floored at
//            1e-10), q = e4m3(clamp(v * (1 / scale)))
//   mode 1 : static  -- q = e4m3(v / *static_scale); the decoded value is the code itself
//   x8     : x holds e4m3 codes (static recipe, pre-quantised): decoded as they are
// Outputs (each optional): deq = decoded values, codes, scales (fp32, dynamic mode), sf32 = the
// scale's exponent byte repeated per 32 elements ([rows, cols/32], dynamic mode).
template <typename TIn, typename TOut>
__global__ void __launch_bounds__(256) k_mx4_act_quant(
    const TIn* __restrict__ x, int64_t rows, int cols, int gated, int has_limit, float limit,
    int mode, const float* __restrict__ static_scale, int x8, TOut* __restrict__ deq,
    uint8_t* __restrict__ codes, float* __restrict__ scales, uint8_t* __restrict__ sf32) {
  const int lane = threadIdx.x & 31;
  const int groups = cols / 128;
  const int64_t total = rows * groups;
  const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int64_t in_ld = gated ? 2 * (int64_t)cols : cols;
  for (int64_t g = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; g < total; g += warps) {
    const int64_t row = g / groups;
    const int col0 = (int)(g - row * groups) * 128 + 4 * lane;
    float v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (x8) {
        v[j] = e4m3_to_f32(reinterpret_cast<const uint8_t*>(x)[row * in_ld + col0 + j]);
      } else if (gated) {
        float gate = load_as(x + row * in_ld + col0 + j);
        float up = load_as(x + row * in_ld + cols + col0 + j);
        if (has_limit) {
          gate = fminf(gate, limit);
          up = fminf(fmaxf(up, -limit), limit);
        }
        const float y = __fdiv_rn(up * gate, 1.0f + expf(-gate));
        v[j] = __bfloat162float(__float2bfloat16_rn(y));
      } else {
        v[j] = load_as(x + row * in_ld + col0 + j);
      }
    }
    float scale = 1.0f, q[4];
    if (x8) {
#pragma unroll
      for (int j = 0; j < 4; ++j) q[j] = v[j];
    } else if (mode == 1) {
      const float s = *static_scale;
#pragma unroll
      for (int j = 0; j < 4; ++j) q[j] = __fdiv_rn(v[j], s);
    } else {
      float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      const float raw = fmaxf(__fdiv_rn(fmaxf(amax, 1.0e-10f), 448.0f), 1.0e-10f);
      const uint32_t bits = __float_as_uint(raw);
      const uint32_t e = ((bits >> 23) & 255u) + ((bits & 0x7fffffu) != 0u ? 1u : 0u);
      scale = __uint_as_float(e << 23);
      const float inv = __fdiv_rn(1.0f, scale);
#pragma unroll
      for (int j = 0; j < 4; ++j) q[j] = fminf(fmaxf(v[j] * inv, -448.0f), 448.0f);
      if (scales != nullptr && lane == 0) scales[g] = scale;
      // the same scale as four E8M0 bytes (one per 32 elements) for the tensor core's block scaling
      if (sf32 != nullptr && lane == 0) reinterpret_cast<uint32_t*>(sf32)[g] = e * 0x01010101u;
    }
    uint32_t packed = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint8_t c = x8 ? reinterpret_cast<const uint8_t*>(x)[row * in_ld + col0 + j]
                           : f32_to_e4m3(q[j]);
      packed |= (uint32_t)c << (8 * j);
      if (deq != nullptr) store_as<TOut>(deq + row * cols + col0 + j, e4m3_to_f32(c) * scale);
    }
    if (codes != nullptr) *reinterpret_cast<uint32_t*>(codes + row * cols + col0) = packed;
  }
}

template <typename TOut>
__global__ void __launch_bounds__(256) k_fp8_group_decode(const uint8_t* __restrict__ codes,
                                                          const float* __restrict__ scales,
                                                          int64_t rows, int cols, int group,
                                                          TOut* __restrict__ out) {
  const int64_t total = rows * cols;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / cols;
    const int col = (int)(i - row * cols);
    store_as<TOut>(out + i, e4m3_to_f32(codes[i]) * scales[row * (cols / group) + col / group]);
  }
}

// rows in the expert-sorted layout: expert of row r = expert_ids[r / 128]
template <typename TOut>
__global__ void __launch_bounds__(256) k_mx4_swiglu_static(
    const float* __restrict__ g1, const int32_t* __restrict__ expert_ids,
    const int32_t* __restrict__ num_valid, int capacity, int inter, int num_experts,
    const float* __restrict__ a1_scale, const float* __restrict__ bias, float alpha, float limit,
    const float* __restrict__ row_weight, const float* __restrict__ a2_scale,
    TOut* __restrict__ out) {
  const int valid = min(*num_valid, capacity);
  const float s1 = *a1_scale, s2 = *a2_scale;
  const int64_t total = (int64_t)valid * inter;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / inter;
    const int col = (int)(i - row * inter);
    const int e = expert_ids[row / 128];
    float gate = g1[row * 2 * inter + col] * s1;
    float up = g1[row * 2 * inter + inter + col] * s1;
    if (bias != nullptr && e >= 0 && e < num_experts) {
      gate += bias[(int64_t)e * 2 * inter + col];
      up += bias[(int64_t)e * 2 * inter + inter + col];
    }
    gate = fminf(gate, limit);
    up = fminf(fmaxf(up, -limit), limit);
    float act = gate * __fdiv_rn(1.0f, 1.0f + expf(-alpha * gate)) * (up + 1.0f);
    if (row_weight != nullptr) act *= row_weight[row];
    store_as<TOut>(out + i, e4m3_to_f32(f32_to_e4m3(__fdiv_rn(act, s2))));
  }
}

template <typename TOut>
__global__ void __launch_bounds__(256) k_mx4_affine_rows(
    const float* __restrict__ g2, const int32_t* __restrict__ expert_ids,
    const int32_t* __restrict__ sorted_ids, const int32_t* __restrict__ num_valid, int capacity,
    int cols, int num_experts, int num_tokens, int topk, const float* __restrict__ scale,
    const float* __restrict__ bias, const float* __restrict__ row_weight, int scatter,
    TOut* __restrict__ out) {
  const int valid = min(*num_valid, capacity);
  const float s = *scale;
  const int64_t total = (int64_t)valid * cols;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / cols;
    const int col = (int)(i - row * cols);
    const int sid = sorted_ids[row];
    const int token = sid & 0xFFFFFF;
    if (token >= num_tokens) continue;      // rows that only pad a tile
    const int e = expert_ids[row / 128];
    float v = g2[i] * s;
    if (bias != nullptr && e >= 0 && e < num_experts) v += bias[(int64_t)e * cols + col];
    if (row_weight != nullptr) v *= row_weight[row];
    const int64_t out_row = scatter ? (int64_t)token * topk + ((uint32_t)sid >> 24) : row;
    store_as<TOut>(out + out_row * cols + col, v);
  }
}

inline unsigned grid_for(int64_t threads) {
  int64_t blocks = (threads + 255) / 256;
  const int64_t cap = (int64_t)sm_count_of_current_device() * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (unsigned)blocks;
}

}  // namespace
}  // namespace bolt

#define BOLT_DISPATCH_OUT(dt, ...)                                        \
  switch (dt) {                                                           \
    case BOLT_BF16: { using TOut = __nv_bfloat16; __VA_ARGS__; break; }   \
    case BOLT_F16: { using TOut = __half; __VA_ARGS__; break; }           \
    case BOLT_F32: { using TOut = float; __VA_ARGS__; break; }            \
    default: set_error("mxfp4: unsupported output dtype %d", dt); return BOLT_ERR_INVALID; \
  }

extern "C" int bolt_mxfp4_decode(const uint8_t* packed, const uint8_t* scales, int64_t rows,
                                 int cols, void* out, int out_dtype, void* stream) {
  using namespace bolt;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  BOLT_REQUIRE(rows >= 0 && cols > 0 && cols % 32 == 0, "mxfp4_decode: cols must be a multiple of 32");
  if (rows == 0) return BOLT_OK;
  BOLT_REQUIRE(packed && scales && out, "mxfp4_decode: null pointer");
  BOLT_REQUIRE(reinterpret_cast<uintptr_t>(packed) % 8 == 0, "mxfp4_decode: packed rows must be 8-byte aligned");
  BOLT_DISPATCH_OUT(out_dtype, (k_mxfp4_decode<TOut><<<grid_for(rows * (cols / 16)), 256, 0, st>>>(
                                   packed, scales, rows, cols, static_cast<TOut*>(out))));
  BOLT_LAUNCH_CHECK();
  return BOLT_OK;
}

extern "C" int bolt_mx4_act_quant(const void* x, int x_dtype, int64_t rows, int cols, int gated,
                                  int has_limit, float limit, int mode, const float* static_scale,
                                  void* deq, int deq_dtype, uint8_t* codes, float* scales,
                                  uint8_t* sf32, void* stream) {
  using namespace bolt;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  BOLT_REQUIRE(rows >= 0 && cols > 0 && cols % 128 == 0,
               "mx4_act_quant: cols %d must be a multiple of 128", cols);
  BOLT_REQUIRE(mode == 0 || mode == 1, "mx4_act_quant: mode %d", mode);
  BOLT_REQUIRE(mode == 0 || static_scale != nullptr || x_dtype == BOLT_FP8_E4M3,
               "mx4_act_quant: the static mode needs its scale");
  BOLT_REQUIRE(x_dtype != BOLT_FP8_E4M3 || (mode == 1 && !gated),
               "mx4_act_quant: e4m3 input is the pre-quantised static recipe");
  if (rows == 0) return BOLT_OK;
  BOLT_REQUIRE(x != nullptr && (deq || codes), "mx4_act_quant: null pointer");
  const unsigned grid = grid_for(rows * (cols / 128) * 32);
  const int x8 = x_dtype == BOLT_FP8_E4M3;
#define BOLT_MX4_LAUNCH(TIN)                                                                   \
  BOLT_DISPATCH_OUT(deq_dtype, (k_mx4_act_quant<TIN, TOut><<<grid, 256, 0, st>>>(               \
                                   static_cast<const TIN*>(x), rows, cols, gated, has_limit,   \
                                   limit, mode, static_scale, x8, static_cast<TOut*>(deq), codes, \
                                   scales, sf32)))
  switch (x_dtype) {
    case BOLT_BF16: BOLT_MX4_LAUNCH(__nv_bfloat16); break;
    case BOLT_F16: BOLT_MX4_LAUNCH(__half); break;
    case BOLT_F32: BOLT_MX4_LAUNCH(float); break;
    case BOLT_FP8_E4M3: BOLT_MX4_LAUNCH(__nv_bfloat16); break;   // read as bytes inside
    default: set_error("mx4_act_quant: unsupported input dtype %d", x_dtype); return BOLT_ERR_INVALID;
  }
#undef BOLT_MX4_LAUNCH
  BOLT_LAUNCH_CHECK();
  return BOLT_OK;
}

extern "C" int bolt_fp8_group_decode(const uint8_t* codes, const float* scales, int64_t rows,
                                     int cols, int group, void* out, int out_dtype, void* stream) {
  using namespace bolt;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  BOLT_REQUIRE(rows >= 0 && cols > 0 && group > 0 && cols % group == 0, "fp8_group_decode: bad shape");
  if (rows == 0) return BOLT_OK;
  BOLT_REQUIRE(codes && scales && out, "fp8_group_decode: null pointer");
  BOLT_DISPATCH_OUT(out_dtype, (k_fp8_group_decode<TOut><<<grid_for(rows * cols), 256, 0, st>>>(
                                   codes, scales, rows, cols, group, static_cast<TOut*>(out))));
  BOLT_LAUNCH_CHECK();
  return BOLT_OK;
}

extern "C" int bolt_mx4_swiglu_static(const float* g1, const int32_t* sorted_expert_ids,
                                      const int32_t* num_valid_ids, int capacity, int inter,
                                      int num_experts, const float* a1_scale, const float* bias,
                                      float alpha, float limit, const float* row_weight,
                                      const float* a2_scale, void* out, int out_dtype,
                                      void* stream) {
  using namespace bolt;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  BOLT_REQUIRE(capacity >= 0 && inter > 0 && num_experts > 0, "mx4_swiglu_static: bad shape");
  if (capacity == 0) return BOLT_OK;
  BOLT_REQUIRE(g1 && sorted_expert_ids && num_valid_ids && a1_scale && a2_scale && out,
               "mx4_swiglu_static: null pointer");
  BOLT_DISPATCH_OUT(out_dtype,
                    (k_mx4_swiglu_static<TOut><<<grid_for((int64_t)capacity * inter), 256, 0, st>>>(
                        g1, sorted_expert_ids, num_valid_ids, capacity, inter, num_experts,
                        a1_scale, bias, alpha, limit, row_weight, a2_scale,
                        static_cast<TOut*>(out))));
  BOLT_LAUNCH_CHECK();
  return BOLT_OK;
}

extern "C" int bolt_mx4_affine_rows(const float* g2, const int32_t* sorted_expert_ids,
                                    const int32_t* sorted_ids, const int32_t* num_valid_ids,
                                    int capacity, int cols, int num_experts, int num_tokens,
                                    int topk, const float* scale, const float* bias,
                                    const float* row_weight, int scatter, void* out,
                                    int out_dtype, void* stream) {
  using namespace bolt;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  BOLT_REQUIRE(capacity >= 0 && cols > 0 && num_experts > 0 && topk > 0, "mx4_affine_rows: bad shape");
  if (capacity == 0) return BOLT_OK;
  BOLT_REQUIRE(g2 && sorted_expert_ids && sorted_ids && num_valid_ids && scale && out,
               "mx4_affine_rows: null pointer");
  BOLT_DISPATCH_OUT(out_dtype,
                    (k_mx4_affine_rows<TOut><<<grid_for((int64_t)capacity * cols), 256, 0, st>>>(
                        g2, sorted_expert_ids, sorted_ids, num_valid_ids, capacity, cols,
                        num_experts, num_tokens, topk, scale, bias, row_weight, scatter,
                        static_cast<TOut*>(out))));
  BOLT_LAUNCH_CHECK();
  return BOLT_OK;
}
