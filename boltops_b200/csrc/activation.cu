// Expert activations (standalone) and the fused activation + per-token
// quantisation.  HBM-bound: 128-bit accesses, fp32 math, one pass.
#include "common.cuh"

namespace bolt {
namespace {

struct ActParams {
  int kind;
  int gated;
  float alpha;
  float limit;
};

__device__ __forceinline__ float gelu_erf(float x) {
  return x * 0.5f * (1.0f + erff(x * 0.7071067811865476f));
}
__device__ __forceinline__ float gelu_tanh(float x) {
  const float k = 0.7978845608028654f;  // sqrt(2/pi)
  return 0.5f * x * (1.0f + tanhf(k * (x + 0.044715f * x * x * x)));
}

// fp32 activation of one (gate, up) pair; `u` is ignored when not gated.
__device__ __forceinline__ float act_pair(const ActParams& p, float g, float u) {
  float a;
  switch (p.kind) {
    case BOLT_ACT_SILU: a = silu_f32(g); break;
    case BOLT_ACT_GELU: a = gelu_erf(g); break;
    case BOLT_ACT_GELU_TANH: a = gelu_tanh(g); break;
    case BOLT_ACT_RELU2: a = g > 0.f ? g * g : 0.f; break;
    case BOLT_ACT_SWIGLU_OAI: {
      const float gc = fminf(g, p.limit);
      const float uc = fminf(fmaxf(u, -p.limit), p.limit);
      return gc * (1.0f / (1.0f + expf(-p.alpha * gc))) * (uc + 1.0f);
    }
    case BOLT_ACT_SWIGLU_STEP:
      a = fminf(silu_f32(g), p.limit);
      u = fminf(fmaxf(u, -p.limit), p.limit);
      break;
    case BOLT_ACT_SILU_CLAMP:
      a = silu_f32(fminf(g, p.limit));
      u = fminf(fmaxf(u, -p.limit), p.limit);
      break;
    case BOLT_ACT_SWIGLU_OAI_INTERLEAVED: {
      const float gc = fminf(g, p.limit);
      const float uc = fminf(fmaxf(u, -p.limit), p.limit);
      return gc * (1.0f / (1.0f + expf(-p.alpha * gc))) * (uc + 1.0f);
    }
    case BOLT_ACT_SITU: {
      // tanh(x) = 2*sigmoid(2x) - 1, the reference's form
      const float tg = 2.0f / (1.0f + expf(-2.0f * (g / p.alpha))) - 1.0f;
      a = p.alpha * tg * (1.0f / (1.0f + expf(-g)));
      if (p.limit > 0.f) u = p.limit * (2.0f / (1.0f + expf(-2.0f * (u / p.limit))) - 1.0f);
      break;
    }
    default: a = g; break;
  }
  return p.gated ? a * u : a;
}

// out[r, c] = act(in[r, c], in[r, n_out + c]); VEC elements per thread.
template <typename T, int VEC>
__global__ void __launch_bounds__(256) k_activation(const T* __restrict__ in, T* __restrict__ out,
                                                    int64_t rows, int n_out, ActParams p,
                                                    const int32_t* __restrict__ rows_dev) {
  using V = Vec<T, VEC>;
  if (rows_dev != nullptr) rows = min(rows, (int64_t)*rows_dev);
  const int nvec = n_out / VEC;
  const int64_t total = rows * nvec;
  const int in_ld = p.gated ? 2 * n_out : n_out;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / nvec;
    const int c = (int)(idx - r * nvec) * VEC;
    const T* row = in + r * in_ld;
    V g = *reinterpret_cast<const V*>(row + c);
    V u = g;
    if (p.gated) u = *reinterpret_cast<const V*>(row + n_out + c);
    V o;
#pragma unroll
    for (int i = 0; i < VEC; ++i) o.v[i] = from_f32<T>(act_pair(p, to_f32(g.v[i]), to_f32(u.v[i])));
    *reinterpret_cast<V*>(out + r * n_out + c) = o;
  }
}

// interleaved gate/up layout: out[r, c] = act(in[r, 2c], in[r, 2c+1])
template <typename T>
__global__ void __launch_bounds__(256) k_activation_interleaved(const T* __restrict__ in,
                                                                T* __restrict__ out, int64_t rows,
                                                                int n_out, ActParams p,
                                                                const int32_t* __restrict__ rows_dev) {
  if (rows_dev != nullptr) rows = min(rows, (int64_t)*rows_dev);
  const int64_t total = rows * n_out;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const float g = to_f32(in[2 * idx]);
    const float u = to_f32(in[2 * idx + 1]);
    out[idx] = from_f32<T>(act_pair(p, g, u));
  }
}

template <typename T>
int launch_activation(const void* in, void* out, int64_t rows, int n_out, ActParams p,
                      const int32_t* rows_dev, cudaStream_t st) {
  constexpr int VEC = 16 / sizeof(T);
  if (p.kind == BOLT_ACT_SWIGLU_OAI_INTERLEAVED) {
    const int64_t n = rows * n_out;
    if (n == 0) return BOLT_OK;
    int64_t nb = (n + 255) / 256;
    const int64_t nb_cap = (int64_t)sm_count_of_current_device() * 32;
    if (nb > nb_cap) nb = nb_cap;
    k_activation_interleaved<T><<<(unsigned)nb, 256, 0, st>>>(
        static_cast<const T*>(in), static_cast<T*>(out), rows, n_out, p, rows_dev);
    BOLT_LAUNCH_CHECK();
    return BOLT_OK;
  }
  const bool vec_ok = (n_out % VEC == 0) && (reinterpret_cast<uintptr_t>(in) % 16 == 0) &&
                      (reinterpret_cast<uintptr_t>(out) % 16 == 0);
  const int64_t total = vec_ok ? rows * (n_out / VEC) : rows * n_out;
  if (total == 0) return BOLT_OK;
  int64_t blocks = (total + 255) / 256;
  const int64_t cap = (int64_t)sm_count_of_current_device() * 32;
  if (blocks > cap) blocks = cap;
  if (vec_ok)
    k_activation<T, VEC><<<(unsigned)blocks, 256, 0, st>>>(
        static_cast<const T*>(in), static_cast<T*>(out), rows, n_out, p, rows_dev);
  else
    k_activation<T, 1><<<(unsigned)blocks, 256, 0, st>>>(
        static_cast<const T*>(in), static_cast<T*>(out), rows, n_out, p, rows_dev);
  BOLT_LAUNCH_CHECK();
  return BOLT_OK;
}

// ---- fused activation + per-token quantisation: one CTA per row ------------------
template <typename T, typename Q, bool INT8>
__global__ void __launch_bounds__(256) k_act_quant(const T* __restrict__ in, Q* __restrict__ q,
                                                   float* __restrict__ scales, int64_t rows,
                                                   int n_out, ActParams p,
                                                   const float* __restrict__ row_mult,
                                                   const int32_t* __restrict__ rows_dev) {
  extern __shared__ float ybuf[];  // [n_out] activation rounded through T
  if (rows_dev != nullptr) rows = min(rows, (int64_t)*rows_dev);
  __shared__ float red[8];
  const int in_ld = p.gated ? 2 * n_out : n_out;
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* row = in + r * in_ld;
    float amax = 0.f;
    for (int c = threadIdx.x; c < n_out; c += blockDim.x) {
      const float g = to_f32(row[c]);
      const float u = p.gated ? to_f32(row[n_out + c]) : 0.f;
      const float y = round_through<T>(act_pair(p, g, u));
      ybuf[c] = y;
      amax = fmaxf(amax, fabsf(y));
    }
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    __syncthreads();  // previous iteration's readers of red[] are done
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = red[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) amax = fmaxf(amax, red[w]);
    const float dmax = INT8 ? 127.0f : 448.0f;
    const float scale = __fdiv_rn(fmaxf(amax, 1.0e-10f), dmax);
    const float inv = __frcp_rn(scale);
    Q* qr = q + r * n_out;
    for (int c = threadIdx.x; c < n_out; c += blockDim.x) {
      const float v = ybuf[c] * inv;
      qr[c] = INT8 ? (Q)f32_to_i8(v) : (Q)f32_to_e4m3(v);
    }
    if (threadIdx.x == 0) scales[r] = row_mult ? scale * row_mult[r] : scale;
  }
}

template <typename T>
int launch_act_quant(const void* in, int64_t rows, int n_out, ActParams p, int q_dtype,
                     const float* row_mult, void* q, float* scales, const int32_t* rows_dev,
                     cudaStream_t st) {
  if (rows == 0) return BOLT_OK;
  int64_t blocks = rows;
  const int64_t cap = (int64_t)sm_count_of_current_device() * 16;
  if (blocks > cap) blocks = cap;
  const size_t smem = (size_t)n_out * sizeof(float);
  BOLT_REQUIRE(smem <= 160 * 1024, "act_quant: row of %d too wide", n_out);
  if (q_dtype == BOLT_INT8) {
    auto kfn = k_act_quant<T, int8_t, true>;
    if (smem > 48 * 1024)
      BOLT_CUDA(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kfn<<<(unsigned)blocks, 256, smem, st>>>(static_cast<const T*>(in), static_cast<int8_t*>(q),
                                             scales, rows, n_out, p, row_mult, rows_dev);
  } else {
    auto kfn = k_act_quant<T, uint8_t, false>;
    if (smem > 48 * 1024)
      BOLT_CUDA(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kfn<<<(unsigned)blocks, 256, smem, st>>>(static_cast<const T*>(in), static_cast<uint8_t*>(q),
                                             scales, rows, n_out, p, row_mult, rows_dev);
  }
  BOLT_LAUNCH_CHECK();
  return BOLT_OK;
}

int check_act(int activation, int gated) {
  BOLT_REQUIRE(activation >= BOLT_ACT_SILU && activation <= BOLT_ACT_SITU,
               "activation: unknown kind %d", activation);
  const bool needs_gate = activation == BOLT_ACT_SWIGLU_OAI || activation == BOLT_ACT_SWIGLU_STEP ||
                          activation == BOLT_ACT_SILU_CLAMP ||
                          activation == BOLT_ACT_SWIGLU_OAI_INTERLEAVED || activation == BOLT_ACT_SITU;
  BOLT_REQUIRE(!needs_gate || gated, "activation: kind %d requires gated mode", activation);
  BOLT_REQUIRE(!(activation == BOLT_ACT_RELU2 && gated), "activation: relu2 is not gated");
  return BOLT_OK;
}

}  // namespace
}  // namespace bolt

extern "C" int bolt_moe_activation(const void* in, void* out, int dtype, int64_t rows, int n_out,
                                   int activation, int gated, float alpha, float limit,
                                   const int32_t* rows_dev, void* stream) {
  using namespace bolt;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  BOLT_REQUIRE(rows >= 0 && n_out > 0, "activation: bad shape");
  if (int rc = check_act(activation, gated)) return rc;
  BOLT_REQUIRE(rows == 0 || (in && out), "activation: null pointer");
  ActParams p{activation, gated ? 1 : 0, alpha, limit};
  switch (dtype) {
    case BOLT_BF16: return launch_activation<__nv_bfloat16>(in, out, rows, n_out, p, rows_dev, st);
    case BOLT_F16: return launch_activation<__half>(in, out, rows, n_out, p, rows_dev, st);
    case BOLT_F32: return launch_activation<float>(in, out, rows, n_out, p, rows_dev, st);
    default: set_error("activation: unsupported dtype %d", dtype); return BOLT_ERR_INVALID;
  }
}

extern "C" int bolt_act_quant(const void* in, int dtype, int64_t rows, int n_out, int activation,
                              int gated, int q_dtype, const float* row_multiplier, void* q,
                              float* scales, const int32_t* rows_dev, void* stream) {
  using namespace bolt;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  BOLT_REQUIRE(rows >= 0 && n_out > 0, "act_quant: bad shape");
  if (int rc = check_act(activation, gated)) return rc;
  BOLT_REQUIRE(q_dtype == BOLT_FP8_E4M3 || q_dtype == BOLT_INT8, "act_quant: bad q_dtype");
  BOLT_REQUIRE(rows == 0 || (in && q && scales), "act_quant: null pointer");
  ActParams p{activation, gated ? 1 : 0, 1.702f, 7.0f};
  switch (dtype) {
    case BOLT_BF16:
      return launch_act_quant<__nv_bfloat16>(in, rows, n_out, p, q_dtype, row_multiplier, q,
                                             scales, rows_dev, st);
    case BOLT_F16:
      return launch_act_quant<__half>(in, rows, n_out, p, q_dtype, row_multiplier, q, scales,
                                      rows_dev, st);
    case BOLT_F32:
      return launch_act_quant<float>(in, rows, n_out, p, q_dtype, row_multiplier, q, scales,
                                     rows_dev, st);
    default: set_error("act_quant: unsupported dtype %d", dtype); return BOLT_ERR_INVALID;
  }
}
