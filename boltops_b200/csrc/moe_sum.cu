// Top-k combine: out[m, :] = cast(scale * sum_k f32(in[m, k, :]) [* w[m, k]]).
// HBM-bound: (topk + 1) * elem bytes per output element, 128-bit accesses,
// k ascending with an fp32 accumulator (matches the reference's summation order).
#include "common.cuh"

namespace bolt {
namespace {

template <typename TIn, typename TOut, int VEC>
__global__ void __launch_bounds__(256) k_moe_sum(const TIn* __restrict__ in, TOut* __restrict__ out,
                                                 int64_t num_tokens, int topk, int n, float scale,
                                                 const float* __restrict__ weights) {
  using VI = Vec<TIn, VEC>;
  using VO = Vec<TOut, VEC>;
  const int nvec = n / VEC;
  const int64_t total = num_tokens * nvec;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t m = idx / nvec;
    const int c = (int)(idx - m * nvec) * VEC;
    const TIn* base = in + (m * topk) * (int64_t)n + c;
    float acc[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[i] = 0.f;
    for (int k = 0; k < topk; ++k) {
      const VI v = *reinterpret_cast<const VI*>(base + (int64_t)k * n);
      if (weights != nullptr) {
        const float w = weights[m * topk + k];
#pragma unroll
        for (int i = 0; i < VEC; ++i) acc[i] = __fadd_rn(acc[i], __fmul_rn(to_f32(v.v[i]), w));
      } else {
#pragma unroll
        for (int i = 0; i < VEC; ++i) acc[i] += to_f32(v.v[i]);
      }
    }
    VO o;
#pragma unroll
    for (int i = 0; i < VEC; ++i) o.v[i] = from_f32<TOut>(acc[i] * scale);
    *reinterpret_cast<VO*>(out + m * (int64_t)n + c) = o;
  }
}

// out[m, :] = cast(scale * sum_j f32(src[pos[m, j], :])) over pos[m, j] >= 0, j ascending.
template <typename T, typename TOut, int VEC>
__global__ void __launch_bounds__(256) k_gather_sum(const T* __restrict__ src,
                                                    const int32_t* __restrict__ pos,
                                                    TOut* __restrict__ out, int64_t num_tokens,
                                                    int slots, int n, float scale) {
  using V = Vec<T, VEC>;
  using VO = Vec<TOut, VEC>;
  const int nvec = n / VEC;
  const int64_t total = num_tokens * nvec;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t m = idx / nvec;
    const int c = (int)(idx - m * nvec) * VEC;
    float acc[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[i] = 0.f;
    for (int j = 0; j < slots; ++j) {
      const int r = __ldg(pos + m * slots + j);
      if (r < 0) continue;
      const V v = *reinterpret_cast<const V*>(src + (int64_t)r * n + c);
#pragma unroll
      for (int i = 0; i < VEC; ++i) acc[i] += to_f32(v.v[i]);
    }
    VO o;
#pragma unroll
    for (int i = 0; i < VEC; ++i) o.v[i] = from_f32<TOut>(acc[i] * scale);
    *reinterpret_cast<VO*>(out + m * (int64_t)n + c) = o;
  }
}

// The same sum, written to other ranks' memory: row m belongs to segment s = m / seg_rows (the
// rank the token came from), rows q = m % seg_rows >= hdr[2 s] are not live and are skipped, and
// the result goes to row hdr[2 s + 1] + q of the region at seg_ptrs[s] (plain stores; the region
// may be peer memory).  first_row = index of row 0 of this call within the whole batch.
template <typename T, typename TOut, int VEC>
__global__ void __launch_bounds__(256) k_gather_sum_to_peers(
    const T* __restrict__ src, const int32_t* __restrict__ pos, int64_t num_tokens, int slots, int n,
    float scale, int64_t seg_rows, const int64_t* __restrict__ seg_ptrs,
    const int32_t* __restrict__ hdr, int64_t first_row) {
  using V = Vec<T, VEC>;
  using VO = Vec<TOut, VEC>;
  const int nvec = n / VEC;
  const int64_t total = num_tokens * nvec;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t m = idx / nvec;
    const int c = (int)(idx - m * nvec) * VEC;
    const int64_t g = first_row + m;
    const int64_t s = g / seg_rows, q = g - s * seg_rows;
    if (q >= hdr[2 * s]) continue;
    float acc[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[i] = 0.f;
    for (int j = 0; j < slots; ++j) {
      const int r = __ldg(pos + m * slots + j);
      if (r < 0) continue;
      const V v = *reinterpret_cast<const V*>(src + (int64_t)r * n + c);
#pragma unroll
      for (int i = 0; i < VEC; ++i) acc[i] += to_f32(v.v[i]);
    }
    VO o;
#pragma unroll
    for (int i = 0; i < VEC; ++i) o.v[i] = from_f32<TOut>(acc[i] * scale);
    TOut* out = reinterpret_cast<TOut*>(seg_ptrs[s]);
    *reinterpret_cast<VO*>(out + (hdr[2 * s + 1] + q) * (int64_t)n + c) = o;
  }
}

template <typename T, typename TOut>
int launch_gather_sum_to_peers(const void* src, const int32_t* pos, int64_t num_tokens, int slots,
                               int n, float scale, int64_t seg_rows, const int64_t* seg_ptrs,
                               const int32_t* hdr, int64_t first_row, cudaStream_t st) {
  constexpr int VEC = 16 / (sizeof(T) > sizeof(TOut) ? sizeof(T) : sizeof(TOut));
  const int64_t total = num_tokens * (n / VEC);
  if (total == 0) return BOLT_OK;
  int64_t blocks = (total + 255) / 256;
  const int64_t cap = (int64_t)sm_count_of_current_device() * 32;
  if (blocks > cap) blocks = cap;
  k_gather_sum_to_peers<T, TOut, VEC><<<(unsigned)blocks, 256, 0, st>>>(
      static_cast<const T*>(src), pos, num_tokens, slots, n, scale, seg_rows, seg_ptrs, hdr, first_row);
  BOLT_LAUNCH_CHECK();
  return BOLT_OK;
}

template <typename T, typename TOut>
int launch_gather_sum(const void* src, const int32_t* pos, void* out, int64_t num_tokens,
                      int slots, int n, float scale, cudaStream_t st) {
  constexpr int VEC = 16 / (sizeof(T) > sizeof(TOut) ? sizeof(T) : sizeof(TOut));
  const bool vec_ok = (n % VEC == 0) && (reinterpret_cast<uintptr_t>(src) % 16 == 0) &&
                      (reinterpret_cast<uintptr_t>(out) % 16 == 0);
  const int64_t total = vec_ok ? num_tokens * (n / VEC) : num_tokens * n;
  if (total == 0) return BOLT_OK;
  int64_t blocks = (total + 255) / 256;
  const int64_t cap = (int64_t)sm_count_of_current_device() * 32;
  if (blocks > cap) blocks = cap;
  if (vec_ok)
    k_gather_sum<T, TOut, VEC><<<(unsigned)blocks, 256, 0, st>>>(
        static_cast<const T*>(src), pos, static_cast<TOut*>(out), num_tokens, slots, n, scale);
  else
    k_gather_sum<T, TOut, 1><<<(unsigned)blocks, 256, 0, st>>>(
        static_cast<const T*>(src), pos, static_cast<TOut*>(out), num_tokens, slots, n, scale);
  BOLT_LAUNCH_CHECK();
  return BOLT_OK;
}

template <typename T>
int dispatch_gather_out(const void* src, const int32_t* pos, void* out, int out_dtype,
                        int64_t num_tokens, int slots, int n, float scale, cudaStream_t st) {
  switch (out_dtype) {
    case BOLT_BF16:
      return launch_gather_sum<T, __nv_bfloat16>(src, pos, out, num_tokens, slots, n, scale, st);
    case BOLT_F16: return launch_gather_sum<T, __half>(src, pos, out, num_tokens, slots, n, scale, st);
    case BOLT_F32: return launch_gather_sum<T, float>(src, pos, out, num_tokens, slots, n, scale, st);
    default: set_error("gather_sum: unsupported output dtype %d", out_dtype); return BOLT_ERR_INVALID;
  }
}

template <typename TIn, typename TOut>
int launch_sum(const void* in, void* out, int64_t num_tokens, int topk, int n, float scale,
               const float* weights, cudaStream_t st) {
  constexpr int VEC = 16 / (sizeof(TIn) > sizeof(TOut) ? sizeof(TIn) : sizeof(TOut));
  const bool vec_ok = (n % VEC == 0) && (reinterpret_cast<uintptr_t>(in) % 16 == 0) &&
                      (reinterpret_cast<uintptr_t>(out) % 16 == 0);
  const int64_t total = vec_ok ? num_tokens * (n / VEC) : num_tokens * n;
  if (total == 0) return BOLT_OK;
  int64_t blocks = (total + 255) / 256;
  const int64_t cap = (int64_t)sm_count_of_current_device() * 32;
  if (blocks > cap) blocks = cap;
  if (vec_ok)
    k_moe_sum<TIn, TOut, VEC><<<(unsigned)blocks, 256, 0, st>>>(
        static_cast<const TIn*>(in), static_cast<TOut*>(out), num_tokens, topk, n, scale, weights);
  else
    k_moe_sum<TIn, TOut, 1><<<(unsigned)blocks, 256, 0, st>>>(
        static_cast<const TIn*>(in), static_cast<TOut*>(out), num_tokens, topk, n, scale, weights);
  BOLT_LAUNCH_CHECK();
  return BOLT_OK;
}

template <typename TIn>
int dispatch_out(const void* in, void* out, int out_dtype, int64_t num_tokens, int topk, int n,
                 float scale, const float* weights, cudaStream_t st) {
  switch (out_dtype) {
    case BOLT_BF16:
      return launch_sum<TIn, __nv_bfloat16>(in, out, num_tokens, topk, n, scale, weights, st);
    case BOLT_F16: return launch_sum<TIn, __half>(in, out, num_tokens, topk, n, scale, weights, st);
    case BOLT_F32: return launch_sum<TIn, float>(in, out, num_tokens, topk, n, scale, weights, st);
    default: set_error("moe_sum: unsupported output dtype %d", out_dtype); return BOLT_ERR_INVALID;
  }
}

}  // namespace
}  // namespace bolt

extern "C" int bolt_moe_sum(const void* in, int in_dtype, void* out, int out_dtype,
                            int64_t num_tokens, int topk, int n, float scale, const float* weights,
                            void* stream) {
  using namespace bolt;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  BOLT_REQUIRE(num_tokens >= 0 && topk > 0 && n > 0, "moe_sum: bad shape");
  BOLT_REQUIRE(num_tokens == 0 || (in && out), "moe_sum: null pointer");
  switch (in_dtype) {
    case BOLT_BF16:
      return dispatch_out<__nv_bfloat16>(in, out, out_dtype, num_tokens, topk, n, scale, weights, st);
    case BOLT_F16:
      return dispatch_out<__half>(in, out, out_dtype, num_tokens, topk, n, scale, weights, st);
    case BOLT_F32:
      return dispatch_out<float>(in, out, out_dtype, num_tokens, topk, n, scale, weights, st);
    default: set_error("moe_sum: unsupported input dtype %d", in_dtype); return BOLT_ERR_INVALID;
  }
}

extern "C" int bolt_moe_gather_sum(const void* src, int dtype, const int32_t* pos, void* out,
                                   int out_dtype, int64_t num_tokens, int slots, int n, float scale,
                                   void* stream) {
  using namespace bolt;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  BOLT_REQUIRE(num_tokens >= 0 && slots > 0 && n > 0, "gather_sum: bad shape");
  BOLT_REQUIRE(num_tokens == 0 || (pos && out), "gather_sum: null pointer");
  switch (dtype) {
    case BOLT_BF16:
      return dispatch_gather_out<__nv_bfloat16>(src, pos, out, out_dtype, num_tokens, slots, n, scale, st);
    case BOLT_F16:
      return dispatch_gather_out<__half>(src, pos, out, out_dtype, num_tokens, slots, n, scale, st);
    case BOLT_F32:
      return dispatch_gather_out<float>(src, pos, out, out_dtype, num_tokens, slots, n, scale, st);
    default: set_error("gather_sum: unsupported dtype %d", dtype); return BOLT_ERR_INVALID;
  }
}

extern "C" int bolt_moe_gather_sum_to_peers(const void* src, int dtype, const int32_t* pos,
                                            int64_t num_tokens, int slots, int n, float scale,
                                            int64_t seg_rows, const int64_t* seg_ptrs,
                                            const int32_t* hdr, int64_t first_row, void* stream) {
  using namespace bolt;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  BOLT_REQUIRE(num_tokens >= 0 && slots > 0 && n > 0 && seg_rows > 0 && first_row >= 0,
               "gather_sum_to_peers: bad shape");
  BOLT_REQUIRE(num_tokens == 0 || (src && pos && seg_ptrs && hdr), "gather_sum_to_peers: null pointer");
  BOLT_REQUIRE(reinterpret_cast<uintptr_t>(src) % 16 == 0, "gather_sum_to_peers: src must be 16-byte aligned");
  switch (dtype) {
    case BOLT_BF16:
      BOLT_REQUIRE(n % 8 == 0, "gather_sum_to_peers: n must be a multiple of 8");
      return launch_gather_sum_to_peers<__nv_bfloat16, __nv_bfloat16>(
          src, pos, num_tokens, slots, n, scale, seg_rows, seg_ptrs, hdr, first_row, st);
    case BOLT_F16:
      BOLT_REQUIRE(n % 8 == 0, "gather_sum_to_peers: n must be a multiple of 8");
      return launch_gather_sum_to_peers<__half, __half>(src, pos, num_tokens, slots, n, scale,
                                                        seg_rows, seg_ptrs, hdr, first_row, st);
    case BOLT_F32:
      BOLT_REQUIRE(n % 4 == 0, "gather_sum_to_peers: n must be a multiple of 4");
      return launch_gather_sum_to_peers<float, float>(src, pos, num_tokens, slots, n, scale, seg_rows,
                                                      seg_ptrs, hdr, first_row, st);
    default: set_error("gather_sum_to_peers: unsupported dtype %d", dtype); return BOLT_ERR_INVALID;
  }
}
