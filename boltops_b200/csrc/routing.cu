// Router front-end: softmax (or sigmoid) over the expert logits of a token, top-k
// selection, optional renormalisation.  One warp per token, logits held in registers;
// HBM-bound (reads M*E logits once, writes 8*topk bytes per token).
#include <float.h>

#include "common.cuh"

namespace bolt {
namespace {

constexpr int kMaxPerLane = 32;  // experts per lane -> up to 1024 experts

template <typename T>
__global__ void __launch_bounds__(256) k_fused_topk(const T* __restrict__ logits, int64_t tokens,
                                                    int experts, int topk, int renormalize,
                                                    int softmax, float* __restrict__ weights,
                                                    int32_t* __restrict__ ids) {
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int per_lane = (experts + 31) / 32;
  for (int64_t m = warp0; m < tokens; m += nwarps) {
    const T* row = logits + m * experts;
    float v[kMaxPerLane];
    float mx = -FLT_MAX;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) {
      const int e = lane + 32 * j;
      v[j] = (j < per_lane && e < experts) ? to_f32(row[e]) : -FLT_MAX;
      mx = fmaxf(mx, v[j]);
    }
    if (softmax) {
      for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      float sum = 0.f;
#pragma unroll
      for (int j = 0; j < kMaxPerLane; ++j) {
        const int e = lane + 32 * j;
        if (j < per_lane && e < experts) {
          v[j] = expf(v[j] - mx);
          sum += v[j];
        } else {
          v[j] = -1.f;  // below every probability
        }
      }
      for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      const float inv = 1.0f / sum;
#pragma unroll
      for (int j = 0; j < kMaxPerLane; ++j)
        if (v[j] >= 0.f) v[j] *= inv;
    } else {
#pragma unroll
      for (int j = 0; j < kMaxPerLane; ++j) {
        const int e = lane + 32 * j;
        v[j] = (j < per_lane && e < experts) ? 1.0f / (1.0f + expf(-v[j])) : -1.f;
      }
    }
    // top-k by repeated warp arg-max (ties: lowest expert index)
    float my_w = 0.f;
    int my_id = 0;
    float total = 0.f;
    for (int k = 0; k < topk; ++k) {
      float best = -2.f;
      int best_e = 0x7fffffff;
#pragma unroll
      for (int j = 0; j < kMaxPerLane; ++j) {
        const int e = lane + 32 * j;
        if (v[j] > best) { best = v[j]; best_e = e; }
      }
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
        if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
      }
      if ((best_e & 31) == lane) {
#pragma unroll
        for (int j = 0; j < kMaxPerLane; ++j)
          if (lane + 32 * j == best_e) v[j] = -3.f;  // taken
      }
      if (lane == k) { my_w = best; my_id = best_e; }
      total += best;
    }
    if (lane < topk) {
      weights[m * topk + lane] = renormalize ? my_w / total : my_w;
      ids[m * topk + lane] = my_id;
    }
  }
}

template <typename T>
int launch_topk(const void* logits, int64_t tokens, int experts, int topk, int renormalize,
                int softmax, float* weights, int32_t* ids, cudaStream_t st) {
  if (tokens == 0) return BOLT_OK;
  int64_t blocks = (tokens + 7) / 8;
  const int64_t cap = (int64_t)sm_count_of_current_device() * 16;
  if (blocks > cap) blocks = cap;
  k_fused_topk<T><<<(unsigned)blocks, 256, 0, st>>>(static_cast<const T*>(logits), tokens, experts,
                                                    topk, renormalize, softmax, weights, ids);
  BOLT_LAUNCH_CHECK();
  return BOLT_OK;
}

}  // namespace
}  // namespace bolt

extern "C" int bolt_fused_topk(const void* gating, int dtype, int64_t num_tokens, int num_experts,
                               int topk, int renormalize, int is_softmax, float* topk_weights,
                               int32_t* topk_ids, void* stream) {
  using namespace bolt;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  BOLT_REQUIRE(num_tokens >= 0 && num_experts > 0, "fused_topk: bad shape");
  BOLT_REQUIRE(num_experts <= 32 * kMaxPerLane, "fused_topk: at most %d experts", 32 * kMaxPerLane);
  BOLT_REQUIRE(topk > 0 && topk <= 32 && topk <= num_experts, "fused_topk: topk %d out of range", topk);
  BOLT_REQUIRE(num_tokens == 0 || (gating && topk_weights && topk_ids), "fused_topk: null pointer");
  switch (dtype) {
    case BOLT_F32:
      return launch_topk<float>(gating, num_tokens, num_experts, topk, renormalize, is_softmax,
                                topk_weights, topk_ids, st);
    case BOLT_BF16:
      return launch_topk<__nv_bfloat16>(gating, num_tokens, num_experts, topk, renormalize,
                                        is_softmax, topk_weights, topk_ids, st);
    case BOLT_F16:
      return launch_topk<__half>(gating, num_tokens, num_experts, topk, renormalize, is_softmax,
                                 topk_weights, topk_ids, st);
    default: set_error("fused_topk: unsupported dtype %d", dtype); return BOLT_ERR_INVALID;
  }
}
