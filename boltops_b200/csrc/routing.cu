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

// Grouped gate (DeepSeek-V3 style): scores = sigmoid(logits), choice = scores + bias;
// group score = sum of a group's two largest choices; keep the topk_group best groups;
// top-k experts by choice inside the kept groups; weights = unbiased scores, renormalised.
// With one fused shared expert the last slot becomes expert id `experts` with weight
// sum(others) / routed_scaling_factor, and the normalisation excludes it.
template <typename T>
__global__ void __launch_bounds__(256) k_fused_gate(const T* __restrict__ logits,
                                                    const float* __restrict__ bias, int64_t tokens,
                                                    int experts, int num_groups, int topk_group,
                                                    int topk, int shared, float routed_scale,
                                                    float* __restrict__ weights,
                                                    int32_t* __restrict__ ids) {
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int per_lane = (experts + 31) / 32;
  const int per_group = experts / num_groups;
  for (int64_t m = warp0; m < tokens; m += nwarps) {
    const T* row = logits + m * experts;
    float score[kMaxPerLane], choice[kMaxPerLane];
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) {
      const int e = lane + 32 * j;
      if (j < per_lane && e < experts) {
        score[j] = 1.0f / (1.0f + expf(-to_f32(row[e])));
        choice[j] = score[j] + bias[e];
      } else {
        score[j] = 0.f;
        choice[j] = -FLT_MAX;
      }
    }
    // group scores: lane g ends up holding the score of group g (num_groups <= 32)
    float my_group_score = -FLT_MAX;
    for (int g = 0; g < num_groups; ++g) {
      float top1 = -FLT_MAX, top2 = -FLT_MAX;
#pragma unroll
      for (int j = 0; j < kMaxPerLane; ++j) {
        const int e = lane + 32 * j;
        if (j < per_lane && e < experts && e / per_group == g) {
          const float c = choice[j];
          if (c > top1) { top2 = top1; top1 = c; } else if (c > top2) { top2 = c; }
        }
      }
      for (int o = 16; o > 0; o >>= 1) {
        const float o1 = __shfl_xor_sync(0xffffffffu, top1, o);
        const float o2 = __shfl_xor_sync(0xffffffffu, top2, o);
        const float hi = fmaxf(top1, o1);
        const float lo = fmaxf(fminf(top1, o1), fmaxf(top2, o2));
        top1 = hi;
        top2 = lo;
      }
      if (lane == g) my_group_score = top1 + top2;
    }
    // keep the topk_group best groups (ties: lowest group index)
    unsigned keep = 0;
    float gs = (lane < num_groups) ? my_group_score : -FLT_MAX;
    for (int r = 0; r < topk_group; ++r) {
      float best = gs;
      int best_g = lane;
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int og = __shfl_xor_sync(0xffffffffu, best_g, o);
        if (ob > best || (ob == best && og < best_g)) { best = ob; best_g = og; }
      }
      keep |= 1u << best_g;
      if (lane == best_g) gs = -FLT_MAX;
    }
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) {
      const int e = lane + 32 * j;
      if (!(j < per_lane && e < experts) || !((keep >> (e / per_group)) & 1u)) choice[j] = -FLT_MAX;
    }
    // top-k by choice, descending; weights are the unbiased scores
    float my_w = 0.f;
    int my_id = 0;
    float total = 0.f;
    const int routed = shared ? topk - 1 : topk;
    for (int k = 0; k < routed; ++k) {
      float best = -FLT_MAX, best_s = 0.f;
      int best_e = 0x7fffffff;
#pragma unroll
      for (int j = 0; j < kMaxPerLane; ++j) {
        const int e = lane + 32 * j;
        if (choice[j] > best) { best = choice[j]; best_e = e; best_s = score[j]; }
      }
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const float os = __shfl_xor_sync(0xffffffffu, best_s, o);
        const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
        if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; best_s = os; }
      }
      if ((best_e & 31) == lane) {
#pragma unroll
        for (int j = 0; j < kMaxPerLane; ++j)
          if (lane + 32 * j == best_e) choice[j] = -FLT_MAX;
      }
      if (lane == k) { my_w = best_s; my_id = best_e; }
      total += best_s;
    }
    if (shared && lane == topk - 1) {
      my_w = total / routed_scale;
      my_id = experts;
    }
    if (lane < topk) {
      weights[m * topk + lane] = my_w / total;
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

// ---------------------------------------------------------------------------
// Expert-parallel dispatch: which ranks does a token go to?
// ---------------------------------------------------------------------------
// One thread per token: ranks hit by any of its top-k experts as a bit mask, written out as
// routes[token][r] = r (hit) or -1 (not hit).  Fed to the stable sort with ranks as
// "experts", this gives the (rank, token)-ordered send list, the per-rank counts and the
// position of every (token, rank) pair in one go.
__global__ void __launch_bounds__(256) k_dest_ranks(const int32_t* __restrict__ topk_ids,
                                                    int64_t num_tokens, int topk, int num_experts,
                                                    int experts_per_rank, int world,
                                                    int64_t chunk_tokens,
                                                    int32_t* __restrict__ routes) {
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < num_tokens;
       t += (int64_t)gridDim.x * blockDim.x) {
    // with token chunks the sort key is (chunk, rank): chunk-major send order
    const int base = chunk_tokens > 0 ? (int)(t / chunk_tokens) * world : 0;
    unsigned long long mask[4] = {0ull, 0ull, 0ull, 0ull};
    for (int k = 0; k < topk; ++k) {
      const int e = topk_ids[t * topk + k];
      if (e >= 0 && e < num_experts) {
        const int r = e / experts_per_rank;
        mask[r >> 6] |= 1ull << (r & 63);
      }
    }
    for (int r = 0; r < world; ++r)
      routes[t * world + r] = ((mask[r >> 6] >> (r & 63)) & 1ull) ? base + r : -1;
  }
}

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

extern "C" int bolt_moe_fused_gate(const void* gating, int dtype, const float* bias,
                                   int64_t num_tokens, int num_experts, int num_expert_group,
                                   int topk_group, int topk, int num_fused_shared_experts,
                                   float routed_scaling_factor, float* topk_weights,
                                   int32_t* topk_ids, void* stream) {
  using namespace bolt;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  BOLT_REQUIRE(num_tokens >= 0 && num_experts > 0 && num_experts <= 32 * kMaxPerLane,
               "fused_gate: bad shape");
  BOLT_REQUIRE(num_expert_group > 0 && num_expert_group <= 32 &&
                   num_experts % num_expert_group == 0 && num_experts / num_expert_group >= 2,
               "fused_gate: bad expert grouping");
  BOLT_REQUIRE(topk_group > 0 && topk_group <= num_expert_group, "fused_gate: bad topk_group");
  BOLT_REQUIRE(num_fused_shared_experts == 0 || num_fused_shared_experts == 1,
               "fused_gate: at most one fused shared expert");
  BOLT_REQUIRE(topk > num_fused_shared_experts && topk <= 32 &&
                   topk - num_fused_shared_experts <= topk_group * (num_experts / num_expert_group),
               "fused_gate: topk %d out of range", topk);
  BOLT_REQUIRE(num_tokens == 0 || (gating && bias && topk_weights && topk_ids),
               "fused_gate: null pointer");
  if (num_tokens == 0) return BOLT_OK;
  int64_t blocks = (num_tokens + 7) / 8;
  const int64_t cap = (int64_t)sm_count_of_current_device() * 16;
  if (blocks > cap) blocks = cap;
#define BOLT_GATE_LAUNCH(T)                                                                    \
  k_fused_gate<T><<<(unsigned)blocks, 256, 0, st>>>(                                          \
      static_cast<const T*>(gating), bias, num_tokens, num_experts, num_expert_group,          \
      topk_group, topk, num_fused_shared_experts, routed_scaling_factor, topk_weights, topk_ids)
  switch (dtype) {
    case BOLT_F32: BOLT_GATE_LAUNCH(float); break;
    case BOLT_BF16: BOLT_GATE_LAUNCH(__nv_bfloat16); break;
    case BOLT_F16: BOLT_GATE_LAUNCH(__half); break;
    default: set_error("fused_gate: unsupported dtype %d", dtype); return BOLT_ERR_INVALID;
  }
#undef BOLT_GATE_LAUNCH
  BOLT_LAUNCH_CHECK();
  return BOLT_OK;
}

extern "C" int bolt_ep_dest_ranks(const int32_t* topk_ids, int64_t num_tokens, int topk,
                                  int num_experts, int experts_per_rank, int world,
                                  int64_t chunk_tokens, int32_t* routes, void* stream) {
  using namespace bolt;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  BOLT_REQUIRE(num_tokens >= 0 && topk > 0 && num_experts > 0 && experts_per_rank > 0,
               "ep_dest_ranks: bad shape");
  BOLT_REQUIRE(world > 0 && world <= 255 &&
                   (int64_t)world * experts_per_rank >= num_experts,
               "ep_dest_ranks: world %d x %d experts per rank does not cover %d experts (max 255 ranks)",
               world, experts_per_rank, num_experts);
  BOLT_REQUIRE(num_tokens == 0 || (topk_ids && routes), "ep_dest_ranks: null pointer");
  if (num_tokens == 0) return BOLT_OK;
  int64_t blocks = (num_tokens + 255) / 256;
  const int64_t cap = (int64_t)sm_count_of_current_device() * 8;
  if (blocks > cap) blocks = cap;
  BOLT_REQUIRE(chunk_tokens >= 0, "ep_dest_ranks: negative chunk size");
  k_dest_ranks<<<(unsigned)blocks, 256, 0, st>>>(topk_ids, num_tokens, topk, num_experts,
                                                 experts_per_rank, world, chunk_tokens, routes);
  BOLT_LAUNCH_CHECK();
  return BOLT_OK;
}

namespace bolt {
namespace {
// One warp per wire row: [row data | scales | top-k ids | top-k weights], every part padded to 16
// bytes, row i taken from token send_ids[first + i] & 0xFFFFFF.
__global__ void __launch_bounds__(256) k_ep_pack_rows(
    const uint4* __restrict__ data, int data_vecs, const float* __restrict__ scales, int groups,
    const int32_t* __restrict__ ids, const float* __restrict__ wts, int topk,
    const int32_t* __restrict__ send_ids, int64_t first, int64_t rows, uint8_t* __restrict__ out,
    int64_t out_stride) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int sc_bytes = (groups * 4 + 15) & ~15, k_bytes = (topk * 4 + 15) & ~15;
  for (int64_t i = warp; i < rows; i += warps) {
    const int64_t t = send_ids[first + i] & 0xFFFFFF;
    uint8_t* o = out + i * out_stride;
    const uint4* src = data + t * data_vecs;
    for (int v = lane; v < data_vecs; v += 32) reinterpret_cast<uint4*>(o)[v] = __ldg(src + v);
    o += (int64_t)data_vecs * 16;
    for (int g = lane; g < groups; g += 32) reinterpret_cast<float*>(o)[g] = scales[t * groups + g];
    o += sc_bytes;
    for (int k = lane; k < topk; k += 32) {
      reinterpret_cast<int32_t*>(o)[k] = ids[t * topk + k];
      reinterpret_cast<float*>(o + k_bytes)[k] = wts[t * topk + k];
    }
  }
}
}  // namespace
}  // namespace bolt

extern "C" int64_t bolt_ep_wire_row_bytes(int row_bytes, int groups, int topk) {
  return (int64_t)((row_bytes + 15) & ~15) + ((groups * 4 + 15) & ~15) + 2 * ((topk * 4 + 15) & ~15);
}

extern "C" int bolt_ep_pack_rows(const void* data, int row_bytes, const float* scales, int groups,
                                 const int32_t* topk_ids, const float* topk_weights, int topk,
                                 const int32_t* send_ids, int64_t first, int64_t rows, void* out,
                                 int64_t out_stride, void* stream) {
  using namespace bolt;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  BOLT_REQUIRE(row_bytes > 0 && row_bytes % 16 == 0, "ep_pack: row_bytes must be a multiple of 16");
  BOLT_REQUIRE(groups >= 0 && topk > 0 && rows >= 0 && first >= 0, "ep_pack: bad sizes");
  BOLT_REQUIRE(out_stride >= bolt_ep_wire_row_bytes(row_bytes, groups, topk) && out_stride % 16 == 0,
               "ep_pack: output row stride too small");
  if (rows == 0) return BOLT_OK;
  BOLT_REQUIRE(data && topk_ids && topk_weights && send_ids && out && (groups == 0 || scales),
               "ep_pack: null pointer");
  BOLT_REQUIRE((reinterpret_cast<uintptr_t>(data) | reinterpret_cast<uintptr_t>(out)) % 16 == 0,
               "ep_pack: buffers must be 16-byte aligned");
  int64_t blocks = (rows + 7) / 8;
  const int64_t cap = (int64_t)sm_count_of_current_device() * 16;
  if (blocks > cap) blocks = cap;
  k_ep_pack_rows<<<(unsigned)blocks, 256, 0, st>>>(
      static_cast<const uint4*>(data), row_bytes / 16, scales, groups, topk_ids, topk_weights, topk,
      send_ids, first, rows, static_cast<uint8_t*>(out), out_stride);
  BOLT_LAUNCH_CHECK();
  return BOLT_OK;
}


// ---------------------------------------------------------------------------
// Direct exchange over peer memory (expert parallelism without a collective library call on the
// data path).  Every rank owns one exchange buffer with the same layout, mapped into all ranks
// (peer pointers in a device table):
//   [ header: per source rank {rows, first return row} ][ flags ][ receive region: world segments
//     of seg_rows wire rows ][ return region: partial output rows in the owner's send order ]
// A sender writes its wire rows for rank d into segment `me` of d's receive region with plain
// 16-byte stores and leaves {rows, first return row} in d's header; the owner of the experts
// later writes a token's partial output row straight into the sender's return region
// (k_gather_sum_to_peers, moe_sum.cu).  Nothing here waits; ranks meet in k_ep_barrier.
namespace bolt {
namespace {

constexpr int kMaxWorld = 64;

// One warp per wire row, rows in send order (rank-major); segment boundaries from the per-rank
// counts of the dispatch sort.
__global__ void __launch_bounds__(256) k_ep_dispatch(
    const uint4* __restrict__ data, int data_vecs, const float* __restrict__ scales, int groups,
    const int32_t* __restrict__ ids, const float* __restrict__ wts, int topk,
    const int32_t* __restrict__ send_ids, const int32_t* __restrict__ counts, int world, int me,
    int64_t seg_rows, const int64_t* __restrict__ peers, int64_t hdr_off, int64_t recv_off,
    int64_t wire_bytes, int32_t* __restrict__ status) {
  __shared__ int starts[kMaxWorld + 1];
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int d = 0; d < world; ++d) {
      starts[d] = acc;
      const int c = counts[d];
      acc += c < 0 ? 0 : (c > seg_rows ? (int)seg_rows : c);
      if ((c < 0 || c > seg_rows) && status != nullptr) atomicCAS(status, 0, 21);
    }
    starts[world] = acc;
  }
  __syncthreads();
  if (blockIdx.x == 0 && threadIdx.x < world) {
    const int d = threadIdx.x;
    int32_t* hdr = reinterpret_cast<int32_t*>(peers[d] + hdr_off) + 2 * me;
    hdr[0] = starts[d + 1] - starts[d];
    hdr[1] = starts[d];
  }
  const int lane = threadIdx.x & 31;
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int sc_bytes = (groups * 4 + 15) & ~15, k_bytes = (topk * 4 + 15) & ~15;
  const int64_t rows = starts[world];
  for (int64_t i = warp; i < rows; i += warps) {
    int d = 0;
    while (d + 1 < world && i >= starts[d + 1]) ++d;
    const int64_t q = i - starts[d];
    const int64_t t = send_ids[i] & 0xFFFFFF;
    uint8_t* o = reinterpret_cast<uint8_t*>(peers[d] + recv_off) + ((int64_t)me * seg_rows + q) * wire_bytes;
    const uint4* src = data + t * data_vecs;
    for (int v = lane; v < data_vecs; v += 32) reinterpret_cast<uint4*>(o)[v] = __ldg(src + v);
    o += (int64_t)data_vecs * 16;
    for (int g = lane; g < groups; g += 32) reinterpret_cast<float*>(o)[g] = scales[t * groups + g];
    o += sc_bytes;
    for (int k = lane; k < topk; k += 32) {
      reinterpret_cast<int32_t*>(o)[k] = ids[t * topk + k];
      reinterpret_cast<float*>(o + k_bytes)[k] = wts[t * topk + k];
    }
    // a wire row with 16 bytes to spare also carries the token's index on this rank (for
    // results that come back per route, addressed by token)
    if (lane == 0 && wire_bytes >= (int64_t)data_vecs * 16 + sc_bytes + 2 * k_bytes + 16)
      *reinterpret_cast<int32_t*>(o + 2 * k_bytes) = (int32_t)t;
  }
}

// Receiver: dense top-k ids / weights of all segment rows; rows a segment does not hold get id -1
// (no expert) so that the local layer ignores them.
__global__ void __launch_bounds__(256) k_ep_unpack_routes(
    const uint8_t* __restrict__ recv, int64_t wire_bytes, int64_t ids_off, int64_t wts_off, int topk,
    int64_t seg_rows, int nseg, const int32_t* __restrict__ hdr, int32_t* __restrict__ ids,
    float* __restrict__ wts, int64_t src_off, int32_t* __restrict__ src) {
  const int64_t total = (int64_t)nseg * seg_rows * topk;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / topk;
    const int k = (int)(i - row * topk);
    const int64_t s = row / seg_rows, q = row - s * seg_rows;
    const bool live = q < hdr[2 * s];
    const uint8_t* r = recv + row * wire_bytes;
    ids[i] = live ? reinterpret_cast<const int32_t*>(r + ids_off)[k] : -1;
    wts[i] = live ? reinterpret_cast<const float*>(r + wts_off)[k] : 0.f;
    if (src != nullptr && k == 0) src[row] = live ? *reinterpret_cast<const int32_t*>(r + src_off) : 0;
  }
}

// All ranks meet: thread r tells rank r "rank `me` has reached epoch n" (a flag in r's buffer) and
// waits until rank r has said the same here.  The epoch is a counter in this rank's own buffer
// (slot `world` behind the flags) that the kernel advances itself, so a step carries no host-side
// state and can be replayed.  Kernels before this launch are complete (stream order), so their
// peer stores are performed before the flag is written; the fences order the flag against them
// at system scope.  The wait is bounded (~1 s): on expiry the status word is set and the kernel
// returns.
__global__ void k_ep_barrier(const int64_t* __restrict__ peers, int world, int me, int64_t flag_off,
                             int32_t* __restrict__ status) {
  __shared__ int epoch_s;
  if (threadIdx.x == 0) {
    int32_t* counter = reinterpret_cast<int32_t*>(peers[me] + flag_off) + world;
    epoch_s = *counter + 1;
    *counter = epoch_s;
  }
  __syncthreads();
  const int epoch = epoch_s;
  const int r = threadIdx.x;
  if (r >= world) return;
  __threadfence_system();
  volatile int32_t* theirs = reinterpret_cast<volatile int32_t*>(peers[r] + flag_off) + me;
  *theirs = epoch;
  __threadfence_system();
  volatile int32_t* mine = reinterpret_cast<volatile int32_t*>(peers[me] + flag_off) + r;
  const long long t0 = clock64();
  while (*mine - epoch < 0) {
    if (clock64() - t0 > 2000000000ll) {
      if (status != nullptr) atomicCAS(status, 0, 20);
      break;
    }
    __nanosleep(100);
  }
  __threadfence_system();
}

}  // namespace
}  // namespace bolt

extern "C" int bolt_ep_dispatch_rows(const void* data, int row_bytes, const float* scales, int groups,
                                     const int32_t* topk_ids, const float* topk_weights, int topk,
                                     const int32_t* send_ids, const int32_t* counts, int world,
                                     int me, int64_t max_rows, int64_t seg_rows,
                                     const int64_t* peers, int64_t hdr_off, int64_t recv_off,
                                     int64_t wire_bytes, int32_t* status, void* stream) {
  using namespace bolt;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  BOLT_REQUIRE(row_bytes > 0 && row_bytes % 16 == 0, "ep_dispatch: row_bytes must be a multiple of 16");
  BOLT_REQUIRE(groups >= 0 && topk > 0 && max_rows >= 0 && seg_rows > 0, "ep_dispatch: bad sizes");
  BOLT_REQUIRE(world > 0 && world <= kMaxWorld && me >= 0 && me < world, "ep_dispatch: bad rank");
  BOLT_REQUIRE(wire_bytes >= bolt_ep_wire_row_bytes(row_bytes, groups, topk) && wire_bytes % 16 == 0,
               "ep_dispatch: wire row too small");
  BOLT_REQUIRE(hdr_off % 16 == 0 && recv_off % 16 == 0, "ep_dispatch: regions must be 16-byte aligned");
  BOLT_REQUIRE(data && topk_ids && topk_weights && send_ids && counts && peers && (groups == 0 || scales),
               "ep_dispatch: null pointer");
  BOLT_REQUIRE(reinterpret_cast<uintptr_t>(data) % 16 == 0, "ep_dispatch: data must be 16-byte aligned");
  int64_t blocks = (max_rows + 7) / 8;
  const int64_t cap = (int64_t)sm_count_of_current_device() * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  k_ep_dispatch<<<(unsigned)blocks, 256, 0, st>>>(
      static_cast<const uint4*>(data), row_bytes / 16, scales, groups, topk_ids, topk_weights, topk,
      send_ids, counts, world, me, seg_rows, peers, hdr_off, recv_off, wire_bytes, status);
  BOLT_LAUNCH_CHECK();
  return BOLT_OK;
}

extern "C" int bolt_ep_unpack_routes(const void* recv, int64_t wire_bytes, int64_t ids_off,
                                     int64_t wts_off, int topk, int64_t seg_rows, int nseg,
                                     const int32_t* hdr, int32_t* topk_ids, float* topk_weights,
                                     int64_t src_off, int32_t* src_tokens, void* stream) {
  using namespace bolt;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  BOLT_REQUIRE(recv && hdr && topk_ids && topk_weights, "ep_unpack: null pointer");
  BOLT_REQUIRE(topk > 0 && seg_rows > 0 && nseg > 0 && wire_bytes % 4 == 0 && ids_off % 4 == 0 &&
                   wts_off % 4 == 0,
               "ep_unpack: bad layout");
  BOLT_REQUIRE(src_tokens == nullptr || (src_off % 4 == 0 && src_off + 4 <= wire_bytes),
               "ep_unpack: bad offset of the source token index");
  const int64_t total = (int64_t)nseg * seg_rows * topk;
  int64_t blocks = (total + 255) / 256;
  const int64_t cap = (int64_t)sm_count_of_current_device() * 16;
  if (blocks > cap) blocks = cap;
  k_ep_unpack_routes<<<(unsigned)blocks, 256, 0, st>>>(static_cast<const uint8_t*>(recv), wire_bytes,
                                                       ids_off, wts_off, topk, seg_rows, nseg, hdr,
                                                       topk_ids, topk_weights, src_off, src_tokens);
  BOLT_LAUNCH_CHECK();
  return BOLT_OK;
}

extern "C" int bolt_ep_barrier(const int64_t* peers, int world, int me, int64_t flag_off,
                               int32_t* status, void* stream) {
  using namespace bolt;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  BOLT_REQUIRE(peers != nullptr && world > 0 && world <= kMaxWorld && me >= 0 && me < world &&
                   flag_off % 4 == 0,
               "ep_barrier: bad arguments");
  k_ep_barrier<<<1, kMaxWorld, 0, st>>>(peers, world, me, flag_off, status);
  BOLT_LAUNCH_CHECK();
  return BOLT_OK;
}
