// Token-to-expert sort / pad for the fused-MoE path (CK format and vLLM format).
//
// Contract (bit-exact, deterministic): a stable counting sort of the M*K routes
// by expert id; every expert's segment is padded to `unit`; position inside an
// expert is ascending flat route index -- computed from prefix sums only, never
// from the arrival order of atomics.
//
// Structure: routes are cut into contiguous per-CTA chunks, each CTA's chunk into
// contiguous per-warp sub-chunks.
//   small inputs : one CTA does everything (count -> scan -> metadata -> scatter).
//   large inputs : k_count  (per-CTA histograms to scratch)
//                  k_scan   (one CTA: column scan over CTAs, padded expert prefix,
//                            per-block expert ids, counts/starts, num_valid)
//                  k_scatter(per-warp histograms in shared memory, warp-ordered
//                            match_any ranking, stable scatter, pad fill).
#include <atomic>
#include "common.cuh"

namespace bolt {
namespace {

constexpr int kSortThreads = 512;
constexpr int kSortWarps = kSortThreads / 32;
constexpr int kSmallRoutes = 4096;  // single-CTA path up to this many routes
constexpr int kMaxCtas = 128;

struct SortParams {
  const int32_t* ids;        // [R]
  const float* weights;      // [R] (CK format) or nullptr
  const int32_t* mask;       // [E] or nullptr (CK format)
  const int32_t* expert_map; // [E] or nullptr (vLLM format)
  int32_t* sorted_ids;
  float* sorted_weights;
  int32_t* expert_ids;       // per block
  int32_t* positions;        // [2E] (CK) or nullptr
  int32_t* num_valid;        // [1]
  int32_t* route_pos;        // [R] sorted position of every route, -1 if it has none (optional)
  int32_t* segments;         // optional [*][4]: {expert label, first row, rows, 0} per run of at
                             // most segment_rows live rows of one expert, in sorted order
  int32_t* num_segments;     // [1]
  int segment_rows;
  int32_t* cta_counts;       // scratch [G][E]: counts, then exclusive offsets
  int32_t* expert_start;     // scratch [E+1]: padded start per expert, -1 if none
  int R, E, topk, tokens, unit;
  int chunk;                 // routes per CTA (multiple of 32*kSortWarps)
  int capacity;              // entries of sorted_ids
  int num_blocks;            // entries of expert_ids
  int vllm;                  // 0 = CK format, 1 = vLLM format
};

__device__ __forceinline__ int load_expert(const SortParams& p, int r) {
  if (r >= p.R) return -1;
  int e = p.ids[r];
  return (e >= 0 && e < p.E) ? e : -1;
}

// Histogram of one CTA's chunk into smem cnt[E] (order-free).
__device__ void cta_histogram(const SortParams& p, int cta, int* cnt) {
  for (int e = threadIdx.x; e < p.E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  const int begin = cta * p.chunk;
  const int end = min(begin + p.chunk, p.R);
  for (int r = begin + threadIdx.x; r < end; r += blockDim.x) {
    int e = load_expert(p, r);
    if (e >= 0) atomicAdd(&cnt[e], 1);
  }
  __syncthreads();
}

// Block-wide exclusive scan of one int per thread-slot over `n` items held in smem
// (in place).  n may exceed blockDim; uses a running carry.  scratch: 33 ints.
__device__ void block_exclusive_scan(int* data, int n, int* scratch, int* total_out) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  int carry = 0;
  for (int base = 0; base < n; base += blockDim.x) {
    int i = base + threadIdx.x;
    int v = (i < n) ? data[i] : 0;
    int x = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int y = __shfl_up_sync(0xffffffffu, x, o);
      if (lane >= o) x += y;
    }
    if (lane == 31) scratch[warp] = x;
    __syncthreads();
    if (warp == 0) {
      int w = (lane < nwarps) ? scratch[lane] : 0;
      int s = w;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int y = __shfl_up_sync(0xffffffffu, s, o);
        if (lane >= o) s += y;
      }
      if (lane < nwarps) scratch[lane] = s - w;  // exclusive warp offsets
      if (lane == 31) scratch[32] = s;           // tile total
    }
    __syncthreads();
    if (i < n) data[i] = carry + scratch[warp] + x - v;
    carry += scratch[32];
    __syncthreads();
  }
  if (total_out && threadIdx.x == 0) *total_out = carry;
}

// From per-expert totals in smem `tot[E]` build padded starts + metadata outputs.
// On return start_s[e] = padded start (or -1 if expert e has no segment),
// start_s[E] = padded total.  tmp: E ints, scratch: 33 ints.
__device__ void build_metadata(const SortParams& p, const int* tot, int* start_s, int* tmp,
                               int* scratch, int* seg_s) {
  const int E = p.E;
  // padded sizes
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    bool on = p.vllm || p.mask == nullptr || p.mask[e] != 0;
    int c = tot[e];
    start_s[e] = on ? ((c + p.unit - 1) / p.unit) * p.unit : 0;
    tmp[e] = (!p.vllm && p.mask != nullptr && p.mask[e] != 0) ? 1 : 0;
  }
  __syncthreads();
  __shared__ int total_s;
  // in-place exclusive scan: afterwards padded size of e = start_s[e+1]-start_s[e]
  block_exclusive_scan(start_s, E, scratch, &total_s);
  if (!p.vllm && p.mask != nullptr) block_exclusive_scan(tmp, E, scratch, nullptr);
  __syncthreads();
  const int total = total_s;
  if (threadIdx.x == 0) {
    start_s[E] = total;
    p.num_valid[0] = total;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int s = start_s[e];
    const int nxt = start_s[e + 1];  // still the raw scan value for e+1 (or total)
    bool on = p.vllm || p.mask == nullptr || p.mask[e] != 0;
    int label = e;
    if (!p.vllm && p.mask != nullptr) label = tmp[e];
    if (p.vllm && p.expert_map != nullptr) label = p.expert_map[e];
    for (int b = s / p.unit; b < nxt / p.unit; ++b) p.expert_ids[b] = label;
    if (p.positions != nullptr) {
      p.positions[e] = tot[e];
      p.positions[E + e] = on ? s : -1;
    }
  }
  if (p.segments != nullptr) {
    // runs of at most segment_rows live rows per expert, numbered in expert order
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
      bool on = p.mask == nullptr || p.mask[e] != 0;
      seg_s[e] = on ? (tot[e] + p.segment_rows - 1) / p.segment_rows : 0;
    }
    __syncthreads();
    __shared__ int seg_total_s;
    block_exclusive_scan(seg_s, E, scratch, &seg_total_s);
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
      bool on = p.mask == nullptr || p.mask[e] != 0;
      if (!on) continue;
      const int c = tot[e];
      const int label = (p.mask != nullptr) ? tmp[e] : e;
      int* dst = p.segments + 4 * seg_s[e];
      for (int r = 0; r < c; r += p.segment_rows, dst += 4) {
        dst[0] = label;
        dst[1] = start_s[e] + r;
        dst[2] = min(p.segment_rows, c - r);
        dst[3] = 0;
      }
    }
    if (threadIdx.x == 0) p.num_segments[0] = seg_total_s;
  }
  if (p.vllm) {
    // blocks beyond the padded total hold expert 0 (mapped) as in the zero-filled buffer
    int label0 = (p.expert_map != nullptr) ? p.expert_map[0] : 0;
    for (int b = total / p.unit + threadIdx.x; b < p.num_blocks; b += blockDim.x)
      p.expert_ids[b] = label0;
  }
  __syncthreads();
  // mark masked experts (after everyone has read start_s[e+1])
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    bool on = p.vllm || p.mask == nullptr || p.mask[e] != 0;
    if (!on) start_s[e] = -1;
  }
  __syncthreads();
}

// Stable scatter of one CTA's chunk.  warp_cnt: [kSortWarps][E] smem;
// base_s[e] = destination of this CTA's first route of expert e (or -1).
__device__ void cta_scatter(const SortParams& p, int cta, int* warp_cnt, const int* base_s) {
  const int E = p.E;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = p.chunk / kSortWarps;  // multiple of 32
  const int begin = cta * p.chunk + warp * sub;
  const int end = min(begin + sub, min((cta + 1) * p.chunk, p.R));
  int* mine = warp_cnt + warp * E;
  for (int e = lane; e < E; e += 32) mine[e] = 0;
  __syncwarp();
  // pass 1: this warp's histogram (order-free)
  for (int r = begin + lane; r < end; r += 32) {
    int e = load_expert(p, r);
    if (e >= 0) atomicAdd(&mine[e], 1);
  }
  __syncthreads();
  // exclusive scan over warps per expert, seeded with the CTA base
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int run = base_s[e];
    for (int w = 0; w < kSortWarps; ++w) {
      int c = warp_cnt[w * E + e];
      warp_cnt[w * E + e] = run;
      run += c;
    }
  }
  __syncthreads();
  // pass 2: warp-ordered ranking
  for (int r0 = begin; r0 < end; r0 += 32) {
    const int r = r0 + lane;
    const int e = (r < end) ? load_expert(p, r) : -1;
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    int dst = -1;
    if (e >= 0) {
      const int base = mine[e];
      if (base_s[e] >= 0) dst = base + __popc(peers & ((1u << lane) - 1u));
    }
    __syncwarp();
    if (e >= 0 && (peers & ((1u << lane) - 1u)) == 0) mine[e] += __popc(peers);
    __syncwarp();
    if (dst >= 0) {
      if (p.vllm) {
        p.sorted_ids[dst] = r;
      } else {
        const int token = r / p.topk, slot = r - token * p.topk;
        p.sorted_ids[dst] = (int32_t)((uint32_t)token | ((uint32_t)slot << 24));
        p.sorted_weights[dst] = p.weights[r];
      }
    }
    // every route is visited exactly once here: routes to masked or out-of-range experts get -1
    if (!p.vllm && p.route_pos != nullptr && r < end) p.route_pos[r] = dst;
  }
}

// Pad fill for experts e = first, first+stride, ...: [start+count, next_start).
__device__ void pad_fill(const SortParams& p, const int* start_s, const int* tot, int first,
                         int stride) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int32_t pad_id = p.vllm ? p.R : (int32_t)((uint32_t)p.tokens | ((uint32_t)p.topk << 24));
  for (int e = first + warp * stride; e < p.E; e += nwarps * stride) {
    const int s = start_s[e];
    if (s < 0) continue;
    const int c = tot[e];
    const int padded = ((c + p.unit - 1) / p.unit) * p.unit;
    for (int i = s + c + lane; i < s + padded; i += 32) {
      p.sorted_ids[i] = pad_id;
      if (!p.vllm) p.sorted_weights[i] = 0.f;
    }
  }
}

// ---- single-CTA path ---------------------------------------------------------
__global__ void __launch_bounds__(kSortThreads) k_sort_small(SortParams p) {
  extern __shared__ int smem[];
  int* tot = smem;                 // [E]
  int* start_s = tot + p.E;        // [E+1]
  int* tmp = start_s + p.E + 1;    // [E]
  int* scratch = tmp + p.E;        // [33]
  int* seg_s = scratch + 33;       // [E]
  int* warp_cnt = seg_s + p.E;     // [kSortWarps][E]
  cta_histogram(p, 0, tot);
  build_metadata(p, tot, start_s, tmp, scratch, seg_s);
  cta_scatter(p, 0, warp_cnt, start_s);
  pad_fill(p, start_s, tot, 0, 1);
  if (p.vllm) {
    const int total = start_s[p.E];
    for (int i = total + threadIdx.x; i < p.capacity; i += blockDim.x) p.sorted_ids[i] = p.R;
  }
}

// ---- multi-CTA path -----------------------------------------------------------
__global__ void __launch_bounds__(kSortThreads) k_sort_count(SortParams p) {
  extern __shared__ int smem[];
  cta_histogram(p, blockIdx.x, smem);
  for (int e = threadIdx.x; e < p.E; e += blockDim.x)
    p.cta_counts[blockIdx.x * p.E + e] = smem[e];
}

__global__ void __launch_bounds__(1024) k_sort_scan(SortParams p, int G) {
  extern __shared__ int smem[];
  int* tot = smem;
  int* start_s = tot + p.E;
  int* tmp = start_s + p.E + 1;
  int* scratch = tmp + p.E;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  // column scan: one warp per expert, lanes across CTAs.  A warp takes its experts four at a
  // time and issues all their loads (G <= 128: four 32-CTA blocks each) before the first scan,
  // so the global-memory latency is paid once per batch, not once per expert and block.
  constexpr int EB = 4, GB = kMaxCtas / 32;
  for (int k0 = 0; warp + k0 * nwarps < p.E; k0 += EB) {
    int v[EB][GB];
#pragma unroll
    for (int j = 0; j < EB; ++j) {
      const int e = warp + (k0 + j) * nwarps;
#pragma unroll
      for (int b = 0; b < GB; ++b) {
        const int g = b * 32 + lane;
        v[j][b] = (e < p.E && g < G) ? p.cta_counts[g * p.E + e] : 0;
      }
    }
#pragma unroll
    for (int j = 0; j < EB; ++j) {
      const int e = warp + (k0 + j) * nwarps;
      if (e >= p.E) break;   // warp-uniform
      int carry = 0;
#pragma unroll
      for (int b = 0; b < GB; ++b) {
        const int g = b * 32 + lane;
        int x = v[j][b];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          int y = __shfl_up_sync(0xffffffffu, x, o);
          if (lane >= o) x += y;
        }
        if (g < G) p.cta_counts[g * p.E + e] = carry + x - v[j][b];
        carry += __shfl_sync(0xffffffffu, x, 31);
      }
      if (lane == 0) tot[e] = carry;
    }
  }
  __syncthreads();
  build_metadata(p, tot, start_s, tmp, scratch, scratch + 33);
  for (int e = threadIdx.x; e <= p.E; e += blockDim.x) p.expert_start[e] = start_s[e];
  // expert totals are needed again by the scatter kernel for the pad fill
  for (int e = threadIdx.x; e < p.E; e += blockDim.x) p.expert_start[p.E + 1 + e] = tot[e];
}

__global__ void __launch_bounds__(kSortThreads) k_sort_scatter(SortParams p) {
  extern __shared__ int smem[];
  int* base_s = smem;               // [E]
  int* start_s = base_s + p.E;      // [E+1]
  int* tot = start_s + p.E + 1;     // [E]
  int* warp_cnt = tot + p.E;        // [kSortWarps][E]
  for (int e = threadIdx.x; e < p.E; e += blockDim.x) {
    const int s = p.expert_start[e];
    start_s[e] = s;
    tot[e] = p.expert_start[p.E + 1 + e];
    base_s[e] = (s < 0) ? -1 : s + p.cta_counts[blockIdx.x * p.E + e];
  }
  if (threadIdx.x == 0) start_s[p.E] = p.expert_start[p.E];
  __syncthreads();
  cta_scatter(p, blockIdx.x, warp_cnt, base_s);
  pad_fill(p, start_s, tot, blockIdx.x, gridDim.x);
  if (p.vllm) {
    const int total = start_s[p.E];
    for (int i = total + blockIdx.x * blockDim.x + threadIdx.x; i < p.capacity;
         i += gridDim.x * blockDim.x)
      p.sorted_ids[i] = p.R;
  }
}

struct SortPlan {
  int G;      // CTAs
  int chunk;  // routes per CTA
};

SortPlan make_plan(int64_t R) {
  const int gran = 32 * kSortWarps;
  SortPlan pl;
  if (R <= kSmallRoutes) {
    pl.G = 1;
    pl.chunk = (int)(((R + gran - 1) / gran) * gran);
    if (pl.chunk == 0) pl.chunk = gran;
    return pl;
  }
  int64_t chunk = (R + kMaxCtas - 1) / kMaxCtas;
  chunk = ((chunk + gran - 1) / gran) * gran;
  pl.chunk = (int)chunk;
  pl.G = (int)((R + chunk - 1) / chunk);
  return pl;
}

size_t workspace_bytes_for(int64_t R, int E) {
  SortPlan pl = make_plan(R);
  if (pl.G == 1) return 16;
  return (size_t)(pl.G * (size_t)E + 2 * (size_t)E + 1) * sizeof(int32_t) + 16;
}

int run_sort(SortParams p, void* workspace, size_t workspace_bytes, cudaStream_t st) {
  SortPlan pl = make_plan(p.R);
  p.chunk = pl.chunk;
  const size_t need = workspace_bytes_for(p.R, p.E);
  if (pl.G == 1) {
    size_t smem = (size_t)(4 * p.E + 1 + 33 + kSortWarps * p.E) * sizeof(int);
    BOLT_REQUIRE(smem <= 200 * 1024, "moe sort: num_experts %d too large", p.E);
    if (smem > 48 * 1024)
      BOLT_CUDA(cudaFuncSetAttribute(k_sort_small, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)smem));
    k_sort_small<<<1, kSortThreads, smem, st>>>(p);
    BOLT_LAUNCH_CHECK();
    return BOLT_OK;
  }
  BOLT_REQUIRE(workspace != nullptr && workspace_bytes >= need,
               "moe sort: workspace too small (%zu < %zu)", workspace_bytes, need);
  BOLT_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 15) == 0,
               "moe sort: workspace must be 16-byte aligned");
  p.cta_counts = static_cast<int32_t*>(workspace);
  p.expert_start = p.cta_counts + (size_t)pl.G * p.E;
  size_t smem1 = (size_t)p.E * sizeof(int);
  size_t smem2 = (size_t)(4 * p.E + 1 + 33) * sizeof(int);
  size_t smem3 = (size_t)(3 * p.E + 1 + kSortWarps * p.E) * sizeof(int);
  BOLT_REQUIRE(smem3 <= 200 * 1024, "moe sort: num_experts %d too large", p.E);
  if (smem3 > 48 * 1024)
    BOLT_CUDA(cudaFuncSetAttribute(k_sort_scatter, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   (int)smem3));
  k_sort_count<<<pl.G, kSortThreads, smem1, st>>>(p);
  BOLT_LAUNCH_CHECK();
  k_sort_scan<<<1, 1024, smem2, st>>>(p, pl.G);
  BOLT_LAUNCH_CHECK();
  k_sort_scatter<<<pl.G, kSortThreads, smem3, st>>>(p);
  BOLT_LAUNCH_CHECK();
  return BOLT_OK;
}

}  // namespace
}  // namespace bolt

extern "C" size_t bolt_moe_sort_workspace_bytes(int num_tokens, int topk, int num_experts) {
  if (num_tokens < 0 || topk <= 0 || num_experts <= 0) return 16;
  return bolt::workspace_bytes_for((int64_t)num_tokens * topk, num_experts);
}

extern "C" int bolt_moe_sort_ck(const int32_t* topk_ids, const float* topk_weights,
                                const int32_t* local_expert_mask, int num_tokens, int topk,
                                int num_experts, int unit_size, int32_t* sorted_ids,
                                float* sorted_weights, int32_t* sorted_expert_ids,
                                int32_t* tokens_positions_per_expert, int32_t* num_valid_ids,
                                int32_t* route_pos, int32_t* segments, int32_t* num_segments,
                                int segment_rows, void* moe_buf, size_t moe_buf_bytes,
                                void* workspace, size_t workspace_bytes, void* stream) {
  using namespace bolt;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  BOLT_REQUIRE(num_tokens >= 0 && num_tokens < (1 << 24), "moe sort: num_tokens %d out of range",
               num_tokens);
  BOLT_REQUIRE(topk > 0 && topk <= 255, "moe sort: topk %d out of range", topk);
  BOLT_REQUIRE(num_experts > 0 && unit_size > 0, "moe sort: bad num_experts/unit_size");
  BOLT_REQUIRE((int64_t)num_tokens * topk < (1ll << 30), "moe sort: too many routes");
  BOLT_REQUIRE(sorted_ids && sorted_weights && sorted_expert_ids && num_valid_ids,
               "moe sort: null output");
  BOLT_REQUIRE(num_tokens == 0 || (topk_ids && topk_weights), "moe sort: null input");
  SortParams p{};
  p.ids = topk_ids;
  p.weights = topk_weights;
  p.mask = local_expert_mask;
  p.sorted_ids = sorted_ids;
  p.sorted_weights = sorted_weights;
  p.expert_ids = sorted_expert_ids;
  p.positions = tokens_positions_per_expert;
  p.num_valid = num_valid_ids;
  p.route_pos = route_pos;
  BOLT_REQUIRE(segments == nullptr || (num_segments != nullptr && segment_rows > 0),
               "moe sort: segments need num_segments and a positive segment_rows");
  p.segments = segments;
  p.num_segments = num_segments;
  p.segment_rows = segment_rows;
  p.R = num_tokens * topk;
  p.E = num_experts;
  p.topk = topk;
  p.tokens = num_tokens;
  p.unit = unit_size;
  p.capacity = p.R + num_experts * unit_size - topk;
  p.num_blocks = (p.capacity + unit_size - 1) / unit_size;
  p.vllm = 0;
  if (moe_buf != nullptr && moe_buf_bytes > 0)
    BOLT_CUDA(cudaMemsetAsync(moe_buf, 0, moe_buf_bytes, st));
  return run_sort(p, workspace, workspace_bytes, st);
}

// ---------------------------------------------------------------------------
// Allocation-free variant of the CK-format sort.
//
// Scratch for the multi-CTA path lives in a fixed array inside the library image
// instead of a caller-provided workspace.  The array's name is only a host-side
// stand-in in host code, so its device address is looked up once per device with
// cudaGetSymbolAddress (with that device current) and passed to the kernels.
// ---------------------------------------------------------------------------
namespace bolt {
namespace {
constexpr size_t kStaticScratchBytes = 1u << 20;  // 1 MiB, held by every GPU that loads the library
static __device__ __align__(256) unsigned char g_sort_scratch[kStaticScratchBytes];
// per-device address of g_sort_scratch; atomic because two host threads may make their first
// call on a device at the same time (both would store the same value)
std::atomic<void*> g_sort_scratch_ptr[64];
}  // namespace
}  // namespace bolt

extern "C" size_t bolt_moe_sort_static_scratch_bytes(void) { return bolt::kStaticScratchBytes; }

extern "C" int bolt_moe_sort_ck_static(const int32_t* topk_ids, const float* topk_weights,
                                       const int32_t* local_expert_mask, int num_tokens, int topk,
                                       int num_experts, int unit_size, int32_t* sorted_ids,
                                       float* sorted_weights, int32_t* sorted_expert_ids,
                                       int32_t* tokens_positions_per_expert,
                                       int32_t* num_valid_ids, void* stream) {
  using namespace bolt;
  BOLT_REQUIRE(num_tokens >= 0 && topk > 0 && num_experts > 0, "moe sort (static): bad sizes");
  const size_t need = workspace_bytes_for((int64_t)num_tokens * topk, num_experts);
  BOLT_REQUIRE(need <= kStaticScratchBytes,
               "moe sort (static): %d tokens x top-%d over %d experts needs %zu bytes of scratch, "
               "the built-in array holds %zu; use bolt_moe_sort_ck with a caller workspace",
               num_tokens, topk, num_experts, need, kStaticScratchBytes);
  int dev = 0;
  BOLT_CUDA(cudaGetDevice(&dev));
  BOLT_REQUIRE(dev >= 0 && dev < 64, "moe sort (static): device index %d out of range", dev);
  void* scratch = g_sort_scratch_ptr[dev].load(std::memory_order_relaxed);
  if (scratch == nullptr) {
    // one-time set-up for this device: resolve the array's device address
    BOLT_CUDA(cudaGetSymbolAddress(&scratch, g_sort_scratch));
    g_sort_scratch_ptr[dev].store(scratch, std::memory_order_relaxed);
  }
  // No entry of the scratch has to start at zero: the count kernel writes every
  // per-CTA histogram entry and the scan kernel every offset before it is read.
  return bolt_moe_sort_ck(topk_ids, topk_weights, local_expert_mask, num_tokens, topk,
                          num_experts, unit_size, sorted_ids, sorted_weights, sorted_expert_ids,
                          tokens_positions_per_expert, num_valid_ids, nullptr, nullptr, nullptr, 0,
                          nullptr, 0, scratch, kStaticScratchBytes, stream);
}

extern "C" int bolt_moe_align_block_size(const int32_t* topk_ids, int numel, int num_experts,
                                         int block_size, const int32_t* expert_map,
                                         int32_t* sorted_ids, int32_t* expert_ids,
                                         int32_t* num_tokens_post_pad, void* workspace,
                                         size_t workspace_bytes, void* stream) {
  using namespace bolt;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  BOLT_REQUIRE(numel >= 0 && numel < (1 << 30), "align: numel out of range");
  BOLT_REQUIRE(num_experts > 0 && block_size > 0, "align: bad num_experts/block_size");
  BOLT_REQUIRE(sorted_ids && expert_ids && num_tokens_post_pad, "align: null output");
  BOLT_REQUIRE(numel == 0 || topk_ids, "align: null input");
  SortParams p{};
  p.ids = topk_ids;
  p.expert_map = expert_map;
  p.sorted_ids = sorted_ids;
  p.expert_ids = expert_ids;
  p.num_valid = num_tokens_post_pad;
  p.R = numel;
  p.E = num_experts;
  p.topk = 1;
  p.tokens = numel;
  p.unit = block_size;
  p.capacity = numel + num_experts * (block_size - 1);
  p.num_blocks = (p.capacity + block_size - 1) / block_size;
  p.vllm = 1;
  return run_sort(p, workspace, workspace_bytes, st);
}
