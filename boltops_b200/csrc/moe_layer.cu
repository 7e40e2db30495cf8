// One fused-MoE layer in one call: sort -> (quantise and) place rows in expert-sorted order ->
// grouped GEMM 1 with SiLU(gate)*up (+ 1x128 re-quantisation) -> grouped GEMM 2 with the router
// weight -> top-k combine, all enqueued on the caller's stream from one host entry with one
// caller-provided workspace.
//
// Why it exists: for decode-sized batches the kernels of a layer take a few tens of
// microseconds, while driving them one by one from Python (an allocation, an argument struct and
// a foreign call each) costs several times that.  This entry is the same schedule as the Python
// orchestration of boltops_b200/fused_moe/layer.py for the common variant (gated SiLU, combined
// output, unquantised 16-bit input), so the host cost per layer is one foreign call.
//
// Reference: the work of fused_experts_impl (boltops/fused_moe/triton/fused_moe.py:1200-1777 of
// the reference project) for that variant.
#include "common.cuh"

#include <cstdlib>
#include <cstring>

namespace bolt {
namespace {

constexpr int kUnit = 128;

// 16-bit and block-scaled experts: GEMM 1 can gather its rows from token order itself -- the
// input as it is, or 8-bit codes that the quantiser writes once per token instead of once per
// route -- instead of reading a copy in sorted order.  Same results.  The gather wins while the
// sorted layout is mostly tile padding (measured on the DeepSeek-V3 fp8 layer: 0.120 vs 0.152 ms
// at 8 routes, 0.49 vs 0.52 ms at 16 routes per expert, even at 128, 4.56 vs 4.51 ms at 256
// routes per expert, where the extra copy instructions slow the accumulator promotion down), so
// it is used up to kGatherMaxAvgRows routes per expert.  BOLTOPS_B200_GATHER=0 / 1 forces it off
// / on.
constexpr int kGatherMaxAvgRows = 64;
bool gather_rows_in_gemm(const bolt_layer_args* a) {
  static const int forced = [] {
    const char* v = std::getenv("BOLTOPS_B200_GATHER");
    if (v == nullptr) return -1;
    return std::strcmp(v, "0") != 0 ? 1 : 0;
  }();
  if (forced >= 0) return forced == 1;
  return (int64_t)a->num_tokens * a->topk <= (int64_t)kGatherMaxAvgRows * a->global_num_experts;
}

inline size_t a256(size_t n) { return (n + 255) & ~size_t(255); }

struct Plan {
  int cap;            // rows of the sorted layout (multiple of 128)
  int blocks;
  bool quant, block, is16;
  bool gather;        // GEMM 1 reads token-order rows through the sorted ids
  int qbytes;         // bytes per operand element of the GEMMs
  size_t off_sorted_ids, off_sorted_w, off_expert_ids, off_positions, off_num_valid, off_route_pos,
      off_sort_ws, sort_ws_bytes, off_a1, off_a1_scale, off_xq, off_xq_scale, off_a2, off_a2_scale,
      off_actf, off_c, total;
};

int make_plan(const bolt_layer_args* a, Plan& p) {
  const int64_t routes = (int64_t)a->num_tokens * a->topk;
  const int64_t cap = routes + (int64_t)a->global_num_experts * kUnit - a->topk;
  BOLT_REQUIRE(cap >= 0 && cap < (1ll << 30), "moe_layer: too many routes");
  p.cap = (int)((cap + kUnit - 1) / kUnit * kUnit);
  p.blocks = p.cap / kUnit;
  p.is16 = a->kind == BOLT_GEMM_BF16 || a->kind == BOLT_GEMM_F16;
  p.block = a->kind == BOLT_GEMM_FP8_BLOCK || a->kind == BOLT_GEMM_INT8_BLOCK;
  p.quant = !p.is16;
  p.qbytes = p.is16 ? 2 : 1;
  p.gather = (p.block || p.is16) && gather_rows_in_gemm(a);
  const int osz = dtype_bytes(a->out_dtype);
  size_t o = 0;
  auto take = [&](size_t bytes) { size_t at = o; o += a256(bytes); return at; };
  p.off_sorted_ids = take((size_t)p.cap * 4);
  p.off_sorted_w = take((size_t)p.cap * 4);
  p.off_expert_ids = take((size_t)(p.blocks > 0 ? p.blocks : 1) * 4);
  p.off_positions = take((size_t)2 * a->global_num_experts * 4);
  p.off_num_valid = take(16);
  p.off_route_pos = take((size_t)routes * 4);
  p.sort_ws_bytes = bolt_moe_sort_workspace_bytes(a->num_tokens, a->topk, a->global_num_experts);
  p.off_sort_ws = take(p.sort_ws_bytes);
  p.off_a1 = take(p.gather ? (p.is16 ? 0 : (size_t)a->num_tokens * a->hidden)
                           : (size_t)p.cap * a->hidden * p.qbytes);
  p.off_a1_scale = take(p.block ? (size_t)(a->hidden / 128) * p.cap * 4 : (p.quant ? (size_t)p.cap * 4 : 0));
  // per-channel kinds quantise every token once, then gather codes and scales
  p.off_xq = take(p.quant && !p.block ? (size_t)a->num_tokens * a->hidden : 0);
  p.off_xq_scale = take(p.quant && !p.block ? (size_t)a->num_tokens * 4 : 0);
  p.off_a2 = take((size_t)p.cap * a->inter * p.qbytes);
  p.off_a2_scale = take(p.block ? (size_t)(a->inter / 128) * p.cap * 4 : (p.quant ? (size_t)p.cap * 4 : 0));
  p.off_actf = take(p.quant && !p.block ? (size_t)p.cap * a->inter * osz : 0);
  p.off_c = take((size_t)p.cap * a->model_dim * osz);
  p.total = o;
  return BOLT_OK;
}

int check_args(const bolt_layer_args* a) {
  BOLT_REQUIRE(a != nullptr, "moe_layer: null args");
  BOLT_REQUIRE(a->kind >= BOLT_GEMM_BF16 && a->kind <= BOLT_GEMM_INT8_BLOCK,
               "moe_layer: kind %d is not built into the one-call layer", a->kind);
  BOLT_REQUIRE(a->num_tokens >= 0 && a->topk > 0 && a->hidden > 0 && a->inter > 0 &&
                   a->model_dim > 0 && a->num_experts > 0 && a->global_num_experts > 0,
               "moe_layer: bad shape");
  BOLT_REQUIRE(a->x_dtype == BOLT_BF16 || a->x_dtype == BOLT_F16,
               "moe_layer: hidden_states must be bf16 or f16");
  BOLT_REQUIRE(a->out_dtype == BOLT_BF16 || a->out_dtype == BOLT_F16 || a->out_dtype == BOLT_F32,
               "moe_layer: bad out_dtype %d", a->out_dtype);
  const bool is16 = a->kind == BOLT_GEMM_BF16 || a->kind == BOLT_GEMM_F16;
  const bool block = a->kind == BOLT_GEMM_FP8_BLOCK || a->kind == BOLT_GEMM_INT8_BLOCK;
  if (is16)
    BOLT_REQUIRE((a->kind == BOLT_GEMM_BF16) == (a->x_dtype == BOLT_BF16),
                 "moe_layer: hidden_states dtype does not match the weights");
  else
    BOLT_REQUIRE(a->w1_scale && a->w2_scale, "moe_layer: weight scales required");
  if (block)
    BOLT_REQUIRE(a->hidden % 128 == 0 && a->inter % 128 == 0,
                 "moe_layer: block-scaled experts need hidden and intermediate sizes in 128s");
  return BOLT_OK;
}

}  // namespace
}  // namespace bolt

extern "C" size_t bolt_moe_layer_workspace_bytes(const bolt_layer_args* a) {
  using namespace bolt;
  Plan p;
  if (check_args(a) != BOLT_OK || make_plan(a, p) != BOLT_OK) return 0;
  return p.total;
}

extern "C" int bolt_moe_layer_kernel_count(const bolt_layer_args* a) {
  using namespace bolt;
  Plan p;
  if (check_args(a) != BOLT_OK || make_plan(a, p) != BOLT_OK) return -1;
  if (a->num_tokens == 0) return 0;
  const int sort = p.sort_ws_bytes <= 16 ? 1 : 3;
  const int place = p.block ? 1 : (p.quant ? 2 : (p.gather ? 0 : 1));
  return sort + place + 2 + (p.quant && !p.block ? 1 : 0) + 1;
}

extern "C" int bolt_moe_layer(const bolt_layer_args* a, void* stream) {
  using namespace bolt;
  int rc = check_args(a);
  if (rc != BOLT_OK) return rc;
  if (a->num_tokens == 0) return BOLT_OK;
  BOLT_REQUIRE(a->hidden_states && a->w1 && a->w2 && a->topk_weights && a->topk_ids && a->out &&
                   a->workspace,
               "moe_layer: null pointer");
  Plan p;
  rc = make_plan(a, p);
  if (rc != BOLT_OK) return rc;
  BOLT_REQUIRE(a->workspace_bytes >= p.total, "moe_layer: workspace too small (%zu < %zu)",
               a->workspace_bytes, p.total);
  BOLT_REQUIRE(reinterpret_cast<uintptr_t>(a->workspace) % 256 == 0,
               "moe_layer: workspace must be 256-byte aligned");
  uint8_t* ws = static_cast<uint8_t*>(a->workspace);
  auto i32 = [&](size_t off) { return reinterpret_cast<int32_t*>(ws + off); };
  auto f32 = [&](size_t off) { return reinterpret_cast<float*>(ws + off); };
  int32_t* sorted_ids = i32(p.off_sorted_ids);
  float* sorted_w = f32(p.off_sorted_w);
  int32_t* expert_ids = i32(p.off_expert_ids);
  int32_t* num_valid = i32(p.off_num_valid);
  int32_t* route_pos = i32(p.off_route_pos);
  const int q_dtype = (a->kind == BOLT_GEMM_FP8_BLOCK || a->kind == BOLT_GEMM_FP8_CHANNEL)
                          ? BOLT_FP8_E4M3 : BOLT_INT8;

  rc = bolt_moe_sort_ck(a->topk_ids, a->topk_weights, a->expert_mask, a->num_tokens, a->topk,
                        a->global_num_experts, kUnit, sorted_ids, sorted_w, expert_ids,
                        i32(p.off_positions), num_valid, route_pos, nullptr, nullptr, 0, nullptr, 0,
                        ws + p.off_sort_ws, p.sort_ws_bytes, stream);
  if (rc != BOLT_OK) return rc;

  void* a1 = ws + p.off_a1;
  float* a1_scale = p.quant ? f32(p.off_a1_scale) : nullptr;
  if (p.block) {
    rc = bolt_quant_scatter_rows(a->hidden_states, a->x_dtype, a->num_tokens, a->hidden, 128,
                                 q_dtype, 0, route_pos, a->topk, sorted_ids, num_valid, p.cap, a1,
                                 a1_scale, p.cap, p.gather ? 1 : 0, stream);
  } else if (p.quant) {
    rc = bolt_quant_rows(a->hidden_states, a->x_dtype, a->num_tokens, a->hidden, a->hidden,
                         q_dtype, 0, ws + p.off_xq, f32(p.off_xq_scale), 0, stream);
    if (rc == BOLT_OK)
      rc = bolt_gather_rows(ws + p.off_xq, a->num_tokens, a->hidden, 0, f32(p.off_xq_scale), 0, 1,
                            sorted_ids, num_valid, p.cap, a1, a1_scale, p.cap, stream);
  } else if (!p.gather) {
    rc = bolt_gather_rows(a->hidden_states, a->num_tokens, a->hidden * 2, 0, nullptr, 0, 0,
                          sorted_ids, num_valid, p.cap, a1, nullptr, 0, stream);
  }
  if (rc != BOLT_OK) return rc;

  bolt_gemm_args g{};
  g.kind = a->kind;
  g.capacity = p.cap;
  g.num_experts = a->num_experts;
  g.num_tokens = a->num_tokens;
  g.topk = a->topk;
  g.sorted_ids = sorted_ids;
  g.sorted_weights = sorted_w;
  g.sorted_expert_ids = expert_ids;
  g.num_valid_ids = num_valid;
  g.status = a->status;
  g.mid_dtype = a->out_dtype;
  g.bias_dtype = a->bias_dtype;

  // ---- GEMM 1: gate / up with SiLU(gate) * up (and the 1x128 re-quantisation) in the epilogue
  void* a2 = ws + p.off_a2;
  float* a2_scale = p.quant ? f32(p.off_a2_scale) : nullptr;
  g.n = 2 * a->inter;
  g.k = a->hidden;
  g.a = (p.gather && p.is16) ? a->hidden_states : a1;
  g.b = a->w1;
  g.a_scale = a1_scale;
  g.a_scale_ld = p.cap;
  g.b_scale = a->w1_scale;
  g.bias = a->b1;
  g.mul_routed_weight = a->apply_router_weight_on_input;
  if (p.gather) {
    g.a_gather = 1;
    g.a_rows = a->num_tokens;
  }
  if (p.block) {
    g.epilogue = BOLT_EPI_SILU_MUL_QUANT;
    g.c = a2;
    g.c_dtype = q_dtype;
    g.c_ld = a->inter;
    g.c_scale = a2_scale;
    g.c_scale_ld = p.cap;
  } else {
    g.epilogue = BOLT_EPI_SILU_MUL;
    g.c = p.quant ? static_cast<void*>(ws + p.off_actf) : a2;
    g.c_dtype = a->out_dtype;
    g.c_ld = a->inter;
  }
  rc = bolt_grouped_gemm(&g, stream);
  if (rc != BOLT_OK) return rc;
  if (p.quant && !p.block) {
    rc = bolt_quant_rows(ws + p.off_actf, a->out_dtype, p.cap, a->inter, a->inter, q_dtype, 0, a2,
                         a2_scale, 0, stream);
    if (rc != BOLT_OK) return rc;
  }

  // ---- GEMM 2: down projection, router weight in the epilogue, rows stay in sorted order
  g.a_gather = 0;
  g.epilogue = BOLT_EPI_STORE;
  g.n = a->model_dim;
  g.k = a->inter;
  g.a = a2;
  g.b = a->w2;
  g.a_scale = a2_scale;
  g.a_scale_ld = p.cap;
  g.b_scale = a->w2_scale;
  g.bias = a->b2;
  g.c = ws + p.off_c;
  g.c_dtype = a->out_dtype;
  g.c_ld = a->model_dim;
  g.c_scale = nullptr;
  g.c_scale_ld = 0;
  g.mul_routed_weight = !a->apply_router_weight_on_input;
  rc = bolt_grouped_gemm(&g, stream);
  if (rc != BOLT_OK) return rc;

  // ---- combine: out[m] = cast(s * sum_k f32(C[route_pos[m, k]])), k ascending
  return bolt_moe_gather_sum(ws + p.off_c, a->out_dtype, route_pos, a->out, a->out_dtype,
                             a->num_tokens, a->topk, a->model_dim, a->routed_scaling_factor, stream);
}
