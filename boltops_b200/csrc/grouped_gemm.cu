// Grouped expert GEMM for sm_100a: persistent, warp-specialised, TMA-fed,
// tcgen05.mma with TMEM accumulators.
//
//   C[rows of tile t, :] = epilogue( A[tile t, :] . B[expert_ids[t], :, :]^T )
//
// A is in the expert-sorted padded layout (128-row tiles, one expert per tile),
// B is [E, N, K] row-major.  One CTA per SM loops over (row tile, column tile)
// pairs; the number of valid row tiles is read from device memory, so the host
// never synchronises.
//
// Roles (384 threads): warp 0 = TMA producer, warp 1 = MMA issuer + TMEM owner,
// warps 4..11 = epilogue (warp w reads TMEM lanes 32*(w%4).., accumulator half (w-4)/4).
//
// Tile: 128 rows x 256 accumulator columns, K step = 128 bytes (one 128B-swizzle
// atom: 64 x 16-bit or 128 x 8-bit).  The 256 columns are two halves of 128, each
// drained by its own four epilogue warps.  For the gated epilogue each half holds
// 64 gate columns and the matching 64 up columns (B rows n0.. and N/2+n0.., loaded
// as four 64-row TMA boxes stacked in one operand tile), so
// SiLU(gate)*up, the rounding steps of the unfused reference path and the 1x128
// group quantisation of the result all happen in registers.
//
// Block-scaled operands (128x128 weight blocks, 1x128 activation groups): each
// 128-deep K block is multiplied into a fresh TMEM stage; the epilogue warps read
// it back and accumulate `partial * (a_scale[row,kb] * b_scale[nb,kb])` in fp32
// registers while the tensor core works on the next K block (two TMEM stages).
//
// Every wait on an mbarrier is bounded; on expiry the kernel records a status
// word, stops issuing work, drains and frees its TMEM before returning.
#include <cuda.h>
#include <atomic>
#include <cstring>

#include "common.cuh"
#include "tc_ptx.cuh"

namespace bolt {
namespace {
using namespace tc;

constexpr int kThreads = 384;
constexpr int kMaxDevices = 64;
// shared-memory operand stages: the block-scaled kinds spend ~950 cycles per K block (three
// stages cover the load latency, and the space goes to bulk-store slots); the others stream a
// K block every ~500 cycles and need four
constexpr int stages_of(bool block_scaled) { return block_scaled ? 3 : 4; }
constexpr int kBM = 128;
constexpr int kAccCols = 256;           // accumulator columns per tile
constexpr int kHalfCols = 128;          // columns of one independently scheduled half
constexpr int kTmemCols = 512;          // two accumulator stages
constexpr int kABytes = kBM * 128;      // 16 KiB
constexpr int kBBytes = kAccCols * 128; // 32 KiB
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kScaleSlots = 8;           // ring of per-K-block activation-scale rows (512 B each)
constexpr int kOutSlotBytes = 32 * 64;    // one 32-row x 64-byte block as a bulk store reads it
// per epilogue warp: block-scaled kinds one slot per 32-column chunk of a tile, the others one
// slot that is reclaimed chunk by chunk (their epilogue overlaps the next tile's MMAs anyway)
constexpr int out_slots_of(bool block_scaled) { return block_scaled ? 4 : 1; }
constexpr int out_stage_bytes_of(bool block_scaled) { return block_scaled ? 4 * kOutSlotBytes : 2560; }
// (the padded 32 x 80 B layout of the staged fallback path fits in either)
constexpr int smem_bytes_of(bool block_scaled) {
  return stages_of(block_scaled) * kStageBytes + 4096 + kScaleSlots * 512 +
         8 * out_stage_bytes_of(block_scaled) + 1024;  // +1024 alignment slack
}
// CTA pairs stage half of the B tile per CTA: 32 KiB per stage, so more stages fit
constexpr int kPairStageBytes = kABytes + kBBytes / 2;
constexpr int pair_stages_of(bool block_scaled) { return block_scaled ? 4 : 5; }
constexpr int pair_smem_bytes_of(bool block_scaled) {
  return pair_stages_of(block_scaled) * kPairStageBytes + 4096 + kScaleSlots * 512 +
         8 * out_stage_bytes_of(block_scaled) + 1024;
}


struct GemmParams {
  const float* a_scale;
  int64_t a_scale_ld;
  const float* b_scale;
  const void* bias;
  int bias_dtype;
  void* c;
  int c_dtype;
  int mid_dtype;
  int64_t c_ld;
  float* c_scale;
  int64_t c_scale_ld;
  int scatter, num_tokens, topk, mul_routed_weight;
  int c_vec_ok;  // output rows are 16-byte aligned: coalesced staged stores may be used
  int c_tma_ok;  // a tensor map over the 16-bit output exists: whole 32-row blocks go out by TMA
  const int32_t* sorted_ids;
  const float* sorted_weights;
  const int32_t* expert_ids;
  const int32_t* num_valid;
  int32_t* status;
  int n;        // B rows per expert
  int n_half;   // n/2 for the gated epilogues
  int k;
  int num_experts;
  int capacity;
  int tiles_n;
  int num_kb;
  int kb_scale_cols;  // k/128 (block-scaled kinds)
  uint32_t idesc;
  int group_m;
  // scattered output with per-segment bases: row of token t goes to row scatter_src[t] * topk + slot
  // of the region that lies scatter_seg_off[t / scatter_seg_rows] ELEMENTS behind c (another
  // rank's memory in the expert-parallel exchange)
  const int32_t* scatter_src;
  const int64_t* scatter_seg_off;
  int scatter_seg_rows;
  // gathered row operand: A is in TOKEN order; sorted position p reads row (sorted_ids[p] & 0xFFFFFF),
  // or zeros when that id is not a token (tile padding)
  int a_gather;
  const void* a_base;
  int a_row_units;   // 16-byte units between rows
  int k_bytes;
  // tile-pair schedule: work list of the sort (runs of at most 256 rows of one expert)
  const int32_t* segments;     // [max_segments][4] = {expert, first row, rows, -}
  const int32_t* num_segments;
  int max_segments;
  // MX kind: E8M0 bytes in 512-byte tiles of (128 rows x 4 K groups), see k_mx_gemm
  const uint8_t* sfa;   // [capacity/128][num_kb][512]
  const uint8_t* sfb;   // [num_experts][n_blocks128][num_kb][512]
  int n_blocks128;
  int mx_stage_tx;      // operand bytes one K block brings (packed 4-bit weights count as stored)
  int mx_group128;      // gated epilogue: 1 x 128 power-of-two groups (the MXFP4 w4a8 recipe)
  float act_alpha, act_beta, act_limit;   // MX gated epilogue
  int act_has_limit;
};

// Store 32 consecutive fp32 values as c_dtype starting at column col0 (masked to ncols).
__device__ __forceinline__ void store_row32(void* c, int dt, int64_t row_off, int col0, int ncols,
                                            const float (&v)[32]) {
  if (col0 >= ncols) return;
  const bool full = col0 + 32 <= ncols;
  if (dt == BOLT_F32) {
    float* dst = static_cast<float*>(c) + row_off + col0;
    if (full && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
      for (int j = 0; j < 32; j += 4)
        *reinterpret_cast<float4*>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < ncols) dst[j] = v[j];
    }
    return;
  }
  uint32_t packed[16];
  if (dt == BOLT_BF16) {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
      packed[j] = *reinterpret_cast<uint32_t*>(&h);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      __half2 h = __floats2half2_rn(v[2 * j], v[2 * j + 1]);
      packed[j] = *reinterpret_cast<uint32_t*>(&h);
    }
  }
  uint16_t* dst = static_cast<uint16_t*>(c) + row_off + col0;
  if (full && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
    for (int j = 0; j < 16; j += 4)
      *reinterpret_cast<uint4*>(dst + 2 * j) =
          make_uint4(packed[j], packed[j + 1], packed[j + 2], packed[j + 3]);
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (col0 + j < ncols) dst[j] = (uint16_t)(packed[j >> 1] >> ((j & 1) * 16));
  }
}

// Pack 32 fp32 values into 64 bytes of bf16 / f16.
__device__ __forceinline__ void pack32_16bit(const float (&v)[32], int dt, uint4 (&w)[4]) {
  uint32_t pk[16];
  if (dt == BOLT_BF16) {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
      pk[j] = *reinterpret_cast<uint32_t*>(&h);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      __half2 h = __floats2half2_rn(v[2 * j], v[2 * j + 1]);
      pk[j] = *reinterpret_cast<uint32_t*>(&h);
    }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) w[j] = make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
}

// Warp-cooperative store of a 32-row x 64-byte block that is held one row per lane.
// A direct store would touch 32 rows with 16 bytes each per instruction; staging the
// block in shared memory (80-byte row pitch: conflict-free both ways) lets every
// instruction write eight complete 64-byte row segments instead.
__device__ __forceinline__ void store_rows_64B(uint8_t* stage, const uint4 (&w)[4], uint8_t* c,
                                               int64_t row_byte_off, bool live, int lane) {
  const unsigned live_mask = __ballot_sync(0xffffffffu, live);
  if (lane == 0) bulk_wait_read();   // a bulk store of an earlier block may still read the buffer
  __syncwarp();
  uint4* mine = reinterpret_cast<uint4*>(stage + lane * 80);
#pragma unroll
  for (int j = 0; j < 4; ++j) mine[j] = w[j];
  __syncwarp();
  const int seg = lane & 3;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int r = (lane >> 2) + 8 * k;
    const int64_t off = __shfl_sync(0xffffffffu, row_byte_off, r);
    if ((live_mask >> r) & 1u) {
      const uint4 x = *reinterpret_cast<const uint4*>(stage + r * 80 + seg * 16);
      *reinterpret_cast<uint4*>(c + off + seg * 16) = x;
    }
  }
  __syncwarp();
}

// Warp-cooperative store of a 32-row x 256-byte block (one row per lane, 128 16-bit columns) to
// rows anywhere in memory: staged in 8 KiB of shared memory (16-byte chunk c of row r at chunk
// position c ^ (r & 15): conflict-free both ways), then sixteen lanes write one row's 256
// contiguous bytes per instruction.  Whole 256-byte segments are what a store over NVLink wants.
__device__ __forceinline__ void store_rows_256B(uint8_t* stage, const float (&v)[4][32], int dt,
                                                uint8_t* c, int64_t row_byte_off, bool live,
                                                int lane) {
  const unsigned live_mask = __ballot_sync(0xffffffffu, live);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint4 w[4];
    pack32_16bit(v[i], dt, w);
#pragma unroll
    for (int j = 0; j < 4; ++j)
      *reinterpret_cast<uint4*>(stage + lane * 256 + (((4 * i + j) ^ (lane & 15)) << 4)) = w[j];
  }
  __syncwarp();
  const int seg = lane & 15;
#pragma unroll
  for (int k = 0; k < 16; ++k) {
    const int r = (lane >> 4) + 2 * k;
    const int64_t off = __shfl_sync(0xffffffffu, row_byte_off, r);
    if ((live_mask >> r) & 1u) {
      const uint4 x = *reinterpret_cast<const uint4*>(stage + r * 256 + ((seg ^ (r & 15)) << 4));
      *reinterpret_cast<uint4*>(c + off + seg * 16) = x;
    }
  }
  __syncwarp();
}

// Warp-cooperative store of a 32-row x 64-byte block (one row per lane, rows row0 .. row0+31 of
// the output) by one bulk tensor copy.  The block is laid out in shared memory the way a
// 64-byte-swizzled tensor map expects it (16-byte chunk index XOR bits 1-2 of the row), which
// also makes the per-lane 16-byte writes conflict-free.  The copy runs asynchronously; every
// chunk of a tile has a slot of its own, and the slots are reclaimed once per tile (the caller
// waits for the previous tile's copies to have read them before the first chunk).
__device__ __forceinline__ void store_rows_tma(uint8_t* stage, const uint4 (&w)[4],
                                               const CUtensorMap* map, int col0, int row0,
                                               int lane) {
  const int sw = (lane >> 1) & 3;
#pragma unroll
  for (int j = 0; j < 4; ++j)
    *reinterpret_cast<uint4*>(stage + lane * 64 + ((j ^ sw) << 4)) = w[j];
  fence_async_smem();
  __syncwarp();
  if (lane == 0) {
    tma_store_2d(map, smem_u32(stage), col0, row0);
    bulk_commit();
  }
}

// 32 fp32 values -> c_dtype at column col0 of this lane's row: by TMA when the whole 32-row
// block is written, else staged through shared memory when possible.  tile_row0 = output row
// of lane 0 (only meaningful when rows are not scattered).
template <int SLOTS>
__device__ __forceinline__ void store_chunk(uint8_t* stage, int slot, const GemmParams& p,
                                            const CUtensorMap* map_c, int tile_row0,
                                            int64_t row_off, int col0, int ncols, bool live,
                                            int lane, const float (&v)[32]) {
  if (p.c_tma_ok && col0 < ncols && __all_sync(0xffffffffu, live)) {   // warp-uniform
    uint4 w[4];
    pack32_16bit(v, p.c_dtype, w);
    if (SLOTS == 1) {   // single slot: wait until the previous chunk's copy has read it
      if (lane == 0) bulk_wait_read();
      __syncwarp();
    }
    store_rows_tma(stage + (SLOTS == 1 ? 0 : slot) * kOutSlotBytes, w, map_c, col0, tile_row0, lane);
  } else if (p.c_vec_ok && p.c_dtype != BOLT_F32 && col0 + 32 <= ncols) {   // warp-uniform
    uint4 w[4];
    pack32_16bit(v, p.c_dtype, w);
    store_rows_64B(stage, w, static_cast<uint8_t*>(p.c), (row_off + col0) * 2, live, lane);
  } else if (live) {
    store_row32(p.c, p.c_dtype, row_off, col0, ncols, v);
  }
}

struct TileCoord {
  int m_blk, n_blk;
};
__device__ __forceinline__ TileCoord tile_coord(int tile, int num_m, int tiles_n, int group_m) {
  const int per_group = group_m * tiles_n;
  const int grp = tile / per_group;
  const int first_m = grp * group_m;
  const int gm = min(num_m - first_m, group_m);
  const int rem = tile - grp * per_group;
  TileCoord t;
  t.m_blk = first_m + rem % gm;
  t.n_blk = rem / gm;
  return t;
}

// ---------------------------------------------------------------------------
// Kernel
// ---------------------------------------------------------------------------
// ---------------------------------------------------------------------------
// Epilogue arithmetic helpers
// ---------------------------------------------------------------------------
// y[j] = round(silu(round(g[j])) * round(u[j])) for 32 columns; returns max |y|.
template <int MID>
__device__ __forceinline__ float silu_mul32(float (&g)[32], const float (&u)[32]) {
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 32; j += 2) {
    float g0 = g[j], g1 = g[j + 1], u0 = u[j], u1 = u[j + 1];
    round2<MID>(g0, g1);
    round2<MID>(u0, u1);
    float y0 = silu_fast(g0) * u0, y1 = silu_fast(g1) * u1;
    round2<MID>(y0, y1);
    g[j] = y0;
    g[j + 1] = y1;
    amax = fmaxf(amax, fmaxf(fabsf(y0), fabsf(y1)));
  }
  return amax;
}
__device__ __forceinline__ float silu_mul32_dyn(float (&g)[32], const float (&u)[32], int mid) {
  if (mid == BOLT_BF16) return silu_mul32<BOLT_BF16>(g, u);
  if (mid == BOLT_F16) return silu_mul32<BOLT_F16>(g, u);
  return silu_mul32<BOLT_F32>(g, u);
}

// Per-row tile metadata, fetched one tile ahead of its use.
struct RowMeta {
  bool has_tile;
  int expert;
  int sid;
  float rw;
  float a_s;  // channel kinds: row scale
};

// ---------------------------------------------------------------------------
// Kernel
// ---------------------------------------------------------------------------
// Accumulator layout.  A tile has 256 accumulator columns (one M128 x N256 MMA per 32-byte
// K step; TMEM stage t at column 256*t) split into two halves of 128, half h being drained
// by epilogue warps 4+4h .. 7+4h.
//   STORE : half h = output columns 256*n_blk + 128*h + [0,128)   (B rows n0 + 128*h ..)
//   GATED : half h = gate columns [0,64) and up columns [64,128) of output columns
//           128*n_blk + 64*h + [0,64)  (B rows n0+64h.. and N/2+n0+64h..)
// PAIR: two CTAs of a cluster work on two row tiles of one expert and share the weight tile
// (tcgen05 cta_group::2, one 256 x 256 MMA per 32-byte K step issued by the even CTA): each CTA
// stages its own 128 rows of A and HALF of the B tile, and drains its own 128 x 256 accumulator
// exactly as in the single-CTA form.  Bulk tensor loads of both CTAs count on the even CTA's
// "full" barrier; MMA completion is committed to both CTAs' "empty" / "tfull" barriers; the odd
// CTA's epilogue warps release TMEM stages on the even CTA's "tempty" barrier.  No load is
// multicast.
template <int OPK, bool BS, int EPI, bool PAIR>
__global__ void __launch_bounds__(kThreads, 1)
k_grouped_gemm(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
               const __grid_constant__ CUtensorMap tma_c, const GemmParams p) {
  constexpr bool GATED = EPI != BOLT_EPI_STORE;
  constexpr int kBKElems = OPK == OP_F16 ? 64 : 128;
  constexpr bool CHANNEL = (OPK != OP_F16) && !BS;
  constexpr int kStages = PAIR ? pair_stages_of(BS) : stages_of(BS);
  constexpr int kStageStride = PAIR ? kPairStageBytes : kStageBytes;
  constexpr int kSlots = out_slots_of(BS);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint8_t* ctrl = smem + kStages * kStageStride;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ctrl);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ctrl + 256);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(ctrl + 260);
  float* amax_x = reinterpret_cast<float*>(ctrl + 1024);  // [2 tile parities][2 halves][128 rows]
  float* as_ring = reinterpret_cast<float*>(ctrl + 4096); // [kScaleSlots][128 rows]

  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_full = smem_u32(bars);              // [kStages]
  const uint32_t bar_empty = bar_full + 8 * kStages;     // [kStages]
  const uint32_t bar_tfull = bar_empty + 8 * kStages;    // [2 TMEM stages]
  const uint32_t bar_tempty = bar_tfull + 16;            // [2 TMEM stages]
  const uint32_t bar_x = bar_tempty + 16;                // absmax exchange between the halves
  const uint32_t bar_as = bar_x + 8;                     // [kScaleSlots] (pairs): scale rows landed

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // CTA pair: rank 0 issues the MMAs and owns the "full" / "tempty" barriers of the pair
  const uint32_t cta_rank = PAIR ? cluster_ctarank() : 0u;
  // row operand gathered by warps 2 and 3: their 64 threads arrive on "full" beside the producer
  const bool gathered = !PAIR && p.a_gather != 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar_full + 8 * s, gathered ? 65 : 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_tfull + 8 * i, 1);
      mbar_init(bar_tempty + 8 * i, PAIR ? 16 : 8);   // epilogue warps of the CTA / of the pair
    }
    mbar_init(bar_x, 8);
    if (PAIR) {
      for (int i = 0; i < kScaleSlots; ++i) mbar_init(bar_as + 8 * i, 1);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    if (PAIR) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                       smem_u32(tmem_slot)),
                   "r"((uint32_t)kTmemCols)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                       smem_u32(tmem_slot)),
                   "r"((uint32_t)kTmemCols)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();   // the peer's barriers are initialised before anything targets them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // Work list.  Single CTAs: (row tile, column tile) pairs over the valid row tiles.  CTA pairs:
  // (segment, column tile), a segment being at most two row tiles of one expert; CTA `rank`
  // takes row tile `rank` of the segment (rank 1 idles through the MMAs of a one-tile segment).
  const int num_valid = min(*p.num_valid, p.capacity);
  const int num_m = PAIR ? min(max(*p.num_segments, 0), p.max_segments) : num_valid / kBM;
  const int total_tiles = num_m * p.tiles_n;
  const int stride = PAIR ? (int)cluster_count_x() : (int)gridDim.x;
  const int first_tile = PAIR ? (int)cluster_id_x() : (int)blockIdx.x;
  // (row tile, column tile, expert, has a live row tile) of a work item
  auto item_of = [&](int tile, TileCoord& tc, int& expert, bool& has_tile) {
    tc = tile_coord(tile, num_m, p.tiles_n, p.group_m);
    if (PAIR) {
      const int4 sg = *reinterpret_cast<const int4*>(p.segments + 4 * (int64_t)tc.m_blk);
      expert = sg.x;
      has_tile = cta_rank == 0 || sg.z > kBM;
      tc.m_blk = (sg.y >> 7) + (has_tile ? (int)cta_rank : 0);   // an idle CTA mirrors rank 0's rows
    } else {
      expert = p.expert_ids[tc.m_blk];
      has_tile = true;
    }
  };

  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    if (warp == 0) {
      // ------------------------------ TMA producer ------------------------------
      if (PAIR && lane == 0) {
        // Each CTA of the pair stages its own A rows and its half of the B tile (boxes 2*rank,
        // 2*rank+1 of the four 64-row boxes); the bytes of both CTAs are counted on rank 0's
        // barrier, which rank 0 arms for the pair.  Activation scales use a barrier of their own
        // in each CTA.
        int s = 0;
        uint32_t ph = 0, kbi = 0;
        bool ok = true;
        for (int tile = first_tile; ok && tile < total_tiles; tile += stride) {
          TileCoord tc;
          int expert;
          bool has_tile;
          item_of(tile, tc, expert, has_tile);
          if (expert < 0 || expert >= p.num_experts) continue;
          int brow[2];
#pragma unroll
          for (int j2 = 0; j2 < 2; ++j2) {
            const int j = 2 * (int)cta_rank + j2;
            brow[j2] = GATED ? ((j & 1) ? p.n_half : 0) + tc.n_blk * 128 + (j >> 1) * 64
                             : tc.n_blk * 256 + j * 64;
          }
          for (int kb = 0; kb < p.num_kb; ++kb) {
            ok = mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag, p.status, 1);
            if (!ok) break;
            const uint32_t full0 = mapa_shared(bar_full + 8 * s, 0);
            const uint32_t sa = smem_base + s * kStageStride;
            if (cta_rank == 0) mbar_expect_tx(bar_full + 8 * s, 2 * kPairStageBytes);
            if (BS) {
              const uint32_t slot = kbi % kScaleSlots;
              mbar_expect_tx(bar_as + 8 * slot, 512);
              bulk_load(smem_u32(as_ring) + slot * 512,
                        p.a_scale + (int64_t)kb * p.a_scale_ld + tc.m_blk * kBM, 512,
                        bar_as + 8 * slot);
              ++kbi;
            }
            tma_load_2d_pair(sa, &tma_a, full0, kb * kBKElems, tc.m_blk * kBM);
#pragma unroll
            for (int j2 = 0; j2 < 2; ++j2)
              tma_load_3d_pair(sa + kABytes + j2 * (kBBytes / 4), &tma_b, full0, kb * kBKElems,
                               brow[j2], expert);
            if (++s == kStages) { s = 0; ph ^= 1; }
          }
        }
      } else if (lane == 0) {
        int s = 0;
        uint32_t ph = 0, kbi = 0;
        bool ok = true;
        int tile = blockIdx.x;
        int expert_next = -1;
        if (tile < total_tiles)
          expert_next = p.expert_ids[tile_coord(tile, num_m, p.tiles_n, p.group_m).m_blk];
        for (; ok && tile < total_tiles; tile += stride) {
          const TileCoord tc = tile_coord(tile, num_m, p.tiles_n, p.group_m);
          const int expert = expert_next;
          if (tile + stride < total_tiles)
            expert_next = p.expert_ids[tile_coord(tile + stride, num_m, p.tiles_n, p.group_m).m_blk];
          if (expert < 0 || expert >= p.num_experts) continue;
          // B rows of the four 64-row boxes of a stage
          int brow[4];
#pragma unroll
          for (int j = 0; j < 4; ++j)
            brow[j] = GATED ? ((j & 1) ? p.n_half : 0) + tc.n_blk * 128 + (j >> 1) * 64
                            : tc.n_blk * 256 + j * 64;
          for (int kb = 0; kb < p.num_kb; ++kb) {
            ok = mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag, p.status, 1);
            if (!ok) break;
            const uint32_t full = bar_full + 8 * s;
            const uint32_t sa = smem_base + s * kStageBytes;
            mbar_expect_tx(full, (gathered ? kBBytes : kStageBytes) + (BS ? 512 : 0));
            if (BS) {
              // activation scales of this K block for the tile's 128 rows.  Ring slot reuse is
              // safe without a barrier of its own: this copy is issued at most kStages K blocks
              // ahead of the MMA and the MMA runs at most 2 ahead of the epilogue that reads it.
              bulk_load(smem_u32(as_ring) + (kbi % kScaleSlots) * 512,
                        p.a_scale + (int64_t)kb * p.a_scale_ld + tc.m_blk * kBM, 512, full);
              ++kbi;
            }
            if (!gathered) tma_load_2d(sa, &tma_a, full, kb * kBKElems, tc.m_blk * kBM);
#pragma unroll
            for (int j = 0; j < 4; ++j)
              tma_load_3d(sa + kABytes + j * (kBBytes / 4), &tma_b, full, kb * kBKElems, brow[j],
                          expert);
            if (++s == kStages) { s = 0; ph ^= 1; }
          }
        }
      }
    } else if (warp >= 2 && gathered) {
      // ---------------- row operand gathered from token order (warps 2 and 3) ----------------
      // Sorted position p of the tile reads token row sorted_ids[p] & 0xFFFFFF; positions that
      // only pad the tile read nothing and are filled with zeros.  64 threads bring the
      // 128 rows x 128 bytes of a K block with sixteen 16-byte asynchronous copies each (eight
      // neighbouring threads cover one row's 128 bytes), placed where the 128-byte-swizzled box
      // copy would put them: 16-byte column c of row r at r * 128 + ((c ^ (r & 7)) << 4).  The
      // copies of a thread arrive on the stage's "full" barrier when they have landed.
      const int t = (int)threadIdx.x - 64;
      const int c16 = t & 7;
      const int r0 = t >> 3;                                  // rows r0 + 8 i, i = 0..15
      const uint32_t dst0 = (uint32_t)r0 * 128u + (uint32_t)((c16 ^ (r0 & 7)) << 4);
      const uint8_t* abase = static_cast<const uint8_t*>(p.a_base) + c16 * 16;
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += stride) {
        const TileCoord tc = tile_coord(tile, num_m, p.tiles_n, p.group_m);
        const int expert = p.expert_ids[tc.m_blk];
        if (expert < 0 || expert >= p.num_experts) continue;
        int roff[16];                          // row offset in 16-byte units, -1 = padding
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int tok = p.sorted_ids[(int64_t)tc.m_blk * kBM + r0 + 8 * i] & 0xFFFFFF;
          roff[i] = tok < p.num_tokens ? tok * p.a_row_units : -1;
        }
        for (int kb = 0; kb < p.num_kb; ++kb) {
          ok = mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag, p.status, 5);
          if (!ok) break;
          const uint32_t sa = smem_base + s * kStageBytes + dst0;
          const int kbyte = kb * 128 + c16 * 16;
          const bool in_k = kbyte < p.k_bytes;                // reduction tail: zeros
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const bool live = in_k && roff[i] >= 0;
            cp_async_16(sa + i * 1024, abase + (live ? (int64_t)roff[i] * 16 + kb * 128 : 0),
                        live ? 16u : 0u);
          }
          cp_async_mbar_arrive_noinc(bar_full + 8 * s);
          if (++s == kStages) { s = 0; ph ^= 1; }
        }
      }
      cp_async_wait_all();
    } else if (warp == 1) {
      // ------------------------------ MMA issuer --------------------------------
      if (PAIR && lane == 0 && cta_rank == 0) {
        // one thread of the even CTA issues the 256-row MMAs of the pair and commits their
        // completion to the barriers of both CTAs
        int s = 0, t = 0;
        uint32_t ph = 0, tph = 0;
        bool ok = true;
        for (int tile = first_tile; ok && tile < total_tiles; tile += stride) {
          TileCoord tc;
          int expert;
          bool has_tile;
          item_of(tile, tc, expert, has_tile);
          if (expert < 0 || expert >= p.num_experts) continue;
          for (int kb = 0; kb < p.num_kb; ++kb) {
            if (BS || kb == 0) {
              ok = mbar_wait(bar_tempty + 8 * t, tph ^ 1, abort_flag, p.status, 2);
              if (!ok) break;
            }
            ok = mbar_wait(bar_full + 8 * s, ph, abort_flag, p.status, 3);
            if (!ok) break;
            tc_fence_after();
            const uint32_t sa = smem_base + s * kStageStride;
            const uint64_t adesc = make_smem_desc(sa);
            const uint64_t bdesc = make_smem_desc(sa + kABytes);
            const uint32_t d = tmem_base + t * kAccCols;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const uint32_t accum = BS ? (k > 0) : (kb > 0 || k > 0);
              tc_mma_pair<OPK>(d, adesc + 2 * k, bdesc + 2 * k, p.idesc, accum);
            }
            tc_commit_pair(bar_empty + 8 * s);
            if (++s == kStages) { s = 0; ph ^= 1; }
            if (BS) {
              tc_commit_pair(bar_tfull + 8 * t);
              if (++t == 2) { t = 0; tph ^= 1; }
            }
          }
          if (!BS && ok) {
            tc_commit_pair(bar_tfull + 8 * t);
            if (++t == 2) { t = 0; tph ^= 1; }
          }
        }
      } else if (!PAIR && lane == 0) {
        int s = 0, t = 0;
        uint32_t ph = 0, tph = 0;
        bool ok = true;
        int tile = blockIdx.x;
        int expert_next = -1;
        if (tile < total_tiles)
          expert_next = p.expert_ids[tile_coord(tile, num_m, p.tiles_n, p.group_m).m_blk];
        for (; ok && tile < total_tiles; tile += stride) {
          const int expert = expert_next;
          if (tile + stride < total_tiles)
            expert_next = p.expert_ids[tile_coord(tile + stride, num_m, p.tiles_n, p.group_m).m_blk];
          if (expert < 0 || expert >= p.num_experts) continue;
          for (int kb = 0; kb < p.num_kb; ++kb) {
            if (BS || kb == 0) {
              ok = mbar_wait(bar_tempty + 8 * t, tph ^ 1, abort_flag, p.status, 2);
              if (!ok) break;
            }
            ok = mbar_wait(bar_full + 8 * s, ph, abort_flag, p.status, 3);
            if (!ok) break;
            tc_fence_after();
            // gathered rows were written through the generic proxy, the MMA reads through the
            // asynchronous one
            if (gathered) fence_async_smem();
            const uint32_t sa = smem_base + s * kStageBytes;
            const uint64_t adesc = make_smem_desc(sa);
            const uint64_t bdesc = make_smem_desc(sa + kABytes);
            const uint32_t d = tmem_base + t * kAccCols;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const uint32_t accum = BS ? (k > 0) : (kb > 0 || k > 0);
              tc_mma<OPK>(d, adesc + 2 * k, bdesc + 2 * k, p.idesc, accum);
            }
            tc_commit(bar_empty + 8 * s);
            if (++s == kStages) { s = 0; ph ^= 1; }
            if (BS) {
              tc_commit(bar_tfull + 8 * t);
              if (++t == 2) { t = 0; tph ^= 1; }
            }
          }
          if (!BS && ok) {
            tc_commit(bar_tfull + 8 * t);
            if (++t == 2) { t = 0; tph ^= 1; }
          }
        }
      }
    }
  } else {
    // ------------------------------ epilogue -----------------------------------
    asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
    const int q = warp & 3;            // TMEM lane quarter
    const int h = (warp - 4) >> 2;     // accumulator half owned by this warp
    const int row_in_tile = 32 * q + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(32 * q) << 16) + h * kHalfCols;
    const bool has_ids = p.sorted_ids != nullptr;
    const bool has_rw = p.mul_routed_weight && p.sorted_weights != nullptr;
    uint8_t* out_stage = ctrl + 4096 + kScaleSlots * 512 + (warp - 4) * out_stage_bytes_of(BS);
    int t = 0;
    uint32_t tph = 0, xph = 0, kbi = 0;
    bool ok = true;

    // coordinates and per-row metadata of a work item (an idle CTA of a pair mirrors rank 0's
    // rows and stores nothing)
    auto fetch_meta = [&](int tile_index, TileCoord& c) {
      RowMeta m;
      item_of(tile_index, c, m.expert, m.has_tile);
      const int r = c.m_blk * kBM + row_in_tile;
      m.sid = has_ids ? p.sorted_ids[r] : 0;
      m.rw = has_rw ? p.sorted_weights[r] : 1.0f;
      m.a_s = CHANNEL ? p.a_scale[r] : 1.0f;
      return m;
    };
    // hand a TMEM stage back to the MMA issuer (of the pair: the even CTA's barrier)
    auto release_tmem = [&](int stage) {
      if (PAIR && cta_rank != 0) mbar_arrive_cluster(mapa_shared(bar_tempty + 8 * stage, 0));
      else mbar_arrive(bar_tempty + 8 * stage);
    };
    // b-scale row pointers of a tile (block-scaled kinds)
    auto bscale_ptrs = [&](int expert, int n_blk, const float*& b0, const float*& b1) {
      const int nb0 = GATED ? n_blk : min(2 * n_blk + h, p.n / 128 - 1);
      const int nb1 = GATED ? p.n_half / 128 + n_blk : nb0;
      b0 = p.b_scale + ((int64_t)expert * (p.n / 128) + nb0) * p.kb_scale_cols;
      b1 = p.b_scale + ((int64_t)expert * (p.n / 128) + nb1) * p.kb_scale_cols;
    };

    int tile = first_tile;
    TileCoord tc_next{0, 0};
    RowMeta next{};
    float b0_first = 0.f, b1_first = 0.f;  // b scales of K block 0 of the next tile
    if (tile < total_tiles) {
      next = fetch_meta(tile, tc_next);
      if (BS && next.expert >= 0 && next.expert < p.num_experts) {
        const float *b0, *b1;
        bscale_ptrs(next.expert, tc_next.n_blk, b0, b1);
        b0_first = __ldg(b0);
        b1_first = __ldg(b1);
      }
    }
    for (; ok && tile < total_tiles; tile += stride) {
      const TileCoord tc = tc_next;
      const RowMeta cur = next;
      const bool more = tile + stride < total_tiles;
      if (more) next = fetch_meta(tile + stride, tc_next);
      const int expert = cur.expert;
      if (expert < 0 || expert >= p.num_experts) {
        if (BS && more && next.expert >= 0 && next.expert < p.num_experts) {
          const float *b0, *b1;
          bscale_ptrs(next.expert, tc_next.n_blk, b0, b1);
          b0_first = __ldg(b0);
          b1_first = __ldg(b1);
        }
        continue;
      }
      const int row = tc.m_blk * kBM + row_in_tile;
      const int tile_row0 = tc.m_blk * kBM + 32 * q;   // output row of lane 0 (sorted layout)
      const int token = cur.sid & 0xFFFFFF;
      const bool live = token < p.num_tokens && cur.has_tile;
      // Gated epilogues feed the next GEMM: padding rows are written as zeros rather than left
      // as stale memory, because operand rows full of arbitrary bits cost tensor-core power
      // (and with it SM clock) in the GEMM that streams them.
      const bool wr = cur.has_tile && (live || (GATED && !p.scatter));
      const float rw = cur.rw;
      int64_t out_row = row;
      int64_t seg_off = 0;
      if (p.scatter) {
        int src = token;
        if (p.scatter_src != nullptr && live) {
          src = p.scatter_src[token];
          seg_off = p.scatter_seg_off[token / p.scatter_seg_rows];
        }
        out_row = (int64_t)src * p.topk + ((uint32_t)cur.sid >> 24);
      }
      const int64_t row_off = seg_off + out_row * p.c_ld;
      const int64_t brow = (int64_t)expert * p.n;  // first bias / channel-scale entry of the expert
      // first output column of this thread's half
      const int ocol = GATED ? tc.n_blk * 128 + 64 * h : tc.n_blk * 256 + 128 * h;

      if (!BS) {
        ok = mbar_wait(bar_tfull + 8 * t, tph, abort_flag, p.status, 4);
        if (!ok) break;
        tc_fence_after();
        if (lane == 0) bulk_wait_read();   // the previous tile's bulk stores have left the slots
        __syncwarp();
        const uint32_t tbase = lane_addr + t * kAccCols;
        const float a_s = cur.a_s;
        if (!GATED) {
          const int ncols = p.n;
#pragma unroll 1
          for (int i = 0; i < 4; ++i) {
            uint32_t raw[32];
            tmem_ld32(tbase + 32 * i, raw);
            tmem_ld_wait();
            const int col0 = ocol + 32 * i;
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = acc_to_f32<OPK>(raw[j]);
            if (CHANNEL) {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                v[j] = v[j] * a_s * __ldg(p.b_scale + brow + min(col0 + j, ncols - 1));
            }
            if (p.bias) {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                v[j] += load_bias(p.bias, p.bias_dtype, brow + min(col0 + j, ncols - 1));
            }
            if (has_rw) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] *= rw;
            }
            store_chunk<kSlots>(out_stage, i, p, &tma_c, tile_row0, row_off, col0, ncols, live, lane, v);
          }
        } else {
#pragma unroll 1
          for (int i = 0; i < 2; ++i) {
            uint32_t rg[32], ru[32];
            tmem_ld32(tbase + 32 * i, rg);
            tmem_ld32(tbase + 64 + 32 * i, ru);
            tmem_ld_wait();
            const int col0 = ocol + 32 * i;
            float g[32], u[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              g[j] = live ? acc_to_f32<OPK>(rg[j]) : 0.f;
              u[j] = live ? acc_to_f32<OPK>(ru[j]) : 0.f;
            }
            if (CHANNEL) {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const int col = min(col0 + j, p.n_half - 1);
                g[j] = g[j] * a_s * __ldg(p.b_scale + brow + col);
                u[j] = u[j] * a_s * __ldg(p.b_scale + brow + p.n_half + col);
              }
            }
            if (p.bias) {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const int col = min(col0 + j, p.n_half - 1);
                g[j] += load_bias(p.bias, p.bias_dtype, brow + col);
                u[j] += load_bias(p.bias, p.bias_dtype, brow + p.n_half + col);
              }
            }
            if (has_rw) {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                g[j] *= rw;
                u[j] *= rw;
              }
            }
            silu_mul32_dyn(g, u, p.mid_dtype);
            store_chunk<kSlots>(out_stage, i, p, &tma_c, tile_row0, row_off, col0, p.n_half, wr, lane, g);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) release_tmem(t);
        if (++t == 2) { t = 0; tph ^= 1; }
      } else {
        // ---- block-scaled: promote every K block into fp32 registers ----
        // acc[i] = 32 columns as 16 packed pairs; chunks 0,1 scale with b0, chunks 2,3 with b1
        float2 acc[4][16];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 16; ++j) acc[i][j] = make_float2(0.f, 0.f);
        const float *bs0, *bs1;
        bscale_ptrs(expert, tc.n_blk, bs0, bs1);
        float b0_next = b0_first, b1_next = b1_first;
        // Software-pipelined promotion: 32-column loads, two staging buffers, one load always in
        // flight while the previous chunk is being accumulated; the first chunk of the next K
        // block is requested before the last chunk of this one is consumed.
        auto fma_chunk = [&](float2 (&a)[16], const uint32_t (&r)[32], float sc) {
          const float2 sc2 = make_float2(sc, sc);
#pragma unroll
          for (int j = 0; j < 16; ++j)
            a[j] = __ffma2_rn(
                make_float2(acc_to_f32<OPK>(r[2 * j]), acc_to_f32<OPK>(r[2 * j + 1])), sc2, a[j]);
        };
        uint32_t ra[32], rb[32];
        ok = mbar_wait(bar_tfull + 8 * t, tph, abort_flag, p.status, 4);
        if (!ok) break;
        tc_fence_after();
        tmem_ld32(lane_addr + t * kAccCols, ra);
        for (int kb = 0; kb < p.num_kb; ++kb) {
          const float b0_cur = b0_next, b1_cur = b1_next;
          if (kb + 1 < p.num_kb) {
            b0_next = __ldg(bs0 + kb + 1);
            b1_next = __ldg(bs1 + kb + 1);
          }
          if (kb == (p.num_kb > 1 ? 1 : 0) && more && next.expert >= 0 &&
              next.expert < p.num_experts) {
            const float *n0, *n1;
            bscale_ptrs(next.expert, tc_next.n_blk, n0, n1);
            b0_first = __ldg(n0);
            b1_first = __ldg(n1);
          }
          // this K block's completion was observed before its first load was issued; the scale
          // row travelled with the operand stage (pairs: on a barrier of its own)
          if (PAIR) {
            ok = mbar_wait(bar_as + 8 * (kbi % kScaleSlots), (kbi / kScaleSlots) & 1u, abort_flag,
                           p.status, 6);
            if (!ok) break;
          }
          const float a_s = as_ring[(kbi % kScaleSlots) * 128 + row_in_tile];
          ++kbi;
          const float s0 = a_s * b0_cur;
          const float s1 = GATED ? a_s * b1_cur : s0;
          const uint32_t tbase = lane_addr + t * kAccCols;
          tmem_ld_wait();
          tmem_ld32(tbase + 32, rb);
          fma_chunk(acc[0], ra, s0);
          tmem_ld_wait();
          tmem_ld32(tbase + 64, ra);
          fma_chunk(acc[1], rb, s0);
          tmem_ld_wait();
          tmem_ld32(tbase + 96, rb);
          fma_chunk(acc[2], ra, s1);
          tmem_ld_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) release_tmem(t);
          if (++t == 2) { t = 0; tph ^= 1; }
          if (kb + 1 < p.num_kb) {
            ok = mbar_wait(bar_tfull + 8 * t, tph, abort_flag, p.status, 4);
            if (!ok) break;
            tc_fence_after();
            tmem_ld32(lane_addr + t * kAccCols, ra);
          }
          fma_chunk(acc[3], rb, s1);
        }
        if (!ok) break;
        // ---- finalise ----
        if (lane == 0) bulk_wait_read();   // the previous tile's bulk stores have left the slots
        __syncwarp();
        // scattered 16-bit rows whose 128 columns are all inside the matrix leave as whole
        // 256-byte segments (warp-uniform)
        const bool wide_rows = !GATED && kSlots == 4 && p.scatter && p.c_vec_ok &&
                               p.c_dtype != BOLT_F32 && ocol + 128 <= p.n;
        float v[4][32];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            v[i][2 * j] = acc[i][j].x;
            v[i][2 * j + 1] = acc[i][j].y;
          }
        if (!GATED) {
          const int ncols = p.n;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int col0 = ocol + 32 * i;
            if (p.bias) {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                v[i][j] += load_bias(p.bias, p.bias_dtype, brow + min(col0 + j, ncols - 1));
            }
            if (has_rw) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[i][j] *= rw;
            }
            if (!wide_rows)
              store_chunk<kSlots>(out_stage, i, p, &tma_c, tile_row0, row_off, col0, ncols, live, lane, v[i]);
          }
          if (wide_rows)
            store_rows_256B(out_stage, v, p.c_dtype, static_cast<uint8_t*>(p.c), (row_off + ocol) * 2,
                            live, lane);
        } else {
          // chunks 0,1 = gate, chunks 2,3 = up of output columns ocol + [0,64)
          float amax = 0.f;
          if (!live) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
              for (int j = 0; j < 32; ++j) v[i][j] = 0.f;
          }
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            const int col0 = ocol + 32 * i;
            if (p.bias) {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const int col = min(col0 + j, p.n_half - 1);
                v[i][j] += load_bias(p.bias, p.bias_dtype, brow + col);
                v[2 + i][j] += load_bias(p.bias, p.bias_dtype, brow + p.n_half + col);
              }
            }
            if (has_rw) {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                v[i][j] *= rw;
                v[2 + i][j] *= rw;
              }
            }
            amax = fmaxf(amax, silu_mul32_dyn(v[i], v[2 + i], p.mid_dtype));
          }
          if (EPI == BOLT_EPI_SILU_MUL) {
#pragma unroll
            for (int i = 0; i < 2; ++i)
              store_chunk<kSlots>(out_stage, i, p, &tma_c, tile_row0, row_off, ocol + 32 * i, p.n_half, wr,
                          lane, v[i]);
          } else {
            // 1x128 group quantisation: the two halves exchange their absmax through shared
            // memory (double-buffered by tile parity; the barrier wait is bounded)
            float* xbuf = amax_x + xph * 256;
            xbuf[h * 128 + row_in_tile] = amax;
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_x);
            ok = mbar_wait(bar_x, xph, abort_flag, p.status, 5);
            if (!ok) break;
            amax = fmaxf(amax, xbuf[(h ^ 1) * 128 + row_in_tile]);
            xph ^= 1;
            const bool to_i8 = p.c_dtype == BOLT_INT8;
            const float scale = __fdiv_rn(fmaxf(amax, 1.0e-10f), to_i8 ? 127.0f : 448.0f);
            const float inv = __frcp_rn(scale);
            {
              uint4 wq[4];
#pragma unroll
              for (int i = 0; i < 2; ++i) {
                uint32_t w[8];
                if (!to_i8) {
#pragma unroll
                  for (int j = 0; j < 8; ++j) {
                    const uint32_t lo = __nv_cvt_float2_to_fp8x2(
                        make_float2(v[i][4 * j] * inv, v[i][4 * j + 1] * inv), __NV_SATFINITE,
                        __NV_E4M3);
                    const uint32_t hi = __nv_cvt_float2_to_fp8x2(
                        make_float2(v[i][4 * j + 2] * inv, v[i][4 * j + 3] * inv), __NV_SATFINITE,
                        __NV_E4M3);
                    w[j] = lo | (hi << 16);
                  }
                } else {
#pragma unroll
                  for (int j = 0; j < 8; ++j) {
                    uint32_t x = 0;
#pragma unroll
                    for (int b = 0; b < 4; ++b)
                      x |= (uint32_t)(uint8_t)f32_to_i8(v[i][4 * j + b] * inv) << (8 * b);
                    w[j] = x;
                  }
                }
                wq[2 * i] = make_uint4(w[0], w[1], w[2], w[3]);
                wq[2 * i + 1] = make_uint4(w[4], w[5], w[6], w[7]);
              }
              // 64 one-byte outputs = one 64-byte row segment: the warp's 32 x 64 B block leaves
              // by one bulk tensor store (a per-thread store touches 32 different lines per
              // instruction); without a tensor map the segment is written directly
              if (p.c_tma_ok && cur.has_tile) {
                store_rows_tma(out_stage, wq, &tma_c, ocol, tile_row0, lane);
              } else if (wr && !p.c_tma_ok) {
                uint4* dst = reinterpret_cast<uint4*>(static_cast<uint8_t*>(p.c) + row_off + ocol);
#pragma unroll
                for (int j = 0; j < 4; ++j) dst[j] = wq[j];
              }
            }
            if (wr) {
              if (h == 0) p.c_scale[(int64_t)tc.n_blk * p.c_scale_ld + row] = live ? scale : 0.f;
            }
          }
        }
      }
    }
  }

  // ------------------------------ teardown ------------------------------------
  if (warp >= 4 && lane == 0) bulk_wait_all();   // bulk stores of this warp's last blocks
  __syncwarp();
  if (*abort_flag) {
    // let bulk copies that are still in flight land before the CTA's memory is released
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();   // the peer may still signal this CTA's barriers or read its tiles
  tc_fence_after();
  if (warp == 1) {
    if (PAIR)
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                   "r"((uint32_t)kTmemCols)
                   : "memory");
    else
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                   "r"((uint32_t)kTmemCols)
                   : "memory");
  }
}

// ---------------------------------------------------------------------------
// MX (microscaled e4m3) grouped GEMM
// ---------------------------------------------------------------------------
// Same tiles, roles and operand pipeline as above, but the 1 x 32 E8M0 scales are applied by the
// tensor core (kind::mxf8f6f4.block_scale): the accumulator stays in TMEM over the whole K loop
// and nothing is promoted in registers.  Scale bytes travel in 512-byte tiles of 128 rows x 4 K
// groups, byte (r % 32) * 16 + (r / 32) * 4 + g for row r and group g: one bulk copy per tile and
// K block into a shared-memory ring, one tcgen05.cp into four TMEM columns.  TMEM: columns
// [0,256) accumulator, [256,260) A scales, [260,268) B scales of the current K block (copies and
// MMAs of one thread execute in order, so the scale columns are reused every K block).  One
// accumulator stage: the epilogue of a tile is not overlapped with the next tile's MMAs.
constexpr int kMxStages = 4;
constexpr int kMxSfSlots = 6;             // >= operand stages + 1
constexpr int kMxSfSlotBytes = 512 * 3;   // A scales + two 128-row blocks of B scales
constexpr int kMxSmemBytes = kMxStages * kStageBytes + 4096 + kMxSfSlots * kMxSfSlotBytes +
                             8 * 2560 + 1024;

//
// GATED: B rows are loaded as [gate n0.., up n0.., gate n0+64.., up n0+64..] (64 each) so that a
// thread holds 32 gate columns and their 32 up columns; the epilogue rounds both through
// mid_dtype, applies min(g,L) * sigmoid(alpha g) * (clamp(u,+-L) + beta) in fp32 and quantises
// the 32 results - exactly one MX group - to e4m3 codes and one exponent byte, all in registers.
template <bool GATED>
__global__ void __launch_bounds__(kThreads, 1)
k_mx_gemm(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
          const __grid_constant__ CUtensorMap tma_c, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint8_t* ctrl = smem + kMxStages * kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ctrl);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ctrl + 256);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(ctrl + 260);
  uint8_t* sf_ring = ctrl + 4096;

  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = bar_full + 8 * kMxStages;
  const uint32_t bar_tfull = bar_empty + 8 * kMxStages;
  const uint32_t bar_tempty = bar_tfull + 8;
  const uint32_t bar_x = bar_tempty + 8;                      // [4 lane quarters]: absmax exchange
  float* amax_x = reinterpret_cast<float*>(ctrl + 1024);      // [2 tile parities][2 halves][128 rows]
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kMxStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    mbar_init(bar_tfull, 1);
    mbar_init(bar_tempty, 8);
    for (int i = 0; i < 4; ++i) mbar_init(bar_x + 8 * i, 2);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"((uint32_t)kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int num_valid = min(*p.num_valid, p.capacity);
  const int num_m = num_valid / kBM;
  const int total_tiles = num_m * p.tiles_n;
  const int stride = gridDim.x;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0, kbi = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += stride) {
        const TileCoord tc = tile_coord(tile, num_m, p.tiles_n, p.group_m);
        const int expert = p.expert_ids[tc.m_blk];
        if (expert < 0 || expert >= p.num_experts) continue;
        const int nb0 = min(2 * tc.n_blk, p.n_blocks128 - 1);
        const int nb1 = min(2 * tc.n_blk + 1, p.n_blocks128 - 1);
        const uint8_t* sfa_t = p.sfa + (int64_t)tc.m_blk * p.num_kb * 512;
        const uint8_t* sfb0 = p.sfb + ((int64_t)expert * p.n_blocks128 + nb0) * p.num_kb * 512;
        const uint8_t* sfb1 = p.sfb + ((int64_t)expert * p.n_blocks128 + nb1) * p.num_kb * 512;
        for (int kb = 0; kb < p.num_kb; ++kb) {
          ok = mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag, p.status, 1);
          if (!ok) break;
          const uint32_t full = bar_full + 8 * s;
          const uint32_t sa = smem_base + s * kStageBytes;
          const uint32_t sf = smem_u32(sf_ring) + (kbi % kMxSfSlots) * kMxSfSlotBytes;
          ++kbi;
          mbar_expect_tx(full, p.mx_stage_tx + kMxSfSlotBytes);
          bulk_load(sf, sfa_t + (int64_t)kb * 512, 512, full);
          bulk_load(sf + 512, sfb0 + (int64_t)kb * 512, 512, full);
          bulk_load(sf + 1024, sfb1 + (int64_t)kb * 512, 512, full);
          tma_load_2d(sa, &tma_a, full, kb * 128, tc.m_blk * kBM);
#pragma unroll
          for (int j = 0; j < 4; ++j)
            tma_load_3d(sa + kABytes + j * (kBBytes / 4), &tma_b, full, kb * 128,
                        GATED ? ((j & 1) ? p.n_half : 0) + tc.n_blk * 128 + (j >> 1) * 64
                              : tc.n_blk * 256 + j * 64,
                        expert);
          if (++s == kMxStages) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0, tph = 0, kbi = 0;
      bool ok = true;
      const uint32_t sfa_t = tmem_base + 256, sfb_t = tmem_base + 260;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += stride) {
        const TileCoord tc = tile_coord(tile, num_m, p.tiles_n, p.group_m);
        const int expert = p.expert_ids[tc.m_blk];
        if (expert < 0 || expert >= p.num_experts) continue;
        ok = mbar_wait(bar_tempty, tph ^ 1, abort_flag, p.status, 2);
        if (!ok) break;
        for (int kb = 0; kb < p.num_kb; ++kb) {
          ok = mbar_wait(bar_full + 8 * s, ph, abort_flag, p.status, 3);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = smem_base + s * kStageBytes;
          const uint32_t sf = smem_u32(sf_ring) + (kbi % kMxSfSlots) * kMxSfSlotBytes;
          ++kbi;
          tc_cp_sf(sfa_t, make_sf_desc(sf));
          tc_cp_sf(sfb_t, make_sf_desc(sf + 512));
          tc_cp_sf(sfb_t + 4, make_sf_desc(sf + 1024));
          const uint64_t adesc = make_smem_desc(sa);
          const uint64_t bdesc = make_smem_desc(sa + kABytes);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            tc_mma_mx(tmem_base, adesc + 2 * k, bdesc + 2 * k,
                      p.idesc | ((uint32_t)k << 4) | ((uint32_t)k << 29), sfa_t, sfb_t,
                      (kb > 0 || k > 0) ? 1u : 0u);
          tc_commit(bar_empty + 8 * s);
          if (++s == kMxStages) { s = 0; ph ^= 1; }
        }
        if (ok) tc_commit(bar_tfull);
        tph ^= 1;
      }
    }
  } else if (warp >= 4) {
    // ------------------------------ epilogue -----------------------------------
    const int q = warp & 3;
    const int h = (warp - 4) >> 2;
    const int row_in_tile = 32 * q + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(32 * q) << 16) + h * kHalfCols;
    const bool has_ids = p.sorted_ids != nullptr;
    const bool has_rw = p.mul_routed_weight && p.sorted_weights != nullptr;
    uint8_t* out_stage = ctrl + 4096 + kMxSfSlots * kMxSfSlotBytes + (warp - 4) * 2560;
    uint32_t tph = 0, xph = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < total_tiles; tile += stride) {
      const TileCoord tc = tile_coord(tile, num_m, p.tiles_n, p.group_m);
      const int expert = p.expert_ids[tc.m_blk];
      if (expert < 0 || expert >= p.num_experts) continue;
      const int row = tc.m_blk * kBM + row_in_tile;
      const int tile_row0 = tc.m_blk * kBM + 32 * q;
      const int sid = has_ids ? p.sorted_ids[row] : 0;
      const float rw = has_rw ? p.sorted_weights[row] : 1.0f;
      const int token = sid & 0xFFFFFF;
      const bool live = token < p.num_tokens;
      int64_t out_row = row;
      if (p.scatter) out_row = (int64_t)token * p.topk + ((uint32_t)sid >> 24);
      const int64_t row_off = out_row * p.c_ld;
      const int ocol = tc.n_blk * 256 + 128 * h;
      ok = mbar_wait(bar_tfull, tph, abort_flag, p.status, 4);
      if (!ok) break;
      tph ^= 1;
      tc_fence_after();
      if (lane == 0) bulk_wait_read();
      __syncwarp();
      // With one accumulator stage the next tile's MMAs wait for this epilogue, so each warp
      // first copies its 128 columns to registers, hands the accumulator back, and only then
      // converts and stores.
      uint32_t raw[4][32];
#pragma unroll
      for (int i = 0; i < 4; ++i) tmem_ld32(lane_addr + 32 * i, raw[i]);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tempty);
      if (!GATED) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(raw[i][j]);
          if (has_rw) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] *= rw;
          }
          store_chunk<1>(out_stage, 0, p, &tma_c, tile_row0, row_off, ocol + 32 * i, p.n, live,
                         lane, v);
        }
      } else if (p.mx_group128) {
        // The w4a8 recipe between its GEMMs (boltops/fused_moe/triton/mxfp4_quant.py:38-56 of the
        // reference project): both operands rounded through mid_dtype, gate <= L, |up| <= L,
        // y = bf16(up * gate / (1 + exp(-gate))), then ONE power-of-two scale per 1 x 128 group:
        // the smallest 2^k >= max(amax, 1e-10) / 448 (not below 1e-10), codes e4m3(y / scale).
        // A tile's 128 output columns are exactly one group; this thread holds 64 of them (half
        // h), the thread of the same row in the other half the rest: the two exchange their
        // absmax through shared memory (bounded barrier per lane quarter).
        const int ocol_g = tc.n_blk * 128 + 64 * h;
        uint8_t* c8 = static_cast<uint8_t*>(p.c) + row * (int64_t)p.c_ld + ocol_g;
        uint8_t* s8 = reinterpret_cast<uint8_t*>(p.c_scale) + row * p.c_scale_ld + ocol_g / 32;
        float y[64];
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            float g0 = __uint_as_float(raw[i][j]), g1 = __uint_as_float(raw[i][j + 1]);
            float u0 = __uint_as_float(raw[2 + i][j]), u1 = __uint_as_float(raw[2 + i][j + 1]);
            if (p.mid_dtype == BOLT_BF16) {
              round2<BOLT_BF16>(g0, g1);
              round2<BOLT_BF16>(u0, u1);
            } else if (p.mid_dtype == BOLT_F16) {
              round2<BOLT_F16>(g0, g1);
              round2<BOLT_F16>(u0, u1);
            }
            if (p.act_has_limit) {
              g0 = fminf(g0, p.act_limit);
              g1 = fminf(g1, p.act_limit);
              u0 = fminf(fmaxf(u0, -p.act_limit), p.act_limit);
              u1 = fminf(fmaxf(u1, -p.act_limit), p.act_limit);
            }
            float y0 = __fdiv_rn(u0 * g0, 1.0f + expf(-g0));
            float y1 = __fdiv_rn(u1 * g1, 1.0f + expf(-g1));
            round2<BOLT_BF16>(y0, y1);
            if (!live) y0 = y1 = 0.f;
            y[32 * i + j] = y0;
            y[32 * i + j + 1] = y1;
            amax = fmaxf(amax, fmaxf(fabsf(y0), fabsf(y1)));
          }
        }
        const int par = (int)(xph & 1u);
        amax_x[(par * 2 + h) * 128 + row_in_tile] = amax;
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_x + 8 * q);
        ok = mbar_wait(bar_x + 8 * q, xph & 1u, abort_flag, p.status, 6);
        if (!ok) break;
        ++xph;
        amax = fmaxf(amax, amax_x[(par * 2 + (h ^ 1)) * 128 + row_in_tile]);
        const float rawsc = fmaxf(__fdiv_rn(fmaxf(amax, 1.0e-10f), 448.0f), 1.0e-10f);
        const uint32_t bits = __float_as_uint(rawsc);
        const uint32_t e = ((bits >> 23) & 255u) + ((bits & 0x7fffffu) != 0u ? 1u : 0u);
        const float inv = __fdiv_rn(1.0f, __uint_as_float(e << 23));
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          uint32_t w[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float v[4];
#pragma unroll
            for (int t = 0; t < 4; ++t)
              v[t] = fminf(fmaxf(y[32 * i + 4 * j + t] * inv, -448.0f), 448.0f);
            const uint32_t lo =
                __nv_cvt_float2_to_fp8x2(make_float2(v[0], v[1]), __NV_SATFINITE, __NV_E4M3);
            const uint32_t hi =
                __nv_cvt_float2_to_fp8x2(make_float2(v[2], v[3]), __NV_SATFINITE, __NV_E4M3);
            w[j] = lo | (hi << 16);
          }
          uint4* dst = reinterpret_cast<uint4*>(c8 + 32 * i);
          dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
          dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
          s8[i] = live ? (uint8_t)e : (uint8_t)0;
        }
      } else {
        // half h: columns [0,64) gate and [64,128) up of output columns 128 n_blk + 64 h + [0,64)
        const int ocol_g = tc.n_blk * 128 + 64 * h;
        uint8_t* c8 = static_cast<uint8_t*>(p.c) + row * (int64_t)p.c_ld + ocol_g;
        uint8_t* s8 = reinterpret_cast<uint8_t*>(p.c_scale) + row * p.c_scale_ld + ocol_g / 32;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const uint32_t(&rg)[32] = raw[i];
          const uint32_t(&ru)[32] = raw[2 + i];
          float v[32];
          float amax = 0.f;
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            float g0 = __uint_as_float(rg[j]), g1 = __uint_as_float(rg[j + 1]);
            float u0 = __uint_as_float(ru[j]), u1 = __uint_as_float(ru[j + 1]);
            if (p.mid_dtype == BOLT_BF16) {
              round2<BOLT_BF16>(g0, g1);
              round2<BOLT_BF16>(u0, u1);
            } else if (p.mid_dtype == BOLT_F16) {
              round2<BOLT_F16>(g0, g1);
              round2<BOLT_F16>(u0, u1);
            }
            if (p.act_has_limit) {
              g0 = fminf(g0, p.act_limit);
              g1 = fminf(g1, p.act_limit);
              u0 = fminf(fmaxf(u0, -p.act_limit), p.act_limit);
              u1 = fminf(fmaxf(u1, -p.act_limit), p.act_limit);
            }
            v[j] = g0 * __frcp_rn(1.0f + expf(-p.act_alpha * g0)) * (u0 + p.act_beta);
            v[j + 1] = g1 * __frcp_rn(1.0f + expf(-p.act_alpha * g1)) * (u1 + p.act_beta);
            if (!live) v[j] = v[j + 1] = 0.f;
            amax = fmaxf(amax, fmaxf(fabsf(v[j]), fabsf(v[j + 1])));
          }
          amax = fmaxf(amax, 1.1754943508222875e-38f);
          const float e =
              fminf(fmaxf(ceilf(log2f(__fdiv_rn(amax, 448.0f))) + 127.0f, 0.0f), 254.0f);
          const float down = exp2f(127.0f - e);
          uint32_t w[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const uint32_t lo = __nv_cvt_float2_to_fp8x2(
                make_float2(v[4 * j] * down, v[4 * j + 1] * down), __NV_SATFINITE, __NV_E4M3);
            const uint32_t hi = __nv_cvt_float2_to_fp8x2(
                make_float2(v[4 * j + 2] * down, v[4 * j + 3] * down), __NV_SATFINITE, __NV_E4M3);
            w[j] = lo | (hi << 16);
          }
          // padding rows are written too (zeros, exponent byte 0): the next GEMM streams them
          uint4* dst = reinterpret_cast<uint4*>(c8 + 32 * i);
          dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
          dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
          s8[i] = live ? (uint8_t)(int)e : (uint8_t)0;
        }
      }
    }
  }

  // ------------------------------ teardown ------------------------------------
  if (warp >= 4 && lane == 0) bulk_wait_all();
  __syncwarp();
  if (*abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"((uint32_t)kTmemCols)
                 : "memory");
  }
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// One-time set-up of a kernel on the CURRENT device (`done` has one slot per device ordinal):
// the dynamic shared-memory opt-in is a per-device attribute, and a kernel that re-splits its
// registers with setmaxnreg must have been compiled to a register count from which the split
// balances -- `setmaxnreg.inc` only gets registers that `setmaxnreg.dec` released in the same
// CTA and waits forever otherwise, so an unbalanced split is refused here instead of launched.
// dec_threads drop to dec_regs, inc_threads rise to inc_regs (0 threads: no split).
template <typename KernelT>
int configure_kernel(KernelT kfn, int smem_bytes, std::atomic<bool>* done, int dec_threads,
                     int dec_regs, int inc_threads, int inc_regs) {
  int dev = 0;
  BOLT_CUDA(cudaGetDevice(&dev));
  BOLT_REQUIRE(dev >= 0 && dev < kMaxDevices, "grouped_gemm: device index %d out of range", dev);
  if (done[dev].load(std::memory_order_acquire)) return BOLT_OK;
  cudaFuncAttributes attr;
  BOLT_CUDA(cudaFuncGetAttributes(&attr, kfn));
  if (dec_threads > 0 &&
      (int64_t)dec_threads * (attr.numRegs - dec_regs) < (int64_t)inc_threads * (inc_regs - attr.numRegs)) {
    set_error("grouped_gemm: kernel was built with %d registers per thread; the register split "
              "%d x %d -> %d / %d x %d -> %d cannot balance, refusing to launch",
              attr.numRegs, dec_threads, attr.numRegs, dec_regs, inc_threads, attr.numRegs, inc_regs);
    return BOLT_ERR_UNSUPPORTED;
  }
  BOLT_CUDA(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
  done[dev].store(true, std::memory_order_release);
  return BOLT_OK;
}

template <int OPK, bool BS, int EPI, bool PAIR>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc,
           const GemmParams& p, int grid, cudaStream_t st) {
  auto kfn = k_grouped_gemm<OPK, BS, EPI, PAIR>;
  constexpr int smem = PAIR ? pair_smem_bytes_of(BS) : smem_bytes_of(BS);
  static std::atomic<bool> configured[kMaxDevices];
  // warps 0-3 drop to 56 registers, the eight epilogue warps rise to 224
  const int rc = configure_kernel(kfn, smem, configured, 128, 56, 256, 224);
  if (rc != BOLT_OK) return rc;
  if (PAIR) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    BOLT_CUDA(cudaLaunchKernelEx(&cfg, kfn, ma, mb, mc, p));
  } else {
    kfn<<<grid, kThreads, smem, st>>>(ma, mb, mc, p);
  }
  BOLT_LAUNCH_CHECK();
  return BOLT_OK;
}

template <int OPK, bool BS, bool PAIR>
int launch_epi2(int epi, const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc,
                const GemmParams& p, int grid, cudaStream_t st) {
  switch (epi) {
    case BOLT_EPI_STORE: return launch<OPK, BS, BOLT_EPI_STORE, PAIR>(ma, mb, mc, p, grid, st);
    case BOLT_EPI_SILU_MUL: return launch<OPK, BS, BOLT_EPI_SILU_MUL, PAIR>(ma, mb, mc, p, grid, st);
    case BOLT_EPI_SILU_MUL_QUANT:
      if constexpr (BS)
        return launch<OPK, true, BOLT_EPI_SILU_MUL_QUANT, PAIR>(ma, mb, mc, p, grid, st);
      set_error("grouped_gemm: fused group quantisation needs a block-scaled kind");
      return BOLT_ERR_UNSUPPORTED;
    default: set_error("grouped_gemm: unknown epilogue %d", epi); return BOLT_ERR_INVALID;
  }
}

template <int OPK, bool BS>
int launch_epi(int epi, bool pair, const CUtensorMap& ma, const CUtensorMap& mb,
               const CUtensorMap& mc, const GemmParams& p, int grid, cudaStream_t st) {
  return pair ? launch_epi2<OPK, BS, true>(epi, ma, mb, mc, p, grid, st)
              : launch_epi2<OPK, BS, false>(epi, ma, mb, mc, p, grid, st);
}

}  // namespace
}  // namespace bolt

extern "C" int bolt_grouped_gemm(const bolt_gemm_args* a, void* stream) {
  using namespace bolt;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  BOLT_REQUIRE(a != nullptr, "grouped_gemm: null args");
  BOLT_REQUIRE(a->capacity >= 0 && a->capacity % kBM == 0,
               "grouped_gemm: capacity %d must be a multiple of 128", a->capacity);
  if (a->capacity == 0) return BOLT_OK;
  BOLT_REQUIRE(a->n > 0 && a->k > 0 && a->num_experts > 0, "grouped_gemm: bad shape");
  BOLT_REQUIRE(a->a && a->b && a->c && a->sorted_expert_ids && a->num_valid_ids,
               "grouped_gemm: null pointer");
  const bool is16 = a->kind == BOLT_GEMM_BF16 || a->kind == BOLT_GEMM_F16;
  const bool block = a->kind == BOLT_GEMM_FP8_BLOCK || a->kind == BOLT_GEMM_INT8_BLOCK;
  const bool is_int = a->kind == BOLT_GEMM_INT8_CHANNEL || a->kind == BOLT_GEMM_INT8_BLOCK;
  const bool mx4 = a->kind == BOLT_GEMM_MXFP4;      // e4m3 rows x packed e2m1 weights
  const bool mx = a->kind == BOLT_GEMM_MXFP8 || mx4;
  BOLT_REQUIRE(a->kind >= BOLT_GEMM_BF16 && a->kind <= BOLT_GEMM_MXFP4,
               "grouped_gemm: unknown kind %d", a->kind);
  if (mx) {
    BOLT_REQUIRE(a->epilogue == BOLT_EPI_STORE || a->epilogue == BOLT_EPI_SILU_MUL_QUANT,
                 "grouped_gemm: the MX kind has the plain and the activation + MX-quantising epilogue");
    BOLT_REQUIRE(a->epilogue == BOLT_EPI_STORE || (a->n / 2) % 128 == 0,
                 "grouped_gemm: the MX gated epilogue needs n/2 a multiple of 128");
    BOLT_REQUIRE(a->k % 128 == 0, "grouped_gemm: the MX kind needs k a multiple of 128");
    BOLT_REQUIRE(a->bias == nullptr, "grouped_gemm: the MX kind takes no bias");
    BOLT_REQUIRE(!mx4 || reinterpret_cast<uintptr_t>(a->b) % 32 == 0,
                 "grouped_gemm: packed e2m1 weights must be 32-byte aligned");
  }
  const int elem = is16 ? 2 : 1;
  BOLT_REQUIRE(((int64_t)a->k * elem) % 16 == 0, "grouped_gemm: k*elem_size must be a multiple of 16");
  BOLT_REQUIRE((reinterpret_cast<uintptr_t>(a->a) | reinterpret_cast<uintptr_t>(a->b)) % 16 == 0,
               "grouped_gemm: operands must be 16-byte aligned");
  const bool gated = a->epilogue != BOLT_EPI_STORE;
  BOLT_REQUIRE(!gated || a->n % 2 == 0, "grouped_gemm: gated epilogue needs even n");
  if (!is16) BOLT_REQUIRE(a->a_scale && a->b_scale, "grouped_gemm: scales required");
  if (block) {
    BOLT_REQUIRE(a->k % 128 == 0 && a->n % 128 == 0,
                 "grouped_gemm: block-scaled kinds need k and n multiples of 128");
    BOLT_REQUIRE(!gated || (a->n / 2) % 128 == 0,
                 "grouped_gemm: gated block-scaled epilogue needs n/2 multiple of 128");
    BOLT_REQUIRE(a->a_scale_ld >= a->capacity, "grouped_gemm: a_scale_ld too small");
  }
  if (a->epilogue == BOLT_EPI_SILU_MUL_QUANT) {
    BOLT_REQUIRE(a->c_dtype == BOLT_FP8_E4M3 || a->c_dtype == BOLT_INT8,
                 "grouped_gemm: quantising epilogue needs an 8-bit c_dtype");
    BOLT_REQUIRE(a->c_scale != nullptr &&
                     a->c_scale_ld >= (mx ? (int64_t)(a->n / 2 / 32) : (int64_t)a->capacity),
                 "grouped_gemm: c_scale / c_scale_ld invalid");
    BOLT_REQUIRE(!mx || a->c_dtype == BOLT_FP8_E4M3, "grouped_gemm: MX codes are e4m3");
    BOLT_REQUIRE(a->c_ld % 16 == 0 && reinterpret_cast<uintptr_t>(a->c) % 16 == 0,
                 "grouped_gemm: quantised output must be 16-byte aligned");
    BOLT_REQUIRE(!a->scatter, "grouped_gemm: quantising epilogue writes sorted rows only");
  } else {
    BOLT_REQUIRE(a->c_dtype == BOLT_BF16 || a->c_dtype == BOLT_F16 || a->c_dtype == BOLT_F32,
                 "grouped_gemm: bad c_dtype %d", a->c_dtype);
  }
  BOLT_REQUIRE(!a->scatter || a->sorted_ids, "grouped_gemm: scatter needs sorted_ids");
  BOLT_REQUIRE(a->scatter_src == nullptr ||
                   (a->scatter && a->scatter_seg_off != nullptr && a->scatter_seg_rows > 0 && !mx),
               "grouped_gemm: segment-scattered output needs scatter, offsets and a segment size "
               "(plain kinds)");
  BOLT_REQUIRE(!a->mul_routed_weight || a->sorted_weights,
               "grouped_gemm: mul_routed_weight needs sorted_weights");

  BOLT_REQUIRE(a->schedule == BOLT_GEMM_SCHEDULE_ROW_TILES ||
                   a->schedule == BOLT_GEMM_SCHEDULE_TILE_PAIRS,
               "grouped_gemm: unknown schedule %d", a->schedule);
  const bool pair = a->schedule == BOLT_GEMM_SCHEDULE_TILE_PAIRS;
  if (pair) {
    BOLT_REQUIRE(!mx, "grouped_gemm: the tile-pair schedule is not built for the MX kind");
    BOLT_REQUIRE(a->segments != nullptr && a->num_segments != nullptr && a->max_segments > 0,
                 "grouped_gemm: the tile-pair schedule needs the segment list of bolt_moe_sort_ck");
  }

  const bool gather = a->a_gather != 0;
  if (gather) {
    BOLT_REQUIRE(!pair && !mx, "grouped_gemm: the gathered row operand needs the single-tile "
                               "schedule of the plain kinds");
    BOLT_REQUIRE(a->sorted_ids != nullptr && a->a_rows >= a->num_tokens && a->a_rows > 0,
                 "grouped_gemm: gathered row operand needs sorted_ids and a_rows >= num_tokens");
    BOLT_REQUIRE((a->a_row_bytes > 0 ? a->a_row_bytes : (int64_t)a->k * elem) / 16 * a->a_rows <
                     (1ll << 31),
                 "grouped_gemm: gathered row operand larger than 32 GiB");
    BOLT_REQUIRE(a->a_row_bytes == 0 ||
                     (a->a_row_bytes % 16 == 0 && a->a_row_bytes >= (int64_t)a->k * elem),
                 "grouped_gemm: a_row_bytes must be a multiple of 16 and cover a row");
  }

  EncodeTiledFn encode = get_encode_fn();
  if (encode == nullptr) {
    set_error("grouped_gemm: cuTensorMapEncodeTiled is unavailable");
    return BOLT_ERR_CUDA;
  }
  const CUtensorMapDataType dt = a->kind == BOLT_GEMM_BF16  ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                 : a->kind == BOLT_GEMM_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                            : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  const cuuint32_t bk = is16 ? 64 : 128;
  CUtensorMap ma, mb;
  {
    // (with a gathered row operand this map is not used by the kernel)
    cuuint64_t dims[2] = {(cuuint64_t)a->k, (cuuint64_t)(gather ? a->a_rows : a->capacity)};
    cuuint64_t strides[1] = {gather && a->a_row_bytes > 0 ? (cuuint64_t)a->a_row_bytes
                                                          : (cuuint64_t)a->k * elem};
    cuuint32_t box[2] = {bk, (cuuint32_t)kBM};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = encode(&ma, dt, 2, const_cast<void*>(a->a), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
      set_error("grouped_gemm: tensor map for A failed (CUresult %d)", (int)r);
      return BOLT_ERR_CUDA;
    }
  }
  {
    // packed e2m1 weights: two values per byte in global memory; the copy spreads every 8 bytes
    // (16 values) over 16 bytes of shared memory, the form the f8f6f4 instruction reads
    const CUtensorMapDataType dtb = mx4 ? CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B : dt;
    const cuuint64_t row_bytes = mx4 ? (cuuint64_t)a->k / 2 : (cuuint64_t)a->k * elem;
    cuuint64_t dims[3] = {(cuuint64_t)a->k, (cuuint64_t)a->n, (cuuint64_t)a->num_experts};
    cuuint64_t strides[2] = {row_bytes, row_bytes * a->n};
    cuuint32_t box[3] = {bk, 64, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = encode(&mb, dtb, 3, const_cast<void*>(a->b), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
      set_error("grouped_gemm: tensor map for B failed (CUresult %d)", (int)r);
      return BOLT_ERR_CUDA;
    }
  }

  GemmParams p{};
  p.a_scale = a->a_scale;
  p.a_scale_ld = a->a_scale_ld;
  p.b_scale = a->b_scale;
  p.bias = a->bias;
  p.bias_dtype = a->bias_dtype;
  p.c = a->c;
  p.c_dtype = a->c_dtype;
  p.mid_dtype = a->mid_dtype;
  p.c_ld = a->c_ld;
  p.c_scale = a->c_scale;
  p.c_scale_ld = a->c_scale_ld;
  p.scatter = a->scatter;
  p.scatter_src = a->scatter_src;
  p.scatter_seg_off = a->scatter_seg_off;
  p.scatter_seg_rows = a->scatter_seg_rows;
  p.c_vec_ok = (reinterpret_cast<uintptr_t>(a->c) % 16 == 0) &&
               ((a->c_ld * (int64_t)dtype_bytes(a->c_dtype)) % 16 == 0);
  // 16-bit output in sorted row order: blocks of 32 rows x 32 columns leave by bulk tensor
  // stores (64-byte-swizzled shared-memory source) instead of per-thread stores
  CUtensorMap mc;
  memset(&mc, 0, sizeof(mc));
  p.c_tma_ok = 0;
  const bool out8 = a->epilogue == BOLT_EPI_SILU_MUL_QUANT;   // e4m3 / int8 rows, never scattered
  if (p.c_vec_ok && !a->scatter && (out8 || a->c_dtype == BOLT_BF16 || a->c_dtype == BOLT_F16)) {
    const int64_t out_cols = gated ? a->n / 2 : a->n;
    const int esz = out8 ? 1 : 2;
    cuuint64_t dims[2] = {(cuuint64_t)out_cols, (cuuint64_t)a->capacity};
    cuuint64_t strides[1] = {(cuuint64_t)a->c_ld * esz};
    cuuint32_t box[2] = {(cuuint32_t)(64 / esz), 32};   // 64 bytes x 32 rows either way
    cuuint32_t estr[2] = {1, 1};
    CUresult r = encode(&mc, out8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_UINT16,
                        2, a->c, dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
                        CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    p.c_tma_ok = (r == CUDA_SUCCESS) ? 1 : 0;   // on failure the per-thread store paths remain
  }
  p.num_tokens = a->sorted_ids ? a->num_tokens : 1;
  p.topk = a->topk;
  p.mul_routed_weight = a->mul_routed_weight;
  p.sorted_ids = a->sorted_ids;
  p.sorted_weights = a->sorted_weights;
  p.expert_ids = a->sorted_expert_ids;
  p.num_valid = a->num_valid_ids;
  p.status = a->status;
  p.n = a->n;
  p.n_half = a->n / 2;
  p.k = a->k;
  p.num_experts = a->num_experts;
  p.capacity = a->capacity;
  p.tiles_n = gated ? (p.n_half + 127) / 128 : (a->n + 255) / 256;
  p.num_kb = (a->k + (int)bk - 1) / (int)bk;
  p.kb_scale_cols = a->k / 128;
  // Row tiles per group of the tile order.  Experts with many row tiles want a large group (the
  // CTAs of a wave then share one expert's weight tiles through L2: 16 beats 4 by 4 % on a
  // 16-tiles-per-expert bf16 layer), experts with one or two tiles a small one (4 beats 16 by
  // 0.8 % at 1.5 tiles per expert).  The sorted layout's capacity tells the average.
  {
    const double routes = a->capacity > a->num_experts * kBM ? a->capacity - a->num_experts * kBM : 0;
    const double tiles_per_expert = routes / ((double)a->num_experts * kBM) + 0.5;
    int g = (int)(2.0 * tiles_per_expert + 0.999);
    p.group_m = g < 4 ? 4 : (g > 16 ? 16 : g);
    if (pair) p.group_m = (p.group_m + 1) / 2;   // the unit of the tile order is a pair of row tiles
  }
  p.a_gather = gather ? 1 : 0;
  p.a_base = a->a;
  p.a_row_units = (int)((a->a_row_bytes > 0 ? a->a_row_bytes : (int64_t)a->k * elem) / 16);
  p.k_bytes = a->k * elem;
  p.segments = a->segments;
  p.num_segments = a->num_segments;
  p.max_segments = a->max_segments;
  const uint32_t fmt = a->kind == BOLT_GEMM_BF16 ? 1u : (is_int ? 1u : 0u);
  const uint32_t cfmt = is_int ? 2u : 1u;
  p.idesc = (cfmt << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(kAccCols >> 3) << 17) |
            ((uint32_t)((pair ? 2 * kBM : kBM) >> 4) << 24);   // M = 256 for a CTA pair
  if (mx) {
    // block-scaled descriptor: e4m3 x e4m3 (formats 0), K-major, N >> 3 at bit 17, E8M0 scales
    // (bit 23), M >> 4 at bit 24; the scale-byte selectors (bits 4-5, 29-30) are set per K step
    p.idesc = ((uint32_t)(kAccCols >> 3) << 17) | (1u << 23) | ((uint32_t)(kBM >> 4) << 24);
    if (mx4) p.idesc |= 5u << 10;      // B format e2m1 (A stays e4m3 = 0)
    // the copy of packed 4-bit values completes the barrier by the bytes it read (half of the
    // shared-memory footprint it writes)
    p.mx_stage_tx = kABytes + (mx4 ? kBBytes / 2 : kBBytes);
    p.mx_group128 = mx4 ? 1 : 0;
    p.sfa = reinterpret_cast<const uint8_t*>(a->a_scale);
    p.sfb = reinterpret_cast<const uint8_t*>(a->b_scale);
    p.n_blocks128 = gated ? 2 * p.tiles_n : (a->n + 127) / 128;
    p.act_alpha = a->act_alpha;
    p.act_beta = a->act_beta;
    p.act_limit = a->act_limit;
    p.act_has_limit = a->act_has_limit;
  }

  int sms = a->sm_count > 0 ? a->sm_count : sm_count_of_current_device();
  const int64_t max_tiles = pair ? 2ll * a->max_segments * p.tiles_n
                                 : (int64_t)(a->capacity / kBM) * p.tiles_n;
  int grid = (int)(max_tiles < sms ? max_tiles : sms);
  if (pair) grid &= ~1;   // whole clusters of two
  if (grid <= 0) return BOLT_OK;

  if (mx) {
    static std::atomic<bool> configured[2][kMaxDevices];
    int rc = configure_kernel(k_mx_gemm<false>, kMxSmemBytes, configured[0], 0, 0, 0, 0);
    if (rc == BOLT_OK) rc = configure_kernel(k_mx_gemm<true>, kMxSmemBytes, configured[1], 0, 0, 0, 0);
    if (rc != BOLT_OK) return rc;
    if (gated)
      k_mx_gemm<true><<<grid, kThreads, kMxSmemBytes, st>>>(ma, mb, mc, p);
    else
      k_mx_gemm<false><<<grid, kThreads, kMxSmemBytes, st>>>(ma, mb, mc, p);
    BOLT_LAUNCH_CHECK();
    return BOLT_OK;
  }
  switch (a->kind) {
    case BOLT_GEMM_BF16:
    case BOLT_GEMM_F16: return launch_epi<OP_F16, false>(a->epilogue, pair, ma, mb, mc, p, grid, st);
    case BOLT_GEMM_FP8_BLOCK: return launch_epi<OP_F8, true>(a->epilogue, pair, ma, mb, mc, p, grid, st);
    case BOLT_GEMM_FP8_CHANNEL: return launch_epi<OP_F8, false>(a->epilogue, pair, ma, mb, mc, p, grid, st);
    case BOLT_GEMM_INT8_CHANNEL: return launch_epi<OP_I8, false>(a->epilogue, pair, ma, mb, mc, p, grid, st);
    case BOLT_GEMM_INT8_BLOCK: return launch_epi<OP_I8, true>(a->epilogue, pair, ma, mb, mc, p, grid, st);
    default: break;
  }
  set_error("grouped_gemm: unsupported kind %d", a->kind);
  return BOLT_ERR_UNSUPPORTED;
}
