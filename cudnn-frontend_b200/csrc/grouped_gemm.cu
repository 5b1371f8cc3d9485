// Block-scaled (MXFP8, MXFP4, NVFP4) grouped GEMM for MoE experts with fused epilogues (sm_100a).
//
//   FC1: C = alpha_e (A SFA)(B_e SFB_e)^T ; D = up * silu(gate) * prob   (gate/up = even/odd
//        32-column blocks of C) ; per-expert amax, or row / column MXFP8 re-quantisation.
//   FC2: D = alpha_e acc * prob ; bf16 + amax, or E4M3 + row / column E8M0 scale factors.
//   dSwiGLU (backward of FC1's activation): G = alpha_e^2 acc is the gradient of the SwiGLU output; with the
//        forward pre-activation C (gate / up = even / odd 32-column blocks, scaled by beta_e) the epilogue
//        writes d_gate = G prob up sig (1 + gate (1 - sig)) and d_up = G prob gate sig into the same blocks
//        of D (twice as wide as the GEMM's N), adds sum(G gate sig up) to dprob, and re-quantises like FC2.
//
//   wgrad (weight gradient): the experts split K instead of M.  A is [m, T] and B is [n, T], both contiguous along
//        the token dimension T; expert e owns tokens [offsets[e-1], offsets[e]) and its own 128x4 block of scale
//        factors; wgrad[e] = gs_e (A_e SFA_e)(B_e SFB_e)^T, [E, m, n] in bf16 / fp16 / float32, stored or added to.
//
// Persistent kernel, one CTA per SM, walking a tile schedule derived on the device from the
// per-expert END offsets: tiles of small expert groups (which stream their weights from HBM for one
// or two row tiles) are interleaved with tiles of large groups (which reuse weights from L2), and
// the sequence is walked with a static stride or through an atomic counter.  Warp roles:
//   warp 0, 10  producers: TMA loads of the A tile (warp 0) and the B tile (warp 10), 128-byte
//               swizzled, plus their 512-byte scale-factor chunks, into a shared-memory ring
//   warp 1      TMEM owner and MMA issuer: tcgen05.cp moves the scale factors to TMEM, then
//               tcgen05.mma.kind::mxf8f6f4.block_scale accumulates into TMEM
//   warps 2..9  epilogue: tcgen05.ld, alpha / SwiGLU / prob / amax / re-quantisation, stores
//
// Two tile modes, one template:
//   single  one CTA computes 128 x 256 (cta_group::1), 4 stages of 48 KB, scale chunks by untiled
//           bulk copies.  Suits small expert groups (no padding beyond 128 rows).
//   pair    two CTAs of a (2,1,1) cluster compute 256 x 256 (cta_group::2): each loads its own
//           128 rows of A and its own 128-row half of B, so a B tile crosses L2 -> SM once per
//           256 rows; 6 stages of 33.5 KB.  Only the leader issues MMAs; every load of either CTA
//           credits the leader's "full" barrier; tcgen05.commit releases the stage in both CTAs.
//
// TMEM (512 columns): accumulator 0 at columns [0,256), accumulator 1 at [224,480), scale
// factors at [480,512).  The two accumulators share 32 columns; the epilogue drains those
// first (even tiles from the top, odd tiles from the bottom) and then lets the MMA warp start
// the next tile while it finishes the rest.
//
// Operand formats (template parameter kFmt): 0 = 8-bit operands (E4M3 / E5M2), one E8M0 scale per 32
// elements, tcgen05.mma.kind::mxf8f6f4; 1 = packed E2M1 (two per byte), one E8M0 scale per 32 elements,
// kind::mxf4; 2 = packed E2M1, one E8M0 or UE4M3 scale per 16 elements, kind::mxf4nvf4.  A k-tile is 128
// bytes of K in every format (128, 256, 256 elements) and four MMAs; it carries 1, 2 or 4 scale chunks
// of 512 bytes per 128 operand rows.  With E2M1 operands the scale factors take 48 TMEM columns (one
// buffer), so the accumulators overlap by 48 columns instead of 32.
//
// Every CTA loads what it needs into its own shared memory with plain (one-destination) TMA
// loads, so the same binary serves single- and multi-GPU processes.
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>

#include <mutex>

#include "b200moe.h"
#include "common.cuh"

namespace b200moe {

// ---------------------------------------------------------------------------------------
// Tile configuration
// ---------------------------------------------------------------------------------------
constexpr int BM = 128;  // rows per CTA
constexpr int BN = 256;
constexpr int BK = 128;  // bytes == elements (E4M3); one 128-byte swizzle row
constexpr int A_STAGE_BYTES = BM * BK;  // 16 KiB
constexpr int NUM_EPI_WARPS = 8;
constexpr int PRODUCER_B_WARP = 2 + NUM_EPI_WARPS;  // the last warp
constexpr int NUM_THREADS = (3 + NUM_EPI_WARPS) * 32;
constexpr int MAX_EXPERTS = 1024;
constexpr int RASTER_GROUP_ROWS = 4096;        // rows of one expert that share a B tile back to back ...
constexpr int64_t RASTER_GROUP_BYTES = 32 << 20;  // ... unless that many rows of A exceed this share of L2

// Defaults of the two schedule options.  Timed round-robin against each other on the DeepSeek-shape
// cases (E = 256, Zipf rows): interleaving experts of one or two row tiles is 2 % faster than walking
// the experts in order (FC1 2.60 against 2.65 ms, FC2 1.37 against 1.41 ms); the evict-first hint
// changes nothing measurable there and stays off.
constexpr int DEFAULT_LIGHT_M_TILES = 2;
constexpr int DEFAULT_STREAM_M_TILES = 0;

constexpr int TMEM_COLS = 512;

// status codes recorded by bounded waits
constexpr int ST_PRODUCER_EMPTY = 101;
constexpr int ST_MMA_FULL = 102;
constexpr int ST_MMA_OVERLAP = 103;
constexpr int ST_EPI_ACC = 104;
constexpr int ST_SCHED_FULL = 105;   // a consumer of the dynamic scheduler's ring
constexpr int ST_SCHED_EMPTY = 106;  // the fetching warp waiting for a free ring slot
constexpr int ST_WGRAD_K_UNALIGNED = 202;  // wgrad: an expert's token range is not a multiple of 32

constexpr int SCHED_RING = 8;  // tile ids in flight between the fetching warp and the other warps (dynamic scheduler)

// kBulk: bf16 D rows leave through a shared-memory staging area and one bulk copy per row (used
// when the rows go to peer GPUs: 256-byte bursts instead of 32-byte stores); the staging area
// takes the place of two (pair) or one (single) pipeline stages.
constexpr int STAGING_ROW_BYTES = 256 + 16;  // 128 bf16 columns of one row, padded against bank conflicts
constexpr int STAGING_WARP_BYTES = 32 * STAGING_ROW_BYTES;

template <bool kPair, bool kBulk = false, int kFmt = 0>
struct Cfg {
  static constexpr int CPK = 1 << kFmt;  // 512-byte scale chunks per k-tile and 128 operand rows
  static constexpr int SFA_STAGE_BYTES = 512 * CPK;
  static constexpr int SFB_STAGE_BYTES = 1024 * CPK;  // [128-row block of B][chunk]
  // TMEM: accumulator 0 at column 0, accumulator 1 at ACC1_COL, scale factors from SF_COL.
  // 8-bit operands: two scale buffers of 16 columns (SFA 4 + SFB 8 used); E2M1: one buffer, SFA at +0
  // (4 columns per chunk), SFB at +16 (8 columns per chunk: both 128-row blocks of B side by side)
  static constexpr int TMEM_ACC1_COL = kFmt ? 208 : 224;
  static constexpr int TMEM_SF_COL = kFmt ? 464 : 480;
  static constexpr int STAGES = kBulk ? (kPair ? 4 : 3) : (kPair ? (kFmt == 2 ? 5 : 6) : 4);
  static constexpr int B_ROWS = kPair ? 128 : 256;  // rows of B this CTA loads per stage
  static constexpr int B_STAGE_BYTES = B_ROWS * BK;
  static constexpr int TILE_M = kPair ? 256 : 128;  // rows of one scheduled tile
  static constexpr int CTAS = kPair ? 2 : 1;
  static constexpr int A_OFF = 0;
  static constexpr int B_OFF = A_OFF + STAGES * A_STAGE_BYTES;
  static constexpr int SFA_OFF = B_OFF + STAGES * B_STAGE_BYTES;
  static constexpr int SFB_OFF = SFA_OFF + STAGES * SFA_STAGE_BYTES;
  static constexpr int BAR_OFF = SFB_OFF + STAGES * SFB_STAGE_BYTES;  // 8-byte barriers
  static constexpr int NUM_BARS = 2 * STAGES + 2 + 1 + 2 * SCHED_RING;
  static constexpr int MISC_OFF = BAR_OFF + NUM_BARS * 8;  // tmem ptr, abort flag, tile totals, scheduler ring
  static constexpr int PREFIX_OFF = MISC_OFF + 16 + SCHED_RING * 4;  // 2 x (E + 1) int32 tile prefixes (heavy, light)
  static constexpr int STAGING_OFF = (PREFIX_OFF + 2 * (MAX_EXPERTS + 1) * 4 + 15) & ~15;
  // column-quantisation scratch, 64 floats per epilogue warp: shares the staging area (staged rows are never
  // quantised); E2M1 operands have no quantised output and no scratch
  static constexpr int COLQ_OFF = STAGING_OFF;
  static constexpr int TOTAL = STAGING_OFF + (kBulk ? NUM_EPI_WARPS * STAGING_WARP_BYTES : (kFmt ? 0 : NUM_EPI_WARPS * 256));
  static constexpr int SMEM_BYTES = TOTAL + 1024;  // slack for manual 1024-byte alignment
  // bytes credited to a "full" barrier per stage (both CTAs of a pair together)
  static constexpr uint32_t TX_BYTES = CTAS * (A_STAGE_BYTES + B_STAGE_BYTES + SFA_STAGE_BYTES + SFB_STAGE_BYTES);
};
static_assert(Cfg<false>::SMEM_BYTES <= 232448 && Cfg<true>::SMEM_BYTES <= 232448, "shared memory budget exceeded");
static_assert(Cfg<false, false, 1>::SMEM_BYTES <= 232448 && Cfg<true, false, 1>::SMEM_BYTES <= 232448, "shared memory budget exceeded");
static_assert(Cfg<false, false, 2>::SMEM_BYTES <= 232448 && Cfg<true, false, 2>::SMEM_BYTES <= 232448, "shared memory budget exceeded");
static_assert(Cfg<false, true>::SMEM_BYTES <= 232448 && Cfg<true, true>::SMEM_BYTES <= 232448, "shared memory budget exceeded");

enum : int { EPI_FC1 = 0, EPI_FC2 = 1, EPI_DSWIGLU = 2, EPI_WGRAD = 3 };

struct GemmParams {
  const uint8_t* sfa;
  const uint8_t* sfb;         // dense: expert e at sfb + e * sfb_expert_bytes
  const int64_t* sfb_ptrs;    // discrete
  const CUtensorMap* b_maps;  // discrete: E tensor maps of B, then E tensor maps of SFB, in the workspace
  const int32_t* offsets;
  const float* alpha;
  const float* prob;
  const float* norm_const;
  const int32_t* d_row_map;  // optional scatter of bf16 D rows
  const int64_t* d_peer_ptrs;  // optional: the scatter targets are peer buffers, see b200moe.h
  int64_t d_peer_slots;
  __nv_bfloat16* c;
  void* d;
  uint8_t* d_col;
  float* amax;
  uint8_t* sfd_row;
  uint8_t* sfd_col;
  int64_t sfb_expert_bytes;
  int m_rows, n, k, num_experts;
  int k_bytes;         // bytes of one operand row: k (8-bit operands) or k / 2 (packed E2M1)
  int n_out;           // n / 2 (FC1) or n (FC2)
  int n_tiles;         // ceil(n / 256)
  int k_tiles;         // ceil(k_bytes / 128)
  int rest_k;          // ceil(ceil(k / sf_vec) / 4): 512-byte scale chunks along K of SFA / SFB
  int n_blocks;        // ceil(n / 128): 128-row blocks of SFB
  int sfd_row_rest_k;  // ceil(ceil(n_out / 32) / 4)
  int sfd_col_rest_k;  // ceil(ceil(m_rows / 32) / 4)
  int d_is_fp8;
  int gen_sfd;        // row (and column) scale factors are generated and D holds scaled values
  int d_e5m2;         // FP8 D (and D_col) in E5M2 instead of E4M3
  float d_rcp_limit;  // 1/448 (E4M3) or 1/128 (E5M2)
  int d_f16, c_f16;   // 16-bit D / C in fp16 instead of bf16
  int d_f32;          // D in float32 (E2M1 operands only)
  int discrete_col_sfd;
  int wide_stores;     // every output row segment of 32 bytes is 32-byte aligned
  const void* c_in;    // dSwiGLU: forward pre-activation [m_rows, 2 n], bf16 / fp16 / E4M3 / E5M2
  int c_in_dtype;
  const float* beta;   // dSwiGLU: per-expert scale of c_in (NULL = 1)
  float* dprob;        // dSwiGLU: [m_rows], atomically accumulated
  const void* bias;    // optional [E][N] (element (n, e) at e * N + n), added after alpha
  int bias_dtype;      // B200MOE_DTYPE_BF16 / _F16 / _F32
  int act_geglu;       // FC1: 0 = SwiGLU, 1 = GeGLU
  uint32_t ab_format;  // A / B format bits of the instruction descriptor (0 = E4M3; E5M2 and E2M1 = 1 in both fields)
  int sf_e4m3;         // scale factors are UE4M3 instead of E8M0 (kFmt 2 only)
  int raster_group_m;  // row tiles per raster group
  int light_m_tiles;   // experts with at most this many row tiles form the "light" class (0 = one class)
  int stream_m_tiles;  // weight tiles of experts with at most this many row tiles are loaded with an evict-first L2 hint
  int accumulate;      // wgrad: add to the output instead of overwriting it
  int first_has_prev;  // offsets[-1] is readable and is the first row of expert 0 (a slice of a longer expert list)
  int b_nmajor;        // B is [K][N] per expert (N contiguous) instead of [N][K]
  int dynamic_sched;   // tiles after each CTA's first come from an atomic counter
  int* tile_counter;   // dynamic scheduler: zeroed before the launch
  int test_skip_b_loads;  // test hook: the B-side producer issues no load, so every wait runs out
  uint64_t wait_limit_ns;
};

// ---------------------------------------------------------------------------------------
// Tile schedule.
//
// Experts fall into two classes by their number of row tiles.  A "heavy" expert has many row tiles
// per weight tile: its weights are read from HBM once and reused from L2, so its tiles are bound by
// the tensor pipe.  A "light" expert (at most `light_m_tiles` row tiles) streams every weight tile
// from HBM for one or two MMAs' worth of rows: its tiles are bound by HBM.  Walking the experts in
// order would alternate between phases where every SM waits for HBM and phases where HBM idles.
// The linear schedule therefore interleaves the two classes evenly (position s is the
// floor(s nL / total)-th light tile when that count steps up at s, else the next heavy tile), so
// that at any time a fixed share of the SMs streams weights while the others compute.
//
// Inside a class expert e owns tiles [prefix[e], prefix[e+1]); inside an expert tiles run in
// groups of `group_m` row tiles, row tile fastest, so that CTAs working on adjacent schedule slots
// read the same B tile at the same time and the A rows of the group stay in L2 while the B tiles
// stream past once.  With groups of 4096 rows every B tile of a Mixtral-size expert comes from HBM
// exactly once; groups of 2048 rows measured 4-6 % slower, 1024 rows 10 %.
// A row tile is 128 rows (single) or 256 rows (pair).
// ---------------------------------------------------------------------------------------
struct Tile {
  int expert, row0, n_tile, row_end, m_tiles;
  // wgrad only: the expert's range of K (tokens) in bytes, its k-tiles, its scale chunks along K and the number
  // of scale chunks (along K, per 128-row block) of all experts before it
  int k0, kbytes, k_tiles, rest_k, chunk0;
};

struct Sched {
  const int* prefix_heavy;  // [E + 1]
  const int* prefix_light;  // [E + 1]
  int n_light, total;
};

__device__ __forceinline__ int expert_first_row(const GemmParams& p, int e) {
  return e == 0 ? (p.first_has_prev ? p.offsets[-1] : 0) : p.offsets[e - 1];
}

__device__ __forceinline__ Tile decode_tile(const Sched& sc, const GemmParams& p, int tile_m, int s) {
  const int* prefix = sc.prefix_heavy;
  int t = s;
  if (sc.n_light > 0) {
    const int before = (int)(((int64_t)s * sc.n_light) / sc.total);
    const int after = (int)(((int64_t)(s + 1) * sc.n_light) / sc.total);
    if (after > before) {
      prefix = sc.prefix_light;
      t = before;
    } else {
      t = s - before;
    }
  }
  int lo = 0, hi = p.num_experts;  // find e with prefix[e] <= t < prefix[e + 1]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (prefix[mid] <= t) lo = mid; else hi = mid;
  }
  const int e = lo;
  const int j = t - prefix[e];
  const int n_tiles = p.n_tiles, group_m = p.raster_group_m;
  const int m_tiles = (prefix[e + 1] - prefix[e]) / n_tiles;
  const int per_group = group_m * n_tiles;
  const int g = j / per_group;
  const int first_m = g * group_m;
  const int gsize = min(group_m, m_tiles - first_m);
  const int jj = j - g * per_group;
  Tile tile;
  tile.expert = e;
  tile.m_tiles = m_tiles;
  tile.n_tile = jj / gsize;
  tile.row0 = expert_first_row(p, e) + (first_m + jj % gsize) * tile_m;
  tile.row_end = p.offsets[e];
  return tile;
}

// wgrad: every expert has the same m_tiles x n_tiles output tiles; the row tile runs fastest so that CTAs working at
// the same time share the B tile.  `chunk_prefix[e]` = scale chunks along K of the experts before e.
__device__ __forceinline__ Tile decode_tile_wgrad(const GemmParams& p, const int* chunk_prefix, int tile_m, int s, int sf_vec_shift, int bytes_shift) {
  const int m_tiles = (p.m_rows + tile_m - 1) / tile_m;
  const int per_expert = m_tiles * p.n_tiles;
  Tile t;
  t.expert = s / per_expert;
  const int j = s - t.expert * per_expert;
  t.n_tile = j / m_tiles;
  t.row0 = (j - t.n_tile * m_tiles) * tile_m;
  t.row_end = p.m_rows;
  t.m_tiles = m_tiles;
  const int tok0 = t.expert == 0 ? 0 : p.offsets[t.expert - 1];
  int toks = max(p.offsets[t.expert] - tok0, 0);
  if ((tok0 | toks) & 31) {  // scale blocks and TMA coordinates need whole blocks of 32 tokens
    atomicCAS(&g_device_status, 0, ST_WGRAD_K_UNALIGNED);
    toks = 0;
  }
  t.k0 = tok0 >> bytes_shift;
  t.kbytes = toks >> bytes_shift;
  t.k_tiles = (t.kbytes + BK - 1) / BK;
  t.rest_k = ((toks >> sf_vec_shift) + 3) >> 2;
  t.chunk0 = chunk_prefix[t.expert];
  return t;
}

// ---------------------------------------------------------------------------------------
// Epilogue helpers.  A thread owns one row of the tile; `v` holds 32 consecutive output
// columns of that row in float32.
// ---------------------------------------------------------------------------------------
// 32 bytes to one row: a single 256-bit store when the caller's buffers allow it (`wide`), else two
// 128-bit stores.  A 128-bit store per lane fills only half of a 32-byte sector of the row it
// touches; the 256-bit form halves the store instructions and writes whole sectors.
__device__ __forceinline__ void store_32B(void* dst, uint4 lo, uint4 hi, bool wide) {
  if (wide) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst), "r"(lo.x), "r"(lo.y), "r"(lo.z),
                 "r"(lo.w), "r"(hi.x), "r"(hi.y), "r"(hi.z), "r"(hi.w)
                 : "memory");
  } else {
    reinterpret_cast<uint4*>(dst)[0] = lo;
    reinterpret_cast<uint4*>(dst)[1] = hi;
  }
}

// 32 values as bf16 (or fp16 when f16 is set): the two 16-bit types share pitch and alignment
__device__ __forceinline__ void store_bf16x32(__nv_bfloat16* dst, const float* v, bool wide, bool f16 = false) {
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    uint4 lo, hi;
    lo.x = pack16x2_from_float(v[16 * i + 0], v[16 * i + 1], f16);
    lo.y = pack16x2_from_float(v[16 * i + 2], v[16 * i + 3], f16);
    lo.z = pack16x2_from_float(v[16 * i + 4], v[16 * i + 5], f16);
    lo.w = pack16x2_from_float(v[16 * i + 6], v[16 * i + 7], f16);
    hi.x = pack16x2_from_float(v[16 * i + 8], v[16 * i + 9], f16);
    hi.y = pack16x2_from_float(v[16 * i + 10], v[16 * i + 11], f16);
    hi.z = pack16x2_from_float(v[16 * i + 12], v[16 * i + 13], f16);
    hi.w = pack16x2_from_float(v[16 * i + 14], v[16 * i + 15], f16);
    store_32B(dst + 16 * i, lo, hi, wide);
  }
}

// 32 values of a 16-bit or float32 D: element index `idx` counts from `base` in elements of D's type
__device__ __forceinline__ void store_d32(__nv_bfloat16* base, int64_t idx, const float* v, bool wide, bool f16, bool f32) {
  if (f32) {
    float* dst = reinterpret_cast<float*>(base) + idx;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4 lo = make_uint4(__float_as_uint(v[8 * i]), __float_as_uint(v[8 * i + 1]), __float_as_uint(v[8 * i + 2]), __float_as_uint(v[8 * i + 3]));
      const uint4 hi = make_uint4(__float_as_uint(v[8 * i + 4]), __float_as_uint(v[8 * i + 5]), __float_as_uint(v[8 * i + 6]), __float_as_uint(v[8 * i + 7]));
      store_32B(dst + 8 * i, lo, hi, wide);
    }
  } else {
    store_bf16x32(base + idx, v, wide, f16);
  }
}

__device__ __forceinline__ void store_e4m3x32(uint8_t* dst, const float* v, float scale, bool wide, bool e5m2 = false) {
  uint32_t o[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float2 lo = mul2(make_float2(v[4 * i], v[4 * i + 1]), scale);
    const float2 hi = mul2(make_float2(v[4 * i + 2], v[4 * i + 3]), scale);
    o[i] = fp8x4_from_float(lo.x, lo.y, hi.x, hi.y, e5m2);
  }
  store_32B(dst, make_uint4(o[0], o[1], o[2], o[3]), make_uint4(o[4], o[5], o[6], o[7]), wide);
}

// Output format of the scale-factor-generating epilogue: the reciprocal of the value the block maximum is
// mapped to (the reference's get_dtype_rcp_limits: 1/448 for E4M3, 1/128 for E5M2, 1 for a 16-bit D) and
// how the scaled values are stored (FP8 bytes, or bf16 / fp16 when D is a 16-bit tensor: the reference
// then keeps the scaled values, which lie in (-1, 1], in D's own type).
struct OutFormat {
  float rcp_limit;
  bool e5m2;
  bool bits16;  // D and D_col hold 16-bit values
  bool f16;     // ... fp16 instead of bf16
};

// 32 scaled values of one row: element `col` of the row that starts at `row_base` (a byte pointer)
__device__ __forceinline__ void store_scaled32(uint8_t* row_base, int64_t col, const float* v, float scale, bool wide, OutFormat fmt) {
  if (fmt.bits16) {
    float t[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) t[i] = v[i];
    scale_inplace<32>(t, scale);
    store_bf16x32(reinterpret_cast<__nv_bfloat16*>(row_base) + col, t, wide, fmt.f16);
  } else {
    store_e4m3x32(row_base + col, v, scale, wide, fmt.e5m2);
  }
}

// Row-wise scaling of one 32-element block: returns the E8M0 byte, stores the 32 scaled values.
__device__ __forceinline__ uint32_t quant_row_block(uint8_t* row_base, int64_t col, const float* v, float norm_const, bool wide,
                                                    OutFormat fmt) {
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
  const float pv = amax * fmt.rcp_limit * norm_const;
  const uint32_t sf = e8m0_from_float(pv);
  store_scaled32(row_base, col, v, quant_scale(norm_const, e8m0_to_float(sf)), wide, fmt);
  return sf;
}

// Column-wise MXFP8: the 32 rows of a scale block are the 32 lanes of the warp.  Lane i
// returns the E8M0 byte of column i; every lane stores its row's 32 E4M3 bytes.
//
// One warp reduction per column yields the 32 column maxima (the same value in every lane); lane 0
// parks them in the warp's 64-float scratch in shared memory (`scratch`, a .shared address), lane i picks up column i, derives that
// column's scale once and parks it in the second half of the scratch, from where every lane reads all
// 32 scales as eight broadcast loads.  (A halving exchange by shuffles, 31 shuffles and 62 selects per
// lane, and 32 more shuffles to hand the scales round, was three times the instructions.)
__device__ __forceinline__ uint32_t quant_col_block(uint8_t* row_base, int64_t col, bool do_store, const float* v, float norm_const,
                                                    bool wide, OutFormat fmt, uint32_t scratch) {
  const uint32_t lane = lane_id();
#pragma unroll
  for (int j = 0; j < 32; j += 4) {
    const float4 m = make_float4(warp_absmax_number(v[j]), warp_absmax_number(v[j + 1]), warp_absmax_number(v[j + 2]), warp_absmax_number(v[j + 3]));
    if (lane == 0) st_shared_f32x4(scratch + 4 * j, m);
  }
  __syncwarp();
  const float cmax = ld_shared_f32(scratch + 4 * lane);
  // scale of column `lane`
  const float pv = cmax * fmt.rcp_limit * norm_const;
  const uint32_t my_sf = e8m0_from_float(pv);
  const float sfv = e8m0_to_float(my_sf);
  float my_sc = sfv == 0.0f ? 0.0f : norm_const * rcp_approx(sfv);
  my_sc = fminf(my_sc, 3.40282346638528859812e38f);
  st_shared_f32(scratch + 128 + 4 * lane, my_sc);
  __syncwarp();
  if (fmt.bits16) {
    float t[32];
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
      const float4 sc = ld_shared_f32x4(scratch + 128 + 4 * i);
      const float2 lo = mul2(make_float2(v[i], v[i + 1]), make_float2(sc.x, sc.y));
      const float2 hi = mul2(make_float2(v[i + 2], v[i + 3]), make_float2(sc.z, sc.w));
      t[i] = lo.x;
      t[i + 1] = lo.y;
      t[i + 2] = hi.x;
      t[i + 3] = hi.y;
    }
    if (do_store) store_bf16x32(reinterpret_cast<__nv_bfloat16*>(row_base) + col, t, wide, fmt.f16);
    return my_sf;
  }
  uint32_t packed[8];
#pragma unroll
  for (int i = 0; i < 32; i += 4) {
    const float4 sc = ld_shared_f32x4(scratch + 128 + 4 * i);
    const float2 lo = mul2(make_float2(v[i], v[i + 1]), make_float2(sc.x, sc.y));
    const float2 hi = mul2(make_float2(v[i + 2], v[i + 3]), make_float2(sc.z, sc.w));
    packed[i >> 2] = fp8x4_from_float(lo.x, lo.y, hi.x, hi.y, fmt.e5m2);
  }
  if (do_store)
    store_32B(row_base + col, make_uint4(packed[0], packed[1], packed[2], packed[3]), make_uint4(packed[4], packed[5], packed[6], packed[7]),
              wide);
  return my_sf;
}

// Eight consecutive bias values (same for every row of the tile) as float32.
__device__ __forceinline__ void load_bias8(const void* bias, int dtype, int64_t idx, float* out) {
  if (dtype == B200MOE_DTYPE_F32) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(bias) + idx));
    const float4 b = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(bias) + idx) + 1);
    out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
    out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
  } else {
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(bias) + idx));
    if (dtype == B200MOE_DTYPE_BF16) {
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        out[2 * j] = f.x;
        out[2 * j + 1] = f.y;
      }
    } else {
      const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(h[j]);
        out[2 * j] = f.x;
        out[2 * j + 1] = f.y;
      }
    }
  }
}

// ---------------------------------------------------------------------------------------
// The kernel
// ---------------------------------------------------------------------------------------
template <int kEpi, bool kDiscrete, bool kPair, bool kBulk = false, int kFmt = 0>
__global__ void __launch_bounds__(NUM_THREADS, 1)
    grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                        const __grid_constant__ CUtensorMap tmap_sfa, const __grid_constant__ CUtensorMap tmap_sfb,
                        const GemmParams p) {
  using C = Cfg<kPair, kBulk, kFmt>;
  constexpr int STAGES = C::STAGES;
  constexpr int CPK = C::CPK;
  constexpr int SFA_STAGE_BYTES = C::SFA_STAGE_BYTES, SFB_STAGE_BYTES = C::SFB_STAGE_BYTES;
  constexpr int TMEM_ACC1_COL = C::TMEM_ACC1_COL, TMEM_SF_COL = C::TMEM_SF_COL;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_base + C::BAR_OFF;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto acc_full_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + b); };
  const uint32_t overlap_bar = bar_base + 8u * (2 * STAGES + 2);
  // dynamic scheduler: ring slot q holds a tile id once info_full(q) completes; its readers arrive on info_empty(q)
  auto info_full_bar = [&](int q) { return bar_base + 8u * (2 * STAGES + 3 + q); };
  auto info_empty_bar = [&](int q) { return bar_base + 8u * (2 * STAGES + 3 + SCHED_RING + q); };
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(smem + C::MISC_OFF);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + C::MISC_OFF + 4);
  int* totals_smem = reinterpret_cast<int*>(smem + C::MISC_OFF + 8);  // [0] all tiles, [1] light tiles
  volatile int* ring = reinterpret_cast<volatile int*>(smem + C::MISC_OFF + 16);
  int* prefix_heavy = reinterpret_cast<int*>(smem + C::PREFIX_OFF);
  int* prefix_light = prefix_heavy + (MAX_EXPERTS + 1);
  const WaitCtx wc = {abort_flag, p.wait_limit_ns};

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // pair mode: rank 0 of the 2-CTA cluster is the leader (issues the MMAs, owns the "full" and
  // "overlap" barriers, fetches tiles for both CTAs); a scheduled tile is 256 rows and this CTA
  // covers rows [128 rank, +128)
  const uint32_t cta_rank = kPair ? cluster_ctarank() : 0u;
  const int sched_id = kPair ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int sched_stride = kPair ? (int)(gridDim.x >> 1) : (int)gridDim.x;

  // ---- set-up -----------------------------------------------------------------------
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(acc_full_bar(0), 1);
    mbar_init(acc_full_bar(1), 1);
    mbar_init(overlap_bar, C::CTAS * NUM_EPI_WARPS);
    for (int q = 0; q < SCHED_RING; ++q) {
      mbar_init(info_full_bar(q), 1);
      // readers of a slot: MMA warp (leader), B producer and 8 epilogue warps per CTA, A producer of the second CTA
      mbar_init(info_empty_bar(q), kPair ? 2 * (NUM_EPI_WARPS + 1) + 2 : NUM_EPI_WARPS + 2);
    }
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tensormap(&tmap_a);
    if (!kDiscrete) prefetch_tensormap(&tmap_b);
    if (kPair) {
      prefetch_tensormap(&tmap_sfa);
      if (!kDiscrete) prefetch_tensormap(&tmap_sfb);
    }
  }
  if (warp == 1) {
    if (kPair) {
      tmem_alloc_pair(smem_u32(tmem_ptr_smem), TMEM_COLS);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(tmem_ptr_smem), TMEM_COLS);
      tmem_relinquish();
    }
  }
  if (kEpi == EPI_WGRAD && warp == 2) {
    // scale chunks along K of the experts before each expert (every expert has the same number of tiles)
    const int sf_shift = kFmt == 2 ? 4 : 5;
    int run = 0;
    for (int e0 = 0; e0 < p.num_experts; e0 += 32) {
      const int e = e0 + lane;
      int c = 0;
      if (e < p.num_experts) {
        const int toks = max(p.offsets[e] - (e == 0 ? 0 : p.offsets[e - 1]), 0);
        c = ((toks >> sf_shift) + 3) >> 2;
      }
      int incl = c;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int o = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += o;
      }
      if (e < p.num_experts) prefix_heavy[e] = run + incl - c;
      run += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) {
      totals_smem[0] = p.num_experts * ((p.m_rows + C::TILE_M - 1) / C::TILE_M) * p.n_tiles;
      totals_smem[1] = 0;
    }
  } else if (warp == 2) {
    // tile prefixes over experts, one per class: lane l scans a contiguous chunk of experts, then a
    // warp scan of the chunk sums
    const int chunk = (p.num_experts + 31) / 32;
    const int e0 = lane * chunk, e1 = min(e0 + chunk, p.num_experts);
    auto tiles_of = [&](int e, bool& light) {
      const int rows = max(p.offsets[e] - expert_first_row(p, e), 0);
      const int m_tiles = (rows + C::TILE_M - 1) / C::TILE_M;
      light = m_tiles <= p.light_m_tiles;
      return m_tiles * p.n_tiles;
    };
    int sum_h = 0, sum_l = 0;
    for (int e = e0; e < e1; ++e) {
      bool light;
      const int t = tiles_of(e, light);
      if (light) sum_l += t; else sum_h += t;
    }
    int incl_h = sum_h, incl_l = sum_l;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int th = __shfl_up_sync(0xffffffffu, incl_h, d);
      const int tl = __shfl_up_sync(0xffffffffu, incl_l, d);
      if (lane >= d) { incl_h += th; incl_l += tl; }
    }
    int run_h = incl_h - sum_h, run_l = incl_l - sum_l;
    for (int e = e0; e < e1; ++e) {
      prefix_heavy[e] = run_h;
      prefix_light[e] = run_l;
      bool light;
      const int t = tiles_of(e, light);
      if (light) run_l += t; else run_h += t;
    }
    if (lane == 31) {
      prefix_heavy[p.num_experts] = incl_h;
      prefix_light[p.num_experts] = incl_l;
      totals_smem[0] = incl_h + incl_l;
      totals_smem[1] = incl_l;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (kPair) {
    // barriers of both CTAs are initialised before either touches the other's
    cluster_arrive();
    cluster_wait();
  }
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;
  const int total_tiles = totals_smem[0];
  const Sched sched = {prefix_heavy, prefix_light, totals_smem[1], total_tiles};
  auto decode = [&](int s) -> Tile {
    if constexpr (kEpi == EPI_WGRAD) return decode_tile_wgrad(p, prefix_heavy, C::TILE_M, s, kFmt == 2 ? 4 : 5, kFmt ? 1 : 0);
    else return decode_tile(sched, p, C::TILE_M, s);
  };

  // ---- tile sequence of this CTA (pair) ---------------------------------------------------
  // Static: schedule positions sched_id, sched_id + stride, ...  Dynamic: the first position is
  // sched_id as well; the following ones are drawn from a global counter by the leader's A-producer
  // warp (`fetcher`), which hands them to every other warp of the CTA pair through a ring in shared
  // memory.  next_tile(i) is what a non-fetching warp calls for its i-th tile (all lanes together);
  // it returns a negative number when the CTA is done (or a wait gave up).
  const bool dynamic = p.dynamic_sched != 0;
  const bool fetcher = dynamic && warp == 0 && cta_rank == 0;
  const uint32_t info_empty_target0 = kPair ? map_to_cta(info_empty_bar(0), 0) : info_empty_bar(0);
  auto next_tile = [&](int i) -> int {
    if (!dynamic || i == 0) {
      const int s = sched_id + i * sched_stride;
      return s < total_tiles ? s : -1;
    }
    const int q = (i - 1) % SCHED_RING;
    if (!mbar_wait<kPair>(info_full_bar(q), (uint32_t)((i - 1) / SCHED_RING) & 1u, wc, ST_SCHED_FULL)) return -1;
    const int s = ring[q];
    __syncwarp();
    if (lane == 0) {
      // the arrival address depends on the value read, so the slot is released only after the read
      const uint32_t target = info_empty_target0 + 8u * q + zero_after(s);
      if (kPair) mbar_arrive_cluster(target); else mbar_arrive(target);
    }
    return s;
  };

  if (warp == 0 || warp == PRODUCER_B_WARP) {
    // ================= producers ======================================================
    // Two single-thread producers share the ring: warp 0 loads the A tile and its scale chunk
    // (and announces the stage's byte count), the last warp loads the B tile and its scale
    // chunks.  One thread issuing every copy of a k-tile was the slowest stream of the kernel.
    const bool side_b = warp != 0;
    {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const uint32_t a_dst0 = smem_base + C::A_OFF, b_dst0 = smem_base + C::B_OFF;
      const uint32_t sfa_dst0 = smem_base + C::SFA_OFF, sfb_dst0 = smem_base + C::SFB_OFF;
      const uint32_t leader_full0 = kPair ? map_to_cta(full_bar(0), 0) : full_bar(0);
      const bool skip_loads = side_b && p.test_skip_b_loads != 0;
      int it = 0;
      int t = fetcher ? (sched_id < total_tiles ? sched_id : -1) : next_tile(0);
      while (t >= 0 && ok) {
        int fetched = 0;
        if (fetcher && lane == 0) fetched = atomicAdd(p.tile_counter, 1) + sched_stride;  // used after the k loop
        const Tile tile = decode(t);
        // the k-tiles of this tile: all of K, or (wgrad) the expert's range of it with the expert's own scale chunks
        const int k_tiles = kEpi == EPI_WGRAD ? tile.k_tiles : p.k_tiles;
        const int rest_k = kEpi == EPI_WGRAD ? tile.rest_k : p.rest_k;
        const int n0 = tile.n_tile * BN;
        const int my_row0 = tile.row0 + (int)cta_rank * BM;
        const int nblk0 = n0 / 128;
        const CUtensorMap* bmap = &tmap_b;
        const CUtensorMap* sfbmap = &tmap_sfb;
        if (kDiscrete && side_b) {
          bmap = p.b_maps + tile.expert;
          tensormap_fence_acquire(bmap);
          sfbmap = p.b_maps + p.num_experts + tile.expert;
          tensormap_fence_acquire(sfbmap);
        }
        // weights that only one or two row tiles will ever read pass through L2 with the lowest
        // priority, so that they do not push out the activations and the weight tiles other CTAs share
        const bool b_stream = tile.m_tiles <= p.stream_m_tiles;
        constexpr uint64_t b_policy = L2_EVICT_FIRST;
        // Everything that changes per k-tile is a running value: the K coordinate, the scale-chunk
        // pointers and the stage's shared-memory / barrier addresses.
        int kc = kEpi == EPI_WGRAD ? tile.k0 : 0;
        if constexpr (kPair) {
          // every load of either CTA credits the leader's barrier of this stage
          const int b_row = n0 + (int)cta_rank * 128;
          const int m_blk = my_row0 / BM;
          for (int kt = 0; kt < k_tiles; ++kt, kc += BK) {
            if (!__all_sync(0xffffffffu, mbar_wait(empty_bar(stage), phase ^ 1, wc, ST_PRODUCER_EMPTY))) { ok = false; break; }
            const uint32_t fb = leader_full0 + 8u * stage;
            if (elect_one() && !skip_loads) {
              if (kEpi == EPI_WGRAD) {
                // scale chunks are addressed by their index in the operand's whole chunk array: the experts' blocks
                // follow one another, each [128-row block][chunk along K]
                if (!side_b) {
                  if (cta_rank == 0) mbar_arrive_expect_tx(full_bar(stage), C::TX_BYTES);
                  tma_load_2d_pair(a_dst0 + stage * A_STAGE_BYTES, &tmap_a, fb, kc, my_row0);
                  tma_load_2d_pair(sfa_dst0 + stage * SFA_STAGE_BYTES, &tmap_sfa, fb, 0,
                                   tile.chunk0 * ((p.m_rows + BM - 1) / BM) + m_blk * rest_k + kt * CPK);
                } else {
                  tma_load_2d_pair(b_dst0 + stage * C::B_STAGE_BYTES, bmap, fb, kc, b_row);
                  const int c = tile.chunk0 * p.n_blocks + nblk0 * rest_k + kt * CPK;
                  tma_load_2d_pair(sfb_dst0 + stage * SFB_STAGE_BYTES, sfbmap, fb, 0, c);
                  tma_load_2d_pair(sfb_dst0 + stage * SFB_STAGE_BYTES + 512 * CPK, sfbmap, fb, 0, c + rest_k);
                }
              } else if (!side_b) {
                if (cta_rank == 0) mbar_arrive_expect_tx(full_bar(stage), C::TX_BYTES);
                tma_load_2d_pair(a_dst0 + stage * A_STAGE_BYTES, &tmap_a, fb, kc, my_row0);
                tma_load_3d_pair(sfa_dst0 + stage * SFA_STAGE_BYTES, &tmap_sfa, fb, 0, kt * CPK, m_blk);
              } else if (kDiscrete) {
                const int c0 = p.b_nmajor ? b_row : kc, c1 = p.b_nmajor ? kc : b_row;
                if (b_stream) tma_load_2d_pair_hint(b_dst0 + stage * C::B_STAGE_BYTES, bmap, fb, c0, c1, b_policy);
                else tma_load_2d_pair(b_dst0 + stage * C::B_STAGE_BYTES, bmap, fb, c0, c1);
                tma_load_3d_pair(sfb_dst0 + stage * SFB_STAGE_BYTES, sfbmap, fb, 0, kt * CPK, nblk0);
              } else {
                const int c0 = p.b_nmajor ? b_row : kc, c1 = p.b_nmajor ? kc : b_row;
                if (b_stream) tma_load_3d_pair_hint(b_dst0 + stage * C::B_STAGE_BYTES, bmap, fb, c0, c1, tile.expert, b_policy);
                else tma_load_3d_pair(b_dst0 + stage * C::B_STAGE_BYTES, bmap, fb, c0, c1, tile.expert);
                tma_load_4d_pair(sfb_dst0 + stage * SFB_STAGE_BYTES, sfbmap, fb, 0, kt * CPK, nblk0, tile.expert);
              }
            }
            __syncwarp();
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
        } else {
          // scale chunks of B: per-expert tensor maps in discrete mode (a 128-row block beyond N reads as
          // zeros and still counts its bytes), plain bulk copies of the chunks that exist otherwise
          const bool two_chunks = kDiscrete || p.n_blocks - nblk0 >= 2;
          if (!side_b) {
            const uint8_t* sfa_src = p.sfa + (int64_t)(tile.row0 / BM) * rest_k * 512;
            if constexpr (kEpi == EPI_WGRAD) sfa_src += (int64_t)tile.chunk0 * ((p.m_rows + BM - 1) / BM) * 512;
            for (int kt = 0; kt < k_tiles; ++kt, kc += BK, sfa_src += 512 * CPK) {
              if (!__all_sync(0xffffffffu, mbar_wait(empty_bar(stage), phase ^ 1, wc, ST_PRODUCER_EMPTY))) { ok = false; break; }
              const uint32_t fb = full_bar(stage);
              // scale chunks this k-tile has (the last k-tile of a row block may have fewer than CPK)
              const uint32_t sf_bytes = 512u * (uint32_t)min(CPK, rest_k - kt * CPK);
              const uint32_t tx = A_STAGE_BYTES + C::B_STAGE_BYTES + sf_bytes + (kDiscrete ? (uint32_t)SFB_STAGE_BYTES : (two_chunks ? 2u : 1u) * sf_bytes);
              if (elect_one()) {
                mbar_arrive_expect_tx(fb, tx);
                tma_load_2d(a_dst0 + stage * A_STAGE_BYTES, &tmap_a, fb, kc, tile.row0);
                bulk_load(sfa_dst0 + stage * SFA_STAGE_BYTES, sfa_src, sf_bytes, fb);
              }
              __syncwarp();
              if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
          } else {
            const uint8_t* sfb_src0 = kDiscrete ? nullptr
                                      : (kEpi == EPI_WGRAD ? p.sfb + ((int64_t)tile.chunk0 * p.n_blocks + (int64_t)nblk0 * rest_k) * 512
                                                           : p.sfb + (int64_t)tile.expert * p.sfb_expert_bytes + (int64_t)nblk0 * rest_k * 512);
            const uint8_t* sfb_src1 = sfb_src0 + (int64_t)rest_k * 512;
            for (int kt = 0; kt < k_tiles; ++kt, kc += BK, sfb_src0 += 512 * CPK, sfb_src1 += 512 * CPK) {
              if (!__all_sync(0xffffffffu, mbar_wait(empty_bar(stage), phase ^ 1, wc, ST_PRODUCER_EMPTY))) { ok = false; break; }
              const uint32_t fb = full_bar(stage);
              if (elect_one() && !skip_loads) {
                const uint32_t b_dst = b_dst0 + stage * C::B_STAGE_BYTES;
                // B tile: one box of 256 rows x 128 K bytes, or (N-major) two slabs of 128 columns x 128 K rows
                const int c0 = p.b_nmajor ? n0 : kc, c1 = p.b_nmajor ? kc : n0;
                if (kDiscrete) {
                  if (b_stream) {
                    tma_load_2d_hint(b_dst, bmap, fb, c0, c1, b_policy);
                    if (p.b_nmajor) tma_load_2d_hint(b_dst + 128 * BK, bmap, fb, n0 + 128, kc, b_policy);
                  } else {
                    tma_load_2d(b_dst, bmap, fb, c0, c1);
                    if (p.b_nmajor) tma_load_2d(b_dst + 128 * BK, bmap, fb, n0 + 128, kc);
                  }
                  tma_load_3d(sfb_dst0 + stage * SFB_STAGE_BYTES, sfbmap, fb, 0, kt * CPK, nblk0);
                } else if constexpr (kEpi == EPI_WGRAD) {
                  tma_load_2d(b_dst, bmap, fb, kc, n0);  // B is [n, T]: no expert dimension
                  const uint32_t sf_bytes = 512u * (uint32_t)min(CPK, rest_k - kt * CPK);
                  bulk_load(sfb_dst0 + stage * SFB_STAGE_BYTES, sfb_src0, sf_bytes, fb);
                  if (two_chunks) bulk_load(sfb_dst0 + stage * SFB_STAGE_BYTES + 512 * CPK, sfb_src1, sf_bytes, fb);
                } else {
                  if (b_stream) {
                    tma_load_3d_hint(b_dst, bmap, fb, c0, c1, tile.expert, b_policy);
                    if (p.b_nmajor) tma_load_3d_hint(b_dst + 128 * BK, bmap, fb, n0 + 128, kc, tile.expert, b_policy);
                  } else {
                    tma_load_3d(b_dst, bmap, fb, c0, c1, tile.expert);
                    if (p.b_nmajor) tma_load_3d(b_dst + 128 * BK, bmap, fb, n0 + 128, kc, tile.expert);
                  }
                  const uint32_t sf_bytes = 512u * (uint32_t)min(CPK, rest_k - kt * CPK);
                  bulk_load(sfb_dst0 + stage * SFB_STAGE_BYTES, sfb_src0, sf_bytes, fb);
                  if (two_chunks) bulk_load(sfb_dst0 + stage * SFB_STAGE_BYTES + 512 * CPK, sfb_src1, sf_bytes, fb);
                }
              }
              __syncwarp();
              if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
          }
        }
        if (!ok) break;
        ++it;
        if (fetcher) {
          // hand the next position (or the end mark) to every other warp of the CTA pair, then take it
          fetched = __shfl_sync(0xffffffffu, fetched, 0);
          const int next = fetched < total_tiles ? fetched : -1;
          const int q = (it - 1) % SCHED_RING;
          if (!__all_sync(0xffffffffu, mbar_wait(info_empty_bar(q), ((uint32_t)((it - 1) / SCHED_RING) & 1u) ^ 1u, wc, ST_SCHED_EMPTY))) { ok = false; break; }
          if (lane == 0) {
            ring[q] = next;
            mbar_arrive(info_full_bar(q));
            if (kPair) {
              st_shared_cluster(map_to_cta(smem_u32(const_cast<int*>(&ring[q])), 1), (uint32_t)next);
              mbar_arrive_cluster_release(map_to_cta(info_full_bar(q), 1));
            }
          }
          __syncwarp();
          t = next;
        } else {
          t = next_tile(it);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ================= MMA issuer (the leader CTA only, in pair mode) =====================
    if (cta_rank == 0) {
      // The whole warp walks the loop (so it stays convergent); one elected lane issues.
      // The issuing thread is a serial instruction stream: four MMAs, three scale copies and a
      // commit per k-tile must cost as few instructions as possible, so every descriptor is
      // (constant high word, running low word) and the instruction descriptors are immediates.
      // B in N-major form: bit 16 of the instruction descriptor, 128-column slabs 16 KB apart
      // (leading byte offset), 32 K rows = 4096 bytes per MMA.
      const uint32_t idesc = (make_idesc_mxf8(C::TILE_M, BN) | p.ab_format | (p.b_nmajor ? (1u << 16) : 0u)) & ~(p.sf_e4m3 ? (1u << 23) : 0u);
      constexpr uint32_t AB_HI = (1024u >> 4) | (1u << 14) | (2u << 29);  // SBO 1024, version 1, 128-byte swizzle
      constexpr uint32_t SF_HI = (128u >> 4) | (1u << 14);                // SBO 128, version 1, no swizzle
      constexpr uint32_t AB_LBO = 1u << 16;                               // leading byte offset 16 (unused by swizzled K-major)
      const uint32_t a_lo0 = ((smem_base + C::A_OFF) >> 4) | AB_LBO;
      const uint32_t b_lo0 = ((smem_base + C::B_OFF) >> 4) | (p.b_nmajor ? ((uint32_t)(128 * BK) >> 4) << 16 : AB_LBO);
      const uint32_t b_kstep = p.b_nmajor ? (32u * 128u) >> 4 : 2u;  // 32 K elements further, in 16-byte units
      const uint32_t sfa_lo0 = (smem_base + C::SFA_OFF) >> 4;
      const uint32_t sfb_lo0 = (smem_base + C::SFB_OFF) >> 4;
      auto desc = [](uint32_t lo, uint32_t hi) { return ((uint64_t)hi << 32) | lo; };
      int stage = 0;
      uint32_t phase = 0;
      uint32_t sf_buf = 0;
      int it = 0;
      bool ok = true;
      for (int t = next_tile(0); t >= 0 && ok; t = next_tile(++it)) {
        const uint32_t acc = tmem_base + ((it & 1) ? TMEM_ACC1_COL : 0);
        // (wgrad: the tile's K range is read from the offsets before the wait below, not between the previous
        // tile's last MMA and this tile's first)
        int k_tiles = p.k_tiles, k_bytes = p.k_bytes;
        if constexpr (kEpi == EPI_WGRAD) {
          const Tile tile = decode(t);
          k_tiles = tile.k_tiles;
          k_bytes = tile.kbytes;
        }
        if (it > 0) {
          // previous tile's epilogue has drained the 32 columns both accumulators share
          if (!__all_sync(0xffffffffu, mbar_wait(overlap_bar, (it - 1) & 1, wc, ST_MMA_OVERLAP))) { ok = false; break; }
          tc_fence_after();
        }
        for (int kt = 0; kt < k_tiles; ++kt) {
          // the stage's bytes were written by TMA (async proxy) and are made visible by the barrier's
          // transaction count; no tcgen05 fence is needed between this wait and the MMAs
          // (the outcome is voted so that a wait that gives up takes the whole warp out of the loop)
          bool landed = mbar_try_wait(full_bar(stage), phase);
          if (!landed) landed = mbar_wait(full_bar(stage), phase, wc, ST_MMA_FULL);
          if (!__all_sync(0xffffffffu, landed)) { ok = false; break; }
          // scale chunks: 8-bit operands alternate between two TMEM buffers; E2M1 operands have one
          // (tcgen05.cp and tcgen05.mma of one thread execute in issue order)
          const uint32_t sfa_t = tmem_base + TMEM_SF_COL + (kFmt ? 0 : 16 * sf_buf);
          const uint32_t sfb_t = sfa_t + (kFmt ? 16 : 4);
          const uint32_t a_lo = a_lo0 + stage * (A_STAGE_BYTES >> 4);
          const uint32_t b_lo = b_lo0 + stage * (C::B_STAGE_BYTES >> 4);
          const uint32_t sfa_lo = sfa_lo0 + stage * (SFA_STAGE_BYTES >> 4);
          const uint32_t sfb_lo = sfb_lo0 + stage * (SFB_STAGE_BYTES >> 4);
          const uint32_t not_first = kt != 0;
          const int k_left = k_bytes - kt * BK;  // bytes of K this k-tile still has
          if (elect_one()) {
            // chunk g of SFA -> 4 columns; chunk g of both 128-row blocks of SFB -> 8 columns side by side.
            // (in pair mode one instruction acts on both CTAs: each copies from its own smem to its own TMEM)
#pragma unroll
            for (int g = 0; g < CPK; ++g) {
              tmem_cp_sf_any<kPair>(sfa_t + 4 * g, desc(sfa_lo + 32 * g, SF_HI));
              tmem_cp_sf_any<kPair>(sfb_t + 8 * g, desc(sfb_lo + 32 * g, SF_HI));
              tmem_cp_sf_any<kPair>(sfb_t + 8 * g + 4, desc(sfb_lo + 32 * (CPK + g), SF_HI));
            }
            // MMA j reads bytes [32 j, 32 j + 32) of K (+2 in 16-byte units inside the 128-byte swizzle row) and
            // the scales of those elements: byte j of the chunk (kFmt 0), bytes 2 (j & 1) .. + 1 of chunk
            // j / 2 (kFmt 1), chunk j (kFmt 2)
            auto mma = [&](int j, uint32_t acc_flag) {
              const uint32_t sf_id = kFmt == 0 ? (uint32_t)j : (kFmt == 1 ? 2u * (j & 1) : 0u);
              const uint32_t chunk = kFmt == 0 ? 0u : (kFmt == 1 ? (uint32_t)(j >> 1) : (uint32_t)j);
              mma_block_scaled<kFmt, kPair>(acc, desc(a_lo + 2 * j, AB_HI), desc(b_lo + j * b_kstep, AB_HI), idesc_with_sf_id(idesc, sf_id, sf_id),
                                            sfa_t + 4 * chunk, sfb_t + 8 * chunk, acc_flag);
            };
            if (k_left >= BK) {
              mma(0, not_first);
              mma(1, 1);
              mma(2, 1);
              mma(3, 1);
            } else {
              const int kblocks = (k_left + 31) / 32;
              for (int kb = 0; kb < kblocks; ++kb) mma(kb, (kt | kb) != 0);
            }
            if constexpr (kPair) tc_commit_pair(empty_bar(stage), 3);  // frees this stage in both CTAs
            else tc_commit(empty_bar(stage));  // frees the smem stage once these MMAs have read it
          }
          __syncwarp();
          sf_buf ^= 1;
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        // the commit must come from the lane that issued the MMAs: elect.sync picks the same lane of
        // an unchanged, fully active warp every time
        if (ok && elect_one()) {
          if constexpr (kPair) tc_commit_pair(acc_full_bar(it & 1), 3);
          else tc_commit(acc_full_bar(it & 1));
        }
        __syncwarp();
      }
    }
    __syncwarp();
  } else {
    // ================= epilogue =========================================================
    const int ew = warp - 2;            // 0..7
    const int quarter = warp & 3;       // TMEM lanes [32 quarter, 32 quarter + 32) belong to this warp
    const int half = ew >> 2;           // column half of the tile: [128 half, 128 half + 128)
    const int r_in_tile = quarter * 32 + lane;
    const float norm_const = p.norm_const ? *p.norm_const : 1.0f;
    const bool wide = p.wide_stores != 0;
    const bool c_f16 = p.c_f16 != 0, d_f16 = p.d_f16 != 0;
    const OutFormat out_fmt = {p.d_rcp_limit, p.d_e5m2 != 0, p.d_is_fp8 == 0, d_f16};
    const int64_t d_row_bytes = (int64_t)p.n_out * (p.d_is_fp8 ? 1 : 2);
    const uint32_t colq_scratch = smem_base + C::COLQ_OFF + ew * 256;
    uint8_t* const stage_row = smem + C::STAGING_OFF + ew * STAGING_WARP_BYTES + lane * STAGING_ROW_BYTES;  // kBulk only
    const uint32_t overlap_target = kPair ? map_to_cta(overlap_bar, 0) : overlap_bar;
    auto arrive_overlap = [&]() {
      if (kPair) mbar_arrive_cluster(overlap_target); else mbar_arrive(overlap_bar);
    };
    // amax: a warp keeps the running maximum of the expert it is working on and sends it (one atomic per warp) when
    // the expert changes and after its last tile: max is associative, so the result is the same as with one atomic
    // per warp and tile on the few amax words
    int amax_expert = -1;
    float run_amax = 0.f, run_amax_up = 0.f;
    auto flush_amax = [&]() {
      if (p.amax == nullptr || amax_expert < 0) return;
      float wmax = run_amax, wmax_up = run_amax_up;
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) {
        wmax = fmaxf(wmax, __shfl_xor_sync(0xffffffffu, wmax, d));
        if (kEpi == EPI_DSWIGLU) wmax_up = fmaxf(wmax_up, __shfl_xor_sync(0xffffffffu, wmax_up, d));
      }
      // non-negative floats order like their bit patterns; -inf (the caller's initial value) has a negative
      // pattern, so a signed integer max is exact.  dSwiGLU: amax[expert][0] = d_gate, amax[expert][1] = d_up
      if (lane == 0) {
        atomicMax(reinterpret_cast<int*>(p.amax) + (kEpi == EPI_DSWIGLU ? 2 * amax_expert : amax_expert), __float_as_int(wmax));
        if (kEpi == EPI_DSWIGLU) atomicMax(reinterpret_cast<int*>(p.amax) + 2 * amax_expert + 1, __float_as_int(wmax_up));
      }
    };
    int it = 0;
    bool ok = true;
    for (int t = next_tile(0); t >= 0 && ok; t = next_tile(++it)) {
      Tile tile = decode(t);
      if (tile.expert != amax_expert) {
        flush_amax();
        amax_expert = tile.expert;
        run_amax = run_amax_up = 0.f;
      }
      tile.row0 += (int)cta_rank * BM;  // this CTA's 128 rows
      const int n0 = tile.n_tile * BN;
      const int row = tile.row0 + r_in_tile;
      // in pair mode the second half of a 256-row tile may lie beyond the expert's last row
      const bool row_ok = row < min(p.m_rows, tile.row_end);
      // wgrad: the product of the two optional per-expert global scales
      const float alpha = kEpi == EPI_WGRAD ? (p.alpha ? p.alpha[tile.expert] : 1.0f) * (p.beta ? p.beta[tile.expert] : 1.0f) : p.alpha[tile.expert];
      const float prob = (p.prob && row_ok) ? p.prob[row] : 1.0f;
      int out_row = (p.d_row_map && row_ok) ? p.d_row_map[row] : row;
      // destination of this thread's bf16 D row: d, or the buffer of the rank the row returns to
      __nv_bfloat16* d_rows = reinterpret_cast<__nv_bfloat16*>(p.d);
      if (p.d_peer_ptrs && out_row >= 0) {
        const int64_t rank = out_row / p.d_peer_slots;
        d_rows = reinterpret_cast<__nv_bfloat16*>(p.d_peer_ptrs[rank]);
        out_row -= (int)(rank * p.d_peer_slots);
      }
      const uint32_t acc = tmem_base + ((it & 1) ? TMEM_ACC1_COL : 0) + ((uint32_t)(quarter * 32) << 16);
      const bool reverse = (it & 1) == 0;  // even tiles drain from the top (shared columns first)
      float thread_amax = 0.f;
      uint32_t sf_row_word = 0;  // four E8M0 bytes of this row (K group = 128 output columns)

      if constexpr (kEpi == EPI_DSWIGLU) {
        // this row's part of the forward C that the tile reads (512 bytes when 16-bit) is requested into L2
        // before the wait for the accumulator: the loads of the four blocks below then find it there
        if (row_ok) {
          const int c_bytes = (p.c_in_dtype == B200MOE_DTYPE_E4M3 || p.c_in_dtype == B200MOE_DTYPE_E5M2) ? 1 : 2;
          const int g0 = n0 + half * 128;  // first column of G of this warp
          const uint8_t* c0 = reinterpret_cast<const uint8_t*>(p.c_in) + ((int64_t)row * p.n_out + 2 * g0) * c_bytes;
#pragma unroll
          for (int q = 0; q < 4; ++q)
            if (q < 2 * c_bytes && g0 + q * (64 / c_bytes) < p.n) prefetch_l2(c0 + 128 * q);
        }
      }
      if (!mbar_wait(acc_full_bar(it & 1), (it >> 1) & 1, wc, ST_EPI_ACC)) { ok = false; break; }
      tc_fence_after();

      if (kEpi == EPI_FC1) {
        // 2 (gate, up) pairs per half: accumulator columns [128 half + 64 pp, +64)
#pragma unroll 1
        for (int i = 0; i < 2; ++i) {
          const int pp = reverse ? 1 - i : i;
          const int col = half * 128 + pp * 64;  // accumulator column of the gate block
          float g[32], u[32];
          tmem_ld_32x32(acc + col, g);
          tmem_ld_32x32(acc + col + 32, u);
          tmem_ld_wait();
          reg_fence32(g);
          reg_fence32(u);
          if (i == 0) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) arrive_overlap();
          }
          const int cn = n0 + col;          // column of C
          const int dn = (n0 >> 1) + half * 64 + pp * 32;  // column of D
          if (cn >= p.n) continue;
          if (p.bias) {
            // C = alpha * acc + bias (one FMA, as the reference's kernel), gate and up alike
            const int64_t b0 = (int64_t)tile.expert * p.n + cn;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              float bg[8], bu[8];
              load_bias8(p.bias, p.bias_dtype, b0 + j, bg);
              load_bias8(p.bias, p.bias_dtype, b0 + 32 + j, bu);
#pragma unroll
              for (int q = 0; q < 8; q += 2) {
                const float2 a2 = make_float2(alpha, alpha);
                const float2 rg = fma2(make_float2(g[j + q], g[j + q + 1]), a2, make_float2(bg[q], bg[q + 1]));
                const float2 ru = fma2(make_float2(u[j + q], u[j + q + 1]), a2, make_float2(bu[q], bu[q + 1]));
                g[j + q] = rg.x;
                g[j + q + 1] = rg.y;
                u[j + q] = ru.x;
                u[j + q + 1] = ru.y;
              }
            }
          } else {
            scale_inplace<32>(g, alpha);
            scale_inplace<32>(u, alpha);
          }
          if (p.c && row_ok) {
            store_bf16x32(p.c + (int64_t)row * p.n + cn, g, wide, c_f16);
            store_bf16x32(p.c + (int64_t)row * p.n + cn + 32, u, wide, c_f16);
          }
          if (p.act_geglu) {
            // GeGLU of the reference: gate <= 7, -7 <= up <= 7 (after the C store),
            // D = (up + 1) * gate * sigmoid(1.702 gate) * prob
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              const float2 gate = make_float2(fminf(g[j], 7.0f), fminf(g[j + 1], 7.0f));
              const float2 up = make_float2(fmaxf(fminf(u[j], 7.0f), -7.0f), fmaxf(fminf(u[j + 1], 7.0f), -7.0f));
              const float2 t = mul2(mul2(gate, 1.702f), -1.4426950408889634f);
              const float2 den = add2(make_float2(ex2_approx(t.x), ex2_approx(t.y)), 1.0f);
              const float2 s = make_float2(rcp_approx(den.x), rcp_approx(den.y));
              const float2 r = mul2(mul2(mul2(s, gate), add2(up, 1.0f)), prob);
              g[j] = r.x;
              g[j + 1] = r.y;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              const float2 gg = make_float2(g[j], g[j + 1]);
              const float2 t = mul2(gg, -1.4426950408889634f);
              const float2 d = add2(make_float2(ex2_approx(t.x), ex2_approx(t.y)), 1.0f);
              const float2 s = make_float2(rcp_approx(d.x), rcp_approx(d.y));
              const float2 r = mul2(mul2(mul2(s, gg), make_float2(u[j], u[j + 1])), prob);
              g[j] = r.x;
              g[j + 1] = r.y;
            }
          }
          if (p.amax && row_ok) {
#pragma unroll
            for (int j = 0; j < 32; ++j) thread_amax = fmaxf(thread_amax, fabsf(g[j]));
          }
          if (!p.gen_sfd) {
            if (row_ok && out_row >= 0) store_d32(d_rows, (int64_t)out_row * p.n_out + dn, g, wide, d_f16, p.d_f32 != 0);
          } else {
            if (row_ok) {
              const uint32_t sf = quant_row_block(reinterpret_cast<uint8_t*>(p.d) + (int64_t)row * d_row_bytes, dn, g, norm_const, wide, out_fmt);
              sf_row_word |= sf << (8 * (half * 2 + pp));
            }
            if (p.d_col) {
              // column scales: one byte per (column, 32-row block); rows beyond m_rows count as zero
              if (!row_ok) {
#pragma unroll
                for (int j = 0; j < 32; ++j) g[j] = 0.f;
              }
              const uint32_t sfc = quant_col_block(p.d_col + (int64_t)row * d_row_bytes, dn, row_ok, g, norm_const, wide, out_fmt, colq_scratch);
              int64_t blk_base = 0;
              int rb = (tile.row0 >> 5) + quarter;
              int rest = p.sfd_col_rest_k;
              if (p.discrete_col_sfd) {
                // per-expert block: rows counted from the expert's first row
                const int start = expert_first_row(p, tile.expert);
                blk_base = (int64_t)(start / 128) * ((p.n_out + 127) / 128) * 512;
                rb = ((tile.row0 - start) >> 5) + quarter;
                rest = ((p.offsets[tile.expert] - start) / 32 + 3) / 4;
              }
              if (tile.row0 + quarter * 32 < min(p.m_rows, tile.row_end)) p.sfd_col[blk_base + sf_offset(dn + lane, rb, rest)] = (uint8_t)sfc;
            }
          }
        }
        if (p.gen_sfd && row_ok && p.sfd_row) {
          // output columns [128 n_tile + 64 half, +64) = scale blocks 2 half, 2 half + 1 of K group n_tile
          uint8_t* dst = p.sfd_row + sf_offset(row, (int64_t)tile.n_tile * 4 + half * 2, p.sfd_row_rest_k);
          const int blocks_left = (p.n_out - ((n0 >> 1) + half * 64) + 31) / 32;
          if (blocks_left >= 2)
            *reinterpret_cast<uint16_t*>(dst) = (uint16_t)(sf_row_word >> (16 * half));
          else if (blocks_left == 1)
            *dst = (uint8_t)(sf_row_word >> (16 * half));
        }
      } else if constexpr (kEpi == EPI_WGRAD) {
        // plain store (or accumulation) of the expert's [m, n] tile, scaled by the expert's global scale
        const bool empty = tile.k_tiles == 0;  // an expert without tokens: nothing was accumulated
        // one [E, m, n] tensor, or (discrete output) one [m, n] allocation per expert behind a pointer array
        void* const d_out = p.d_peer_ptrs ? reinterpret_cast<void*>(p.d_peer_ptrs[tile.expert]) : p.d;
        const int64_t out_base = ((int64_t)(p.d_peer_ptrs ? 0 : tile.expert) * p.m_rows + row) * p.n;
#pragma unroll 1
        for (int i = 0; i < 4; ++i) {
          const int bb = reverse ? 3 - i : i;
          const int col = half * 128 + bb * 32;
          float v[32];
          tmem_ld_32x32(acc + col, v);
          tmem_ld_wait();
          reg_fence32(v);
          if (i == (kFmt ? 1 : 0)) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) arrive_overlap();
          }
          const int dn = n0 + col;
          if (dn >= p.n || !row_ok) continue;
          scale_inplace<32>(v, alpha);
          if (empty) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = 0.f;
          }
          if (p.accumulate) {
            if (p.d_f32) {
              const float4* src = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(d_out) + out_base + dn);
#pragma unroll
              for (int q = 0; q < 8; ++q) {
                const float4 o = src[q];
                v[4 * q] += o.x; v[4 * q + 1] += o.y; v[4 * q + 2] += o.z; v[4 * q + 3] += o.w;
              }
            } else {
              const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(d_out) + out_base + dn);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const uint4 o = src[q];
                const uint16_t* h = reinterpret_cast<const uint16_t*>(&o);
#pragma unroll
                for (int j = 0; j < 8; ++j)
                  v[8 * q + j] += d_f16 ? __half2float(__ushort_as_half(h[j])) : __uint_as_float((uint32_t)h[j] << 16);
              }
            }
          }
          store_d32(reinterpret_cast<__nv_bfloat16*>(d_out), out_base + dn, v, wide, d_f16, p.d_f32 != 0);
        }
      } else if constexpr (kEpi == EPI_DSWIGLU) {
        // 4 blocks of 32 accumulator columns per half; block b of the GEMM's N owns columns [64 b, 64 b + 64) of C and D
        const float alpha2 = alpha * alpha;
        const float beta = p.beta ? p.beta[tile.expert] : 1.0f;
        const int c_bytes = (p.c_in_dtype == B200MOE_DTYPE_E4M3 || p.c_in_dtype == B200MOE_DTYPE_E5M2) ? 1 : 2;
        const uint8_t* c_row = reinterpret_cast<const uint8_t*>(p.c_in) + (int64_t)row * p.n_out * c_bytes;
        float dprob_sum = 0.f, amax_up = 0.f;  // thread_amax collects d_gate, amax_up collects d_up
#pragma unroll 1
        for (int i = 0; i < 4; ++i) {
          const int bb = reverse ? 3 - i : i;
          const int col = half * 128 + bb * 32;
          const int dn = n0 + col;  // column of the GEMM result
          const bool live = dn < p.n;
          // this row's gate and up block of the forward C (64 consecutive elements), requested before the TMEM load
          uint4 craw[8];
          if (live && row_ok) {
            const uint4* src = reinterpret_cast<const uint4*>(c_row + (int64_t)dn * 2 * c_bytes);
#pragma unroll
            for (int q = 0; q < 8; ++q)
              if (q < 4 * c_bytes) craw[q] = __ldg(src + q);
          } else {
#pragma unroll
            for (int q = 0; q < 8; ++q) craw[q] = make_uint4(0, 0, 0, 0);
          }
          float v[32];
          tmem_ld_32x32(acc + col, v);
          tmem_ld_wait();
          reg_fence32(v);
          if (i == (kFmt ? 1 : 0)) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) arrive_overlap();
          }
          if (!live) continue;
          float d1[32];  // d_gate; v becomes d_up
          const bool c_e5m2 = p.c_in_dtype == B200MOE_DTYPE_E5M2, c_is_f16 = p.c_in_dtype == B200MOE_DTYPE_F16;
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            // elements j, j + 1 of the gate block and of the up block
            float2 cg, cu;
            if (c_bytes == 2) {
              const uint32_t* w = reinterpret_cast<const uint32_t*>(craw);
              const uint32_t wg = w[j >> 1], wu = w[16 + (j >> 1)];
              if (c_is_f16) {
                cg = __half22float2(*reinterpret_cast<const __half2*>(&wg));
                cu = __half22float2(*reinterpret_cast<const __half2*>(&wu));
              } else {
                cg = make_float2(__uint_as_float(wg << 16), __uint_as_float(wg & 0xffff0000u));
                cu = make_float2(__uint_as_float(wu << 16), __uint_as_float(wu & 0xffff0000u));
              }
            } else {
              const uint8_t* b8 = reinterpret_cast<const uint8_t*>(craw);
              cg = make_float2(fp8_to_float(b8[j], c_e5m2), fp8_to_float(b8[j + 1], c_e5m2));
              cu = make_float2(fp8_to_float(b8[32 + j], c_e5m2), fp8_to_float(b8[33 + j], c_e5m2));
            }
            // the reference kernel's operation order, every product and sum rounded on its own (two elements per instruction)
            const float2 g = mul2(make_float2(v[j], v[j + 1]), alpha2);
            const float2 gate = mul2(cg, beta);
            const float2 up = mul2(cu, beta);
            const float2 t = mul2(gate, -1.4426950408889634f);
            const float2 den = add2(make_float2(ex2_approx(t.x), ex2_approx(t.y)), 1.0f);
            const float2 sig = make_float2(rcp_approx(den.x), rcp_approx(den.y));
            const float2 swish = mul2(gate, sig);
            const float2 dp = mul2(mul2(up, swish), g);
            dprob_sum = __fadd_rn(__fadd_rn(dprob_sum, dp.x), dp.y);
            const float2 gp = mul2(g, prob);
            const float2 dup = mul2(gp, swish);
            v[j] = dup.x;
            v[j + 1] = dup.y;
            // 1 - sig as one fused multiply-add (sig * -1 is exact, so the rounding is the subtraction's)
            const float2 one_minus_sig = fma2(sig, make_float2(-1.0f, -1.0f), make_float2(1.0f, 1.0f));
            const float2 dsig1 = add2(mul2(gate, one_minus_sig), 1.0f);
            const float2 dg = mul2(mul2(mul2(gp, up), sig), dsig1);
            d1[j] = dg.x;
            d1[j + 1] = dg.y;
          }
          if (p.amax && row_ok) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              thread_amax = fmaxf(thread_amax, fabsf(d1[j]));
              amax_up = fmaxf(amax_up, fabsf(v[j]));
            }
          }
          const int64_t on = 2 * (int64_t)dn;  // column of D of the gate block; the up block follows it
          if (!p.gen_sfd) {
            if (row_ok) {
              store_d32(d_rows, (int64_t)row * p.n_out + on, d1, wide, d_f16, p.d_f32 != 0);
              store_d32(d_rows, (int64_t)row * p.n_out + on + 32, v, wide, d_f16, p.d_f32 != 0);
            }
          } else {
            if (row_ok) {
              uint8_t* d_row_base = reinterpret_cast<uint8_t*>(p.d) + (int64_t)row * d_row_bytes;
              const uint32_t sf1 = quant_row_block(d_row_base, on, d1, norm_const, wide, out_fmt);
              const uint32_t sf2 = quant_row_block(d_row_base, on + 32, v, norm_const, wide, out_fmt);
              // scale blocks 2 (dn / 32) and 2 (dn / 32) + 1 of this row: two adjacent bytes of one K group
              if (p.sfd_row) *reinterpret_cast<uint16_t*>(p.sfd_row + sf_offset(row, on >> 5, p.sfd_row_rest_k)) = (uint16_t)(sf1 | (sf2 << 8));
            }
            if (p.d_col) {
              if (!row_ok) {
#pragma unroll
                for (int j = 0; j < 32; ++j) { d1[j] = 0.f; v[j] = 0.f; }
              }
              int64_t blk_base = 0;
              int rb = (tile.row0 >> 5) + quarter;
              int rest = p.sfd_col_rest_k;
              if (p.discrete_col_sfd) {
                const int start = expert_first_row(p, tile.expert);
                blk_base = (int64_t)(start / 128) * ((p.n_out + 127) / 128) * 512;
                rb = ((tile.row0 - start) >> 5) + quarter;
                rest = ((p.offsets[tile.expert] - start) / 32 + 3) / 4;
              }
              const bool rows_live = tile.row0 + quarter * 32 < min(p.m_rows, tile.row_end);
              uint8_t* d_col_base = p.d_col + (int64_t)row * d_row_bytes;
              const uint32_t sfc1 = quant_col_block(d_col_base, on, row_ok, d1, norm_const, wide, out_fmt, colq_scratch);
              if (rows_live) p.sfd_col[blk_base + sf_offset(on + lane, rb, rest)] = (uint8_t)sfc1;
              const uint32_t sfc2 = quant_col_block(d_col_base, on + 32, row_ok, v, norm_const, wide, out_fmt, colq_scratch);
              if (rows_live) p.sfd_col[blk_base + sf_offset(on + 32 + lane, rb, rest)] = (uint8_t)sfc2;
            }
          }
        }
        if (p.dprob && row_ok) atomicAdd(p.dprob + row, dprob_sum);
        run_amax_up = fmaxf(run_amax_up, amax_up);
      } else {
        // FC2: 4 blocks of 32 columns per half
        if constexpr (kBulk) bulk_wait_read0();  // the previous tile's row copies have left the staging area
#pragma unroll 1
        for (int i = 0; i < 4; ++i) {
          const int bb = reverse ? 3 - i : i;
          const int col = half * 128 + bb * 32;
          float v[32];
          tmem_ld_32x32(acc + col, v);
          tmem_ld_wait();
          reg_fence32(v);
          // the accumulators share 32 columns (48 with E2M1 operands: two blocks)
          if (i == (kFmt ? 1 : 0)) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) arrive_overlap();
          }
          const int dn = n0 + col;
          if (dn >= p.n) continue;
          if (p.bias) {
            // D = alpha * acc + bias * prob: the reference's fused form (prob scales the bias only)
            const int64_t b0 = (int64_t)tile.expert * p.n + dn;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              float bv[8];
              load_bias8(p.bias, p.bias_dtype, b0 + j, bv);
#pragma unroll
              for (int q = 0; q < 8; q += 2) {
                const float2 r = fma2(make_float2(v[j + q], v[j + q + 1]), make_float2(alpha, alpha), mul2(make_float2(bv[q], bv[q + 1]), prob));
                v[j + q] = r.x;
                v[j + q + 1] = r.y;
              }
            }
          } else {
            scale_inplace<32>(v, alpha);
            scale_inplace<32>(v, prob);
          }
          if (p.amax && row_ok) {
#pragma unroll
            for (int j = 0; j < 32; ++j) thread_amax = fmaxf(thread_amax, fabsf(v[j]));
          }
          if (!p.gen_sfd) {
            if constexpr (kBulk) {
              // this row's 32 columns -> its slot of the staging area (64 bytes)
              uint4* st = reinterpret_cast<uint4*>(stage_row + bb * 64);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                uint4 o;
                o.x = pack16x2_from_float(v[8 * q + 0], v[8 * q + 1], d_f16);
                o.y = pack16x2_from_float(v[8 * q + 2], v[8 * q + 3], d_f16);
                o.z = pack16x2_from_float(v[8 * q + 4], v[8 * q + 5], d_f16);
                o.w = pack16x2_from_float(v[8 * q + 6], v[8 * q + 7], d_f16);
                st[q] = o;
              }
            } else {
              if (row_ok && out_row >= 0) store_d32(d_rows, (int64_t)out_row * p.n_out + dn, v, wide, d_f16, p.d_f32 != 0);
            }
          } else {
            if (row_ok) {
              const uint32_t sf = quant_row_block(reinterpret_cast<uint8_t*>(p.d) + (int64_t)row * d_row_bytes, dn, v, norm_const, wide, out_fmt);
              sf_row_word |= sf << (8 * bb);
            }
            if (p.d_col) {
              if (!row_ok) {
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = 0.f;
              }
              const uint32_t sfc = quant_col_block(p.d_col + (int64_t)row * d_row_bytes, dn, row_ok, v, norm_const, wide, out_fmt, colq_scratch);
              int64_t blk_base = 0;
              int rb = (tile.row0 >> 5) + quarter;
              int rest = p.sfd_col_rest_k;
              if (p.discrete_col_sfd) {
                const int start = expert_first_row(p, tile.expert);
                blk_base = (int64_t)(start / 128) * ((p.n_out + 127) / 128) * 512;
                rb = ((tile.row0 - start) >> 5) + quarter;
                rest = ((p.offsets[tile.expert] - start) / 32 + 3) / 4;
              }
              if (tile.row0 + quarter * 32 < min(p.m_rows, tile.row_end)) p.sfd_col[blk_base + sf_offset(dn + lane, rb, rest)] = (uint8_t)sfc;
            }
          }
        }
        if constexpr (kBulk) {
          if (!p.gen_sfd) {
            // one asynchronous copy per row: up to 128 columns = 256 contiguous bytes at the destination
            fence_proxy_async_smem();
            const int c0 = n0 + half * 128;
            const int ncols = min(128, p.n - c0);
            if (row_ok && out_row >= 0 && ncols > 0)
              bulk_store(d_rows + (int64_t)out_row * p.n_out + c0, smem_u32(stage_row), (uint32_t)ncols * 2);
            bulk_commit();
          }
        }
        if (p.gen_sfd && row_ok && p.sfd_row) {
          // output columns [256 n_tile + 128 half, +128) = K group 2 n_tile + half, 4 blocks
          uint8_t* dst = p.sfd_row + sf_offset(row, (int64_t)(tile.n_tile * 2 + half) * 4, p.sfd_row_rest_k);
          const int blocks_left = (p.n_out - (n0 + half * 128) + 31) / 32;
          if (blocks_left >= 4) {
            *reinterpret_cast<uint32_t*>(dst) = sf_row_word;
          } else {
            for (int b = 0; b < blocks_left; ++b) dst[b] = (uint8_t)(sf_row_word >> (8 * b));
          }
        }
      }

      run_amax = fmaxf(run_amax, thread_amax);
    }
    flush_amax();
  }

  // ---- teardown ----------------------------------------------------------------------
  if constexpr (kBulk) bulk_wait_all();  // row copies still reading this CTA's shared memory
  tc_fence_before();
  __syncthreads();
  if (kPair) {
    // the peer may still arrive on this CTA's barriers and the leader's MMAs write the peer's TMEM:
    // neither CTA frees anything before both are done
    cluster_arrive();
    cluster_wait();
  }
  if (warp == 1) {
    tc_fence_after();
    if (kPair) tmem_dealloc_pair(tmem_base, TMEM_COLS);
    else tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------
// Discrete weights: build one tensor map per expert in the caller's workspace.  The host
// encodes a prototype map of an [n, k] matrix; this kernel copies it per expert and patches
// the global address with the pointer read from the device-resident pointer array, so the
// host never needs the pointer values (the launch stays capturable in a CUDA graph).
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(32)
    build_expert_tensormaps_kernel(const __grid_constant__ CUtensorMap proto_b, const __grid_constant__ CUtensorMap proto_sfb,
                                   const int64_t* b_ptrs, const int64_t* sfb_ptrs, const void* fallback_b, const void* fallback_sf,
                                   CUtensorMap* out, int num_experts) {
  // slots [0, E): weight maps; slots [E, 2E): scale-factor maps
  __shared__ __align__(128) CUtensorMap s_map;
  const int slot = blockIdx.x;
  if (slot >= 2 * num_experts) return;
  const bool is_sf = slot >= num_experts;
  const int e = is_sf ? slot - num_experts : slot;
  const int lane = threadIdx.x;
  const uint32_t* proto = reinterpret_cast<const uint32_t*>(is_sf ? &proto_sfb : &proto_b);
  reinterpret_cast<uint32_t*>(&s_map)[lane] = proto[lane];
  __syncwarp();
  if (lane == 0) {
    uint64_t addr = (uint64_t)(is_sf ? sfb_ptrs[e] : b_ptrs[e]);
    const uint32_t map_smem = smem_u32(&s_map);
    if (addr == 0 || (addr & 15)) {
      // A misaligned or null pointer would fault the TMA unit.  Record it, point the map at memory
      // that is known to be valid (the caller's A / SFA) and shrink the map's extents to what that
      // memory surely holds (16 bytes of A, one 512-byte chunk of SFA): every load through the map
      // then reads at most that and fills the rest of its box with zeros.  The expert's results are
      // meaningless; the status word says why.
      atomicCAS(&g_device_status, 0, 201);
      addr = (uint64_t)(is_sf ? fallback_sf : fallback_b);
      if (!is_sf) asm volatile("tensormap.replace.tile.global_dim.shared::cta.b1024.b32 [%0], 0, %1;" ::"r"(map_smem), "r"(16) : "memory");
      asm volatile("tensormap.replace.tile.global_dim.shared::cta.b1024.b32 [%0], 1, %1;" ::"r"(map_smem), "r"(1) : "memory");
      if (is_sf) asm volatile("tensormap.replace.tile.global_dim.shared::cta.b1024.b32 [%0], 2, %1;" ::"r"(map_smem), "r"(1) : "memory");
    }
    asm volatile("tensormap.replace.tile.global_address.shared::cta.b1024.b64 [%0], %1;" ::"r"(map_smem), "l"(addr) : "memory");
  }
  __syncwarp();
  asm volatile(
      "tensormap.cp_fenceproxy.global.shared::cta.tensormap::generic.release.gpu.sync.aligned [%0], "
      "[%1], 128;" ::"l"(out + slot),
      "r"(smem_u32(&s_map))
      : "memory");
}

// ---------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------
static thread_local char tl_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(tl_error, sizeof(tl_error), fmt, ap);
  va_end(ap);
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(tl_error, sizeof(tl_error), fmt, ap);
  va_end(ap);
  return code;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

// Tiled tensor map over `rank` dimensions (innermost first).  strides[i] is the byte stride of
// dimension i + 1.
static int encode_map(CUtensorMap* map, CUtensorMapDataType dtype, const void* base, int rank, const uint64_t* dims,
                      const uint64_t* strides, const uint32_t* box, CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return fail(B200MOE_E_DEVICE, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t gdim[5] = {1, 1, 1, 1, 1};
  cuuint64_t gstr[4] = {0, 0, 0, 0};
  cuuint32_t bx[5] = {1, 1, 1, 1, 1};
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bx[i] = box[i];
    if (i + 1 < rank) gstr[i] = strides[i];
  }
  CUresult r = fn(map, dtype, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstr, bx, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(B200MOE_E_SHAPE, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return B200MOE_OK;
}

struct DeviceInfo {
  int sm_count = 0;
  int cc_major = 0;
  bool attr_set[3][4][2][2] = {};
  bool attr_set_bulk[2] = {};
};

static int get_device_info(DeviceInfo** out) {
  static DeviceInfo infos[64];
  static std::mutex mu;
  int dev = 0;
  B200_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(B200MOE_E_DEVICE, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(mu);
  DeviceInfo& di = infos[dev];
  if (di.sm_count == 0) {
    B200_CUDA_CHECK(cudaDeviceGetAttribute(&di.cc_major, cudaDevAttrComputeCapabilityMajor, dev));
    B200_CUDA_CHECK(cudaDeviceGetAttribute(&di.sm_count, cudaDevAttrMultiProcessorCount, dev));
  }
  *out = &di;
  return B200MOE_OK;
}

template <int kEpi, bool kDiscrete, bool kPair, bool kBulk = false, int kFmt = 0>
static int launch(const CUtensorMap* maps, const GemmParams& p, int grid, DeviceInfo* di, cudaStream_t stream) {
  auto kern = grouped_gemm_kernel<kEpi, kDiscrete, kPair, kBulk, kFmt>;
  constexpr int smem = Cfg<kPair, kBulk, kFmt>::SMEM_BYTES;
  bool& attr_set = kBulk ? di->attr_set_bulk[kPair ? 1 : 0] : di->attr_set[kFmt][kEpi][kDiscrete ? 1 : 0][kPair ? 1 : 0];
  if (!attr_set) {
    B200_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    attr_set = true;
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  if (kPair) {
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  B200_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kern, maps[0], maps[1], maps[2], maps[3], p));
  return B200MOE_OK;
}

template <int kEpi, int kFmt>
static int dispatch_fmt(bool discrete, bool pair, const CUtensorMap* maps, const GemmParams& p, int grid, DeviceInfo* di,
                        cudaStream_t stream) {
  if (discrete) {
    return pair ? launch<kEpi, true, true, false, kFmt>(maps, p, grid, di, stream) : launch<kEpi, true, false, false, kFmt>(maps, p, grid, di, stream);
  }
  return pair ? launch<kEpi, false, true, false, kFmt>(maps, p, grid, di, stream) : launch<kEpi, false, false, false, kFmt>(maps, p, grid, di, stream);
}

template <int kEpi>
static int dispatch(int fmt, bool discrete, bool pair, const CUtensorMap* maps, const GemmParams& p, int grid, DeviceInfo* di,
                    cudaStream_t stream) {
  if (fmt == 1) return dispatch_fmt<kEpi, 1>(discrete, pair, maps, p, grid, di, stream);
  if (fmt == 2) return dispatch_fmt<kEpi, 2>(discrete, pair, maps, p, grid, di, stream);
  return dispatch_fmt<kEpi, 0>(discrete, pair, maps, p, grid, di, stream);
}

static int run_gemm(int epi, const b200moe_gemm_args* a, void* stream_v) {
  cudaStream_t stream = (cudaStream_t)stream_v;
  if (!a) return fail(B200MOE_E_NULL, "args is NULL");
  const bool discrete = a->b_ptrs != nullptr || a->sfb_ptrs != nullptr;
  const char* op = epi == EPI_FC1 ? "fc1_swiglu" : (epi == EPI_FC2 ? "fc2_quant" : "dswiglu");
  if (a->m_rows == 0 || a->num_experts == 0) return B200MOE_OK;
  if (!a->a || !a->sfa || !a->padded_offsets || !a->alpha || !a->d)
    return fail(B200MOE_E_NULL, "%s: a, sfa, padded_offsets, alpha and d are required", op);
  if (discrete) {
    if (!a->b_ptrs || !a->sfb_ptrs || a->b || a->sfb)
      return fail(B200MOE_E_NULL, "%s: pass either (b, sfb) or (b_ptrs, sfb_ptrs)", op);
  } else if (!a->b || !a->sfb) {
    return fail(B200MOE_E_NULL, "%s: b and sfb are required in dense mode", op);
  }
  if (epi != EPI_FC1 && !a->prob) return fail(B200MOE_E_NULL, "%s: prob is required", op);
  if (epi == EPI_DSWIGLU && (!a->c || !a->dprob)) return fail(B200MOE_E_NULL, "%s: c (the forward pre-activation) and dprob are required", op);
  if (epi == EPI_DSWIGLU && (a->bias || a->d_row_map)) return fail(B200MOE_E_UNSUPPORTED, "%s: no bias and no row map", op);
  if (a->m_rows < 0 || a->m_rows > (1ll << 30) || a->n <= 0 || a->k <= 0 || a->num_experts < 0)
    return fail(B200MOE_E_SHAPE, "%s: bad sizes m=%lld n=%lld k=%lld E=%d", op, (long long)a->m_rows, (long long)a->n,
                (long long)a->k, a->num_experts);
  if (a->num_experts > MAX_EXPERTS)
    return fail(B200MOE_E_SHAPE, "%s: at most %d experts are supported, got %d", op, MAX_EXPERTS, a->num_experts);
  if (a->k % 16 != 0) return fail(B200MOE_E_SHAPE, "%s: k (%lld) must be a multiple of 16", op, (long long)a->k);
  // operand format: 0 = 8-bit operands with E8M0 scales per 32; 1 = E2M1, E8M0 per 32; 2 = E2M1, E8M0 or UE4M3 per 16
  const bool fp4 = a->ab_dtype == B200MOE_DTYPE_E2M1;
  const int sf_vec = a->sf_vec_size == 0 ? 32 : a->sf_vec_size;
  const bool sf_e4m3 = a->sf_dtype == B200MOE_DTYPE_E4M3;
  if (sf_vec != 16 && sf_vec != 32) return fail(B200MOE_E_SHAPE, "%s: sf_vec_size must be 16 or 32, got %d", op, sf_vec);
  if (a->sf_dtype != 0 && !sf_e4m3) return fail(B200MOE_E_UNSUPPORTED, "%s: sf_dtype %d (0 = E8M0 and E4M3 are built)", op, a->sf_dtype);
  if (!fp4 && (sf_vec != 32 || sf_e4m3)) return fail(B200MOE_E_SHAPE, "%s: 8-bit operands take E8M0 scale factors per 32 elements", op);
  if (sf_e4m3 && sf_vec != 16) return fail(B200MOE_E_SHAPE, "%s: E4M3 scale factors go with sf_vec_size 16", op);
  if (fp4 && a->k % 64 != 0)
    return fail(B200MOE_E_UNSUPPORTED, "%s: E2M1 operands need k (%lld) to be a multiple of 64 (one MMA consumes 64 elements)", op, (long long)a->k);
  if (fp4 && (a->flags & B200MOE_FLAG_B_NMAJOR)) return fail(B200MOE_E_SHAPE, "%s: E2M1 operands need a K-major B", op);
  const int fmt = !fp4 ? 0 : (sf_vec == 32 ? 1 : 2);
  if ((a->flags & B200MOE_FLAG_B_NMAJOR) && a->n % 16 != 0)
    return fail(B200MOE_E_SHAPE, "%s: N-major B needs n (%lld) to be a multiple of 16", op, (long long)a->n);
  if (epi == EPI_FC1 && a->n % 64 != 0)
    return fail(B200MOE_E_SHAPE, "%s: n (%lld) must be a multiple of 64 (32-column gate/up blocks)", op, (long long)a->n);
  if (epi != EPI_FC1 && a->n % 32 != 0)
    return fail(B200MOE_E_SHAPE, "%s: n (%lld) must be a multiple of 32", op, (long long)a->n);
  if (a->n * a->k > (1ll << 40)) return fail(B200MOE_E_SHAPE, "%s: n*k too large", op);
  const bool d_fp8 = a->d_dtype == B200MOE_DTYPE_E4M3 || a->d_dtype == B200MOE_DTYPE_E5M2;
  if (a->d_row_map && (d_fp8 || a->c)) return fail(B200MOE_E_UNSUPPORTED, "%s: d_row_map needs a bf16 D and no C", op);
  if (a->d_peer_ptrs && (!a->d_row_map || a->d_peer_slots <= 0))
    return fail(B200MOE_E_SHAPE, "%s: d_peer_ptrs needs d_row_map and a positive d_peer_slots", op);
  const bool d_f32 = a->d_dtype == B200MOE_DTYPE_F32;
  if (a->d_dtype != B200MOE_DTYPE_BF16 && a->d_dtype != B200MOE_DTYPE_F16 && !d_fp8 && !d_f32)
    return fail(B200MOE_E_UNSUPPORTED, "%s: d_dtype %d", op, a->d_dtype);
  if (d_f32 && !fp4) return fail(B200MOE_E_UNSUPPORTED, "%s: a float32 D goes with E2M1 operands only (as in the reference)", op);
  if (d_f32 && a->d_row_map) return fail(B200MOE_E_UNSUPPORTED, "%s: d_row_map needs a bf16 D", op);
  if (fp4 && d_fp8) return fail(B200MOE_E_SHAPE, "%s: E2M1 operands take a bf16, fp16 or float32 D", op);
  const bool c_fp8 = a->c_dtype == B200MOE_DTYPE_E4M3 || a->c_dtype == B200MOE_DTYPE_E5M2;
  if (a->c_dtype != B200MOE_DTYPE_BF16 && a->c_dtype != B200MOE_DTYPE_F16 && !(epi == EPI_DSWIGLU && c_fp8))
    return fail(B200MOE_E_UNSUPPORTED, "%s: c_dtype %d (bf16 and fp16 are built; E4M3 and E5M2 as the input of dswiglu)", op, a->c_dtype);
  if (a->ab_dtype != 0 && a->ab_dtype != B200MOE_DTYPE_E4M3 && a->ab_dtype != B200MOE_DTYPE_E5M2 && !fp4)
    return fail(B200MOE_E_UNSUPPORTED, "%s: ab_dtype %d (E4M3, E5M2 and E2M1 are built)", op, a->ab_dtype);
  if (a->act_func != B200MOE_ACT_SWIGLU && a->act_func != B200MOE_ACT_GEGLU)
    return fail(B200MOE_E_UNSUPPORTED, "%s: act_func %d", op, a->act_func);
  if (a->wait_limit_ms < 0) return fail(B200MOE_E_SHAPE, "%s: wait_limit_ms must not be negative", op);
  if (a->sched_light_m_tiles < -1) return fail(B200MOE_E_SHAPE, "%s: sched_light_m_tiles must be -1, 0 or positive", op);
  const bool dynamic = (a->flags & B200MOE_FLAG_DYNAMIC_SCHED) != 0;
  const bool b_nmajor = (a->flags & B200MOE_FLAG_B_NMAJOR) != 0;
  if (a->bias) {
    if (a->bias_dtype != B200MOE_DTYPE_BF16 && a->bias_dtype != B200MOE_DTYPE_F16 && a->bias_dtype != B200MOE_DTYPE_F32)
      return fail(B200MOE_E_UNSUPPORTED, "%s: bias_dtype %d", op, a->bias_dtype);
    if ((uintptr_t)a->bias % 16 != 0 || a->n % 8 != 0)
      return fail(B200MOE_E_ALIGN, "%s: bias must be 16-byte aligned and n a multiple of 8", op);
  }
  // Scale factors are generated when sfd_row and norm_const are given (always for an FP8 D; for a 16-bit
  // D the reference then stores the scaled values, block maximum mapped to 1, in D's own type)
  const bool gen_sfd = a->sfd_row != nullptr && a->norm_const != nullptr;
  if (gen_sfd && fp4) return fail(B200MOE_E_UNSUPPORTED, "%s: scale-factor generation goes with 8-bit operands only (as in the reference)", op);
  if (d_fp8 && !gen_sfd) return fail(B200MOE_E_NULL, "%s: FP8 output needs sfd_row and norm_const", op);
  if (gen_sfd && ((a->d_col == nullptr) != (a->sfd_col == nullptr)))
    return fail(B200MOE_E_NULL, "%s: d_col and sfd_col go together", op);
  if (gen_sfd && a->d_row_map) return fail(B200MOE_E_UNSUPPORTED, "%s: d_row_map cannot be combined with scale-factor generation", op);
  const uintptr_t align_or = (uintptr_t)a->a | (uintptr_t)a->sfa | (uintptr_t)a->b | (uintptr_t)a->sfb | (uintptr_t)a->c |
                             (uintptr_t)a->d | (uintptr_t)a->d_col | (uintptr_t)a->sfd_row | (uintptr_t)a->sfd_col;
  if (align_or & 15) return fail(B200MOE_E_ALIGN, "%s: tensor base addresses must be 16-byte aligned", op);

  DeviceInfo* di = nullptr;
  int rc = get_device_info(&di);
  if (rc) return rc;
  if (di->cc_major != 10) return fail(B200MOE_E_DEVICE, "%s: needs an sm_100 device, found compute capability %d.x", op, di->cc_major);

  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.sfa = (const uint8_t*)a->sfa;
  p.sfb = (const uint8_t*)a->sfb;
  p.sfb_ptrs = a->sfb_ptrs;
  p.offsets = a->padded_offsets;
  p.alpha = a->alpha;
  p.prob = a->prob;
  p.norm_const = a->norm_const;
  p.ab_format = (a->ab_dtype == B200MOE_DTYPE_E5M2 || fp4) ? ((1u << 7) | (1u << 10)) : 0u;  // E5M2 of mxf8f6f4 and E2M1 of mxf4 are both code 1
  p.sf_e4m3 = sf_e4m3 ? 1 : 0;
  p.bias = a->bias;
  p.bias_dtype = a->bias_dtype;
  p.act_geglu = (epi == EPI_FC1 && a->act_func == B200MOE_ACT_GEGLU) ? 1 : 0;
  p.d_row_map = a->d_row_map;
  p.d_peer_ptrs = a->d_row_map ? a->d_peer_ptrs : nullptr;
  p.d_peer_slots = a->d_peer_slots;
  p.c = epi == EPI_FC1 ? (__nv_bfloat16*)a->c : nullptr;
  p.c_in = epi == EPI_DSWIGLU ? a->c : nullptr;
  p.c_in_dtype = a->c_dtype;
  p.beta = a->beta;
  p.dprob = epi == EPI_DSWIGLU ? a->dprob : nullptr;
  p.d = a->d;
  p.d_col = gen_sfd ? (uint8_t*)a->d_col : nullptr;
  p.gen_sfd = gen_sfd ? 1 : 0;
  p.amax = a->amax;
  p.sfd_row = (uint8_t*)a->sfd_row;
  p.sfd_col = (uint8_t*)a->sfd_col;
  p.m_rows = (int)a->m_rows;
  p.n = (int)a->n;
  p.k = (int)a->k;
  p.num_experts = a->num_experts;
  p.n_out = epi == EPI_FC1 ? p.n / 2 : (epi == EPI_DSWIGLU ? 2 * p.n : p.n);
  p.n_tiles = (p.n + BN - 1) / BN;
  p.k_bytes = fp4 ? p.k / 2 : p.k;
  p.k_tiles = (p.k_bytes + BK - 1) / BK;
  p.rest_k = ((p.k + sf_vec - 1) / sf_vec + 3) / 4;
  p.n_blocks = (p.n + 127) / 128;
  p.sfb_expert_bytes = (int64_t)p.n_blocks * p.rest_k * 512;
  p.sfd_row_rest_k = ((p.n_out + 31) / 32 + 3) / 4;
  p.sfd_col_rest_k = ((p.m_rows + 31) / 32 + 3) / 4;
  p.d_is_fp8 = d_fp8;
  p.d_e5m2 = a->d_dtype == B200MOE_DTYPE_E5M2;
  p.d_rcp_limit = !d_fp8 ? 1.0f : (p.d_e5m2 ? 1.0f / 128.0f : 1.0f / 448.0f);
  p.d_f16 = a->d_dtype == B200MOE_DTYPE_F16;
  p.d_f32 = d_f32 ? 1 : 0;
  p.c_f16 = a->c_dtype == B200MOE_DTYPE_F16;
  p.discrete_col_sfd = (a->flags & B200MOE_FLAG_DISCRETE_COL_SFD) ? 1 : 0;
  p.first_has_prev = (a->flags & B200MOE_FLAG_OFFSETS_HAVE_PREV) ? 1 : 0;
  p.b_nmajor = b_nmajor ? 1 : 0;
  p.dynamic_sched = dynamic ? 1 : 0;
  p.test_skip_b_loads = (a->flags & B200MOE_FLAG_TEST_SKIP_B_LOADS) ? 1 : 0;
  p.wait_limit_ns = a->wait_limit_ms > 0 ? (uint64_t)a->wait_limit_ms * 1000000ull : kWaitLimitNs;
  // experts of at most this many row tiles count as weight-streaming ("light") in the tile schedule
  p.stream_m_tiles = a->l2_stream_m_tiles < 0 ? 0 : (a->l2_stream_m_tiles == 0 ? DEFAULT_STREAM_M_TILES : a->l2_stream_m_tiles);
  p.light_m_tiles = a->sched_light_m_tiles < 0 ? 0 : (a->sched_light_m_tiles == 0 ? DEFAULT_LIGHT_M_TILES : a->sched_light_m_tiles);
  {
    // 256-bit stores need 32-byte aligned bases and row pitches that keep a 32-column block aligned
    const int64_t d_pitch = (int64_t)p.n_out * (d_fp8 ? 1 : (d_f32 ? 4 : 2));
    const uintptr_t bases = (epi == EPI_FC1 ? (uintptr_t)a->c : 0) | (uintptr_t)a->d | (uintptr_t)a->d_col;
    p.wide_stores = (bases % 32 == 0) && (d_pitch % 32 == 0) && (((int64_t)p.n * 2) % 32 == 0);
  }

  // Tile mode.  A pair (two CTAs, 256 x 256) moves half the weight bytes per SM but rounds every
  // expert group up to 256 rows; the host sees only the average group size, so pairs are used when
  // groups are large on average or the caller forces them.
  bool pair;
  if (a->flags & B200MOE_FLAG_TILE_SINGLE) pair = false;
  else if (a->flags & B200MOE_FLAG_TILE_PAIR) pair = true;
  else pair = a->m_rows / a->num_experts >= 1024;
  {
    const int64_t rows = std::min<int64_t>(RASTER_GROUP_ROWS, RASTER_GROUP_BYTES / std::max<int64_t>(p.k_bytes, 1));
    p.raster_group_m = (int)std::max<int64_t>(1, rows / (pair ? 2 * BM : BM));
  }

  CUtensorMap maps[4];  // A, B (or its prototype), SFA, SFB (or its prototype); the last two only in pair mode
  memset(maps, 0, sizeof(maps));
  const uint32_t b_rows = pair ? 128 : BN;
  {
    const uint64_t dims[2] = {(uint64_t)p.k_bytes, (uint64_t)p.m_rows};
    const uint64_t strides[1] = {(uint64_t)p.k_bytes};
    const uint32_t box[2] = {BK, BM};
    rc = encode_map(&maps[0], CU_TENSOR_MAP_DATA_TYPE_UINT8, a->a, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
  }
  const uint64_t sf_chunk_stride = 512, sf_row_stride = (uint64_t)p.rest_k * 512;
  const uint32_t cpk = 1u << fmt;  // scale chunks per k-tile
  if (pair) {
    // scale factors as 512-byte chunks of 128 uint32: (chunk word, K group, 128-row block[, expert])
    const uint64_t dims[3] = {128, (uint64_t)p.rest_k, (uint64_t)((p.m_rows + 127) / 128)};
    const uint64_t strides[2] = {sf_chunk_stride, sf_row_stride};
    const uint32_t box[3] = {128, cpk, 1};
    rc = encode_map(&maps[2], CU_TENSOR_MAP_DATA_TYPE_UINT32, a->sfa, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
  }
  // workspace: [E x 2 tensor maps of 128 bytes] (discrete) then [128 bytes, the tile counter] (dynamic scheduler)
  const int64_t maps_bytes = discrete ? (int64_t)p.num_experts * 256 : 0;
  const int64_t need = maps_bytes + (dynamic ? 128 : 0);
  if (need > 0 && (!a->workspace || a->workspace_bytes < need || ((uintptr_t)a->workspace & 127)))
    return fail(B200MOE_E_WORKSPACE, "%s: needs a 128-byte aligned workspace of %lld bytes (b200moe_workspace_bytes)", op, (long long)need);
  if (!discrete) {
    if (!b_nmajor) {
      const uint64_t dims[3] = {(uint64_t)p.k_bytes, (uint64_t)p.n, (uint64_t)p.num_experts};
      const uint64_t strides[2] = {(uint64_t)p.k_bytes, (uint64_t)p.n * (uint64_t)p.k_bytes};
      const uint32_t box[3] = {BK, b_rows, 1};
      rc = encode_map(&maps[1], CU_TENSOR_MAP_DATA_TYPE_UINT8, a->b, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    } else {
      // [E][K][N]: slabs of 128 columns x 128 K rows (128-byte swizzle rows run along N)
      const uint64_t dims[3] = {(uint64_t)p.n, (uint64_t)p.k, (uint64_t)p.num_experts};
      const uint64_t strides[2] = {(uint64_t)p.n, (uint64_t)p.n * (uint64_t)p.k};
      const uint32_t box[3] = {128, BK, 1};
      rc = encode_map(&maps[1], CU_TENSOR_MAP_DATA_TYPE_UINT8, a->b, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    }
    if (rc) return rc;
    if (pair) {
      const uint64_t sdims[4] = {128, (uint64_t)p.rest_k, (uint64_t)p.n_blocks, (uint64_t)p.num_experts};
      const uint64_t sstrides[3] = {sf_chunk_stride, sf_row_stride, (uint64_t)p.sfb_expert_bytes};
      const uint32_t sbox[4] = {128, cpk, 2, 1};
      rc = encode_map(&maps[3], CU_TENSOR_MAP_DATA_TYPE_UINT32, a->sfb, 4, sdims, sstrides, sbox, CU_TENSOR_MAP_SWIZZLE_NONE);
      if (rc) return rc;
    }
  } else {
    // prototypes; the global addresses are patched per expert on the device
    if (!b_nmajor) {
      const uint64_t dims[2] = {(uint64_t)p.k_bytes, (uint64_t)p.n};
      const uint64_t strides[1] = {(uint64_t)p.k_bytes};
      const uint32_t box[2] = {BK, b_rows};
      rc = encode_map(&maps[1], CU_TENSOR_MAP_DATA_TYPE_UINT8, a->a, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    } else {
      const uint64_t dims[2] = {(uint64_t)p.n, (uint64_t)p.k};
      const uint64_t strides[1] = {(uint64_t)p.n};
      const uint32_t box[2] = {128, BK};
      rc = encode_map(&maps[1], CU_TENSOR_MAP_DATA_TYPE_UINT8, a->a, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    }
    if (rc) return rc;
    const uint64_t sdims[3] = {128, (uint64_t)p.rest_k, (uint64_t)p.n_blocks};
    const uint64_t sstrides[2] = {sf_chunk_stride, sf_row_stride};
    const uint32_t sbox[3] = {128, cpk, 2};
    rc = encode_map(&maps[3], CU_TENSOR_MAP_DATA_TYPE_UINT32, a->sfa, 3, sdims, sstrides, sbox, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
    p.b_maps = (const CUtensorMap*)a->workspace;
    build_expert_tensormaps_kernel<<<2 * p.num_experts, 32, 0, stream>>>(maps[1], maps[3], a->b_ptrs, a->sfb_ptrs, a->a, a->sfa,
                                                                          (CUtensorMap*)a->workspace, p.num_experts);
    B200_CUDA_CHECK(cudaGetLastError());
  }
  if (dynamic) {
    p.tile_counter = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(a->workspace) + maps_bytes);
    B200_CUDA_CHECK(cudaMemsetAsync(p.tile_counter, 0, sizeof(int), stream));
  }

  const int tile_m = pair ? 256 : 128;
  // upper bound of scheduled tiles: every expert may add one partial row tile
  const int64_t max_tiles = ((a->m_rows + tile_m - 1) / tile_m + (pair ? a->num_experts : 0)) * p.n_tiles;
  int units = di->sm_count - (a->sm_margin > 0 ? a->sm_margin : 0);
  if (pair) units /= 2;
  if (units < 1) units = 1;
  if ((int64_t)units > max_tiles) units = (int)max_tiles;
  const int grid = pair ? 2 * units : units;

  // FC2 rows that go to peer buffers leave through shared memory and one bulk copy per row
  if (epi == EPI_FC2 && !discrete && !d_fp8 && !gen_sfd && fmt == 0 && p.d_peer_ptrs && ((uintptr_t)a->d % 16 == 0))
    return pair ? launch<EPI_FC2, false, true, true>(maps, p, grid, di, stream)
                : launch<EPI_FC2, false, false, true>(maps, p, grid, di, stream);
  if (epi == EPI_DSWIGLU) return dispatch<EPI_DSWIGLU>(fmt, discrete, pair, maps, p, grid, di, stream);
  return epi == EPI_FC1 ? dispatch<EPI_FC1>(fmt, discrete, pair, maps, p, grid, di, stream)
                        : dispatch<EPI_FC2>(fmt, discrete, pair, maps, p, grid, di, stream);
}

// ---------------------------------------------------------------------------------------
// Weight gradient: the experts partition the contraction dimension (tokens).
// ---------------------------------------------------------------------------------------
static int run_wgrad(const b200moe_gemm_args* a, void* stream_v) {
  cudaStream_t stream = (cudaStream_t)stream_v;
  const char* op = "wgrad";
  if (!a) return fail(B200MOE_E_NULL, "args is NULL");
  if (a->num_experts == 0 || a->m_rows == 0 || a->n == 0) return B200MOE_OK;
  if (!a->a || !a->b || !a->sfa || !a->sfb || !a->padded_offsets || (!a->d && !a->d_peer_ptrs))
    return fail(B200MOE_E_NULL, "%s: a, b, sfa, sfb, padded_offsets (token END offsets) and d (or d_peer_ptrs) are required", op);
  if (a->b_ptrs || a->sfb_ptrs) return fail(B200MOE_E_UNSUPPORTED, "%s: a and b are single tensors (per-expert outputs go in d_peer_ptrs)", op);
  if (a->m_rows < 0 || a->m_rows > (1ll << 30) || a->n <= 0 || a->k < 0 || a->k > (1ll << 30) || a->num_experts < 0 || a->num_experts > MAX_EXPERTS)
    return fail(B200MOE_E_SHAPE, "%s: bad sizes m=%lld n=%lld tokens=%lld E=%d", op, (long long)a->m_rows, (long long)a->n, (long long)a->k, a->num_experts);
  const bool fp4 = a->ab_dtype == B200MOE_DTYPE_E2M1;
  const int sf_vec = a->sf_vec_size == 0 ? 32 : a->sf_vec_size;
  const bool sf_e4m3 = a->sf_dtype == B200MOE_DTYPE_E4M3;
  if (sf_vec != 16 && sf_vec != 32) return fail(B200MOE_E_SHAPE, "%s: sf_vec_size must be 16 or 32, got %d", op, sf_vec);
  if (!fp4 && (sf_vec != 32 || sf_e4m3)) return fail(B200MOE_E_SHAPE, "%s: 8-bit operands take E8M0 scale factors per 32 elements", op);
  if (sf_e4m3 && sf_vec != 16) return fail(B200MOE_E_SHAPE, "%s: E4M3 scale factors go with sf_vec_size 16", op);
  if (a->ab_dtype != 0 && a->ab_dtype != B200MOE_DTYPE_E4M3 && a->ab_dtype != B200MOE_DTYPE_E5M2 && !fp4)
    return fail(B200MOE_E_UNSUPPORTED, "%s: ab_dtype %d", op, a->ab_dtype);
  if (a->k % 32 != 0) return fail(B200MOE_E_SHAPE, "%s: the token count (%lld) must be a multiple of 32", op, (long long)a->k);
  if (a->n % 32 != 0) return fail(B200MOE_E_SHAPE, "%s: n (%lld) must be a multiple of 32", op, (long long)a->n);
  const bool d_f32 = a->d_dtype == B200MOE_DTYPE_F32;
  if (a->d_dtype != B200MOE_DTYPE_BF16 && a->d_dtype != B200MOE_DTYPE_F16 && !d_f32)
    return fail(B200MOE_E_UNSUPPORTED, "%s: d_dtype %d (bf16, fp16 and float32 are built)", op, a->d_dtype);
  if (a->wait_limit_ms < 0) return fail(B200MOE_E_SHAPE, "%s: wait_limit_ms must not be negative", op);
  const uintptr_t align_or = (uintptr_t)a->a | (uintptr_t)a->sfa | (uintptr_t)a->b | (uintptr_t)a->sfb | (uintptr_t)a->d;
  if (align_or & 15) return fail(B200MOE_E_ALIGN, "%s: tensor base addresses must be 16-byte aligned", op);
  const int fmt = !fp4 ? 0 : (sf_vec == 32 ? 1 : 2);

  DeviceInfo* di = nullptr;
  int rc = get_device_info(&di);
  if (rc) return rc;
  if (di->cc_major != 10) return fail(B200MOE_E_DEVICE, "%s: needs an sm_100 device, found compute capability %d.x", op, di->cc_major);

  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.sfa = (const uint8_t*)a->sfa;
  p.sfb = (const uint8_t*)a->sfb;
  p.offsets = a->padded_offsets;
  p.alpha = a->alpha;
  p.beta = a->beta;
  p.ab_format = (a->ab_dtype == B200MOE_DTYPE_E5M2 || fp4) ? ((1u << 7) | (1u << 10)) : 0u;
  p.sf_e4m3 = sf_e4m3 ? 1 : 0;
  p.d = a->d;
  p.d_peer_ptrs = a->d_peer_ptrs;  // discrete output: one [m, n] allocation per expert (the kernel trusts them to be 16-byte aligned)
  p.m_rows = (int)a->m_rows;
  p.n = (int)a->n;
  p.k = (int)a->k;
  p.num_experts = a->num_experts;
  p.n_out = p.n;
  p.n_tiles = (p.n + BN - 1) / BN;
  p.n_blocks = (p.n + 127) / 128;
  p.k_bytes = fp4 ? p.k / 2 : p.k;
  p.d_f16 = a->d_dtype == B200MOE_DTYPE_F16;
  p.d_f32 = d_f32 ? 1 : 0;
  p.accumulate = (a->flags & B200MOE_FLAG_ACCUMULATE) ? 1 : 0;
  p.raster_group_m = 1;
  p.wait_limit_ns = a->wait_limit_ms > 0 ? (uint64_t)a->wait_limit_ms * 1000000ull : kWaitLimitNs;
  p.wide_stores = !a->d_peer_ptrs && ((uintptr_t)a->d % 32 == 0) && (((int64_t)p.n * (d_f32 ? 4 : 2)) % 32 == 0);

  CUtensorMap maps[4];
  memset(maps, 0, sizeof(maps));
  {
    const uint64_t dims[2] = {(uint64_t)p.k_bytes, (uint64_t)p.m_rows};
    const uint64_t strides[1] = {(uint64_t)p.k_bytes};
    const uint32_t box[2] = {BK, BM};
    rc = encode_map(&maps[0], CU_TENSOR_MAP_DATA_TYPE_UINT8, a->a, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
  }
  {
    const uint64_t dims[2] = {(uint64_t)p.k_bytes, (uint64_t)p.n};
    const uint64_t strides[1] = {(uint64_t)p.k_bytes};
    const uint32_t box[2] = {BK, BN};
    rc = encode_map(&maps[1], CU_TENSOR_MAP_DATA_TYPE_UINT8, a->b, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
  }
  // 256 x 256 tiles on CTA pairs when the output has at least two row blocks (every expert has the same tiles, so
  // nothing is lost to padding beyond m's own remainder); flags force either mode
  bool pair = p.m_rows > BM;
  if (a->flags & B200MOE_FLAG_TILE_SINGLE) pair = false;
  if (a->flags & B200MOE_FLAG_TILE_PAIR) pair = true;
  if (pair) {
    // B: this CTA's half of the 256 columns; scale chunks as a plain array of 512-byte chunks (an expert's blocks may
    // hold up to one chunk per row block more than k / (4 sf_vec): the bound below covers that)
    const uint64_t dims[2] = {(uint64_t)p.k_bytes, (uint64_t)p.n};
    const uint64_t strides[1] = {(uint64_t)p.k_bytes};
    const uint32_t box[2] = {BK, 128};
    rc = encode_map(&maps[1], CU_TENSOR_MAP_DATA_TYPE_UINT8, a->b, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    const uint64_t chunks_k = (uint64_t)((p.k + sf_vec - 1) / sf_vec + 3) / 4 + (uint64_t)p.num_experts;
    const uint32_t sbox[2] = {128, 1u << fmt};
    const uint64_t sstrides[1] = {512};
    const uint64_t adims[2] = {128, chunks_k * (uint64_t)((p.m_rows + 127) / 128)};
    rc = encode_map(&maps[2], CU_TENSOR_MAP_DATA_TYPE_UINT32, a->sfa, 2, adims, sstrides, sbox, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
    const uint64_t bdims[2] = {128, chunks_k * (uint64_t)p.n_blocks};
    rc = encode_map(&maps[3], CU_TENSOR_MAP_DATA_TYPE_UINT32, a->sfb, 2, bdims, sstrides, sbox, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
  }
  const int tile_m = pair ? 2 * BM : BM;
  const int64_t tiles = (int64_t)p.num_experts * ((p.m_rows + tile_m - 1) / tile_m) * p.n_tiles;
  int units = di->sm_count - (a->sm_margin > 0 ? a->sm_margin : 0);
  if (pair) units /= 2;
  if (units < 1) units = 1;
  if ((int64_t)units > tiles) units = (int)tiles;
  if (pair) {
    if (fmt == 1) return launch<EPI_WGRAD, false, true, false, 1>(maps, p, 2 * units, di, stream);
    if (fmt == 2) return launch<EPI_WGRAD, false, true, false, 2>(maps, p, 2 * units, di, stream);
    return launch<EPI_WGRAD, false, true, false, 0>(maps, p, 2 * units, di, stream);
  }
  if (fmt == 1) return launch<EPI_WGRAD, false, false, false, 1>(maps, p, units, di, stream);
  if (fmt == 2) return launch<EPI_WGRAD, false, false, false, 2>(maps, p, units, di, stream);
  return launch<EPI_WGRAD, false, false, false, 0>(maps, p, units, di, stream);
}

// ---------------------------------------------------------------------------------------
// Discrete-weight FC1 for callers that cannot allocate device memory.
//
// The per-expert tensor maps normally live in a workspace the caller allocates.  Some callers have
// no way to do that: code running after an inference server has handed every free byte of the GPU
// to its own arena, plugins that are given tensors but no allocator handle, and latency-critical
// loops that must never reach cudaMalloc because it synchronises the whole device.  For them the
// maps live in the fixed array below, which is part of the library image: every GPU that loads
// the library holds these bytes from load until the process exits.
//
// The array's name is only a host-side handle; the device address is looked up once per device
// (with that device current) and cached.  All calls on a device share the array, and it keeps
// whatever the previous call wrote: each call rewrites the slots of its own experts before its
// GEMM reads them, so nothing has to be cleared, but two calls that overlap on the same GPU
// (different streams) race on it.
// ---------------------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_noalloc_scratch[B200MOE_NOALLOC_SCRATCH_BYTES];

static int noalloc_scratch_address(void** out) {
  static void* address[64] = {nullptr};
  static std::mutex mu;
  int dev = 0;
  B200_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(B200MOE_E_DEVICE, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (address[dev] == nullptr) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr)
      return fail(e != cudaSuccess ? (int)e : B200MOE_E_DEVICE, "cudaGetSymbolAddress(scratch) failed on device %d: %s", dev,
                  cudaGetErrorString(e));
    address[dev] = p;
  }
  *out = address[dev];
  return B200MOE_OK;
}

}  // namespace b200moe

extern "C" {

int b200moe_fc1_swiglu_discrete_noalloc(const b200moe_gemm_args* args, void* stream) {
  using namespace b200moe;
  if (!args) return fail(B200MOE_E_NULL, "args is NULL");
  if (!args->b_ptrs || !args->sfb_ptrs || args->b || args->sfb)
    return fail(B200MOE_E_NULL, "fc1_swiglu_discrete_noalloc: takes discrete weights only (b_ptrs and sfb_ptrs, no b / sfb)");
  if (args->num_experts > B200MOE_NOALLOC_MAX_EXPERTS)
    return fail(B200MOE_E_SHAPE, "fc1_swiglu_discrete_noalloc: %d experts exceed the built-in scratch (at most %d); use b200moe_fc1_swiglu with a caller workspace",
                args->num_experts, B200MOE_NOALLOC_MAX_EXPERTS);
  if (b200moe_workspace_bytes(args->num_experts, 1) > (int64_t)B200MOE_NOALLOC_SCRATCH_BYTES)
    return fail(B200MOE_E_SHAPE, "fc1_swiglu_discrete_noalloc: built-in scratch too small for %d experts", args->num_experts);
  if (args->flags & B200MOE_FLAG_DYNAMIC_SCHED)
    return fail(B200MOE_E_UNSUPPORTED, "fc1_swiglu_discrete_noalloc: the dynamic tile scheduler needs a caller workspace; use b200moe_fc1_swiglu");
  if (args->m_rows == 0 || args->num_experts <= 0) return run_gemm(EPI_FC1, args, stream);
  void* scratch = nullptr;
  int rc = noalloc_scratch_address(&scratch);
  if (rc) return rc;
  b200moe_gemm_args local = *args;
  local.workspace = scratch;
  local.workspace_bytes = B200MOE_NOALLOC_SCRATCH_BYTES;
  return run_gemm(EPI_FC1, &local, stream);
}

int b200moe_fc1_swiglu(const b200moe_gemm_args* args, void* stream) { return b200moe::run_gemm(b200moe::EPI_FC1, args, stream); }

int b200moe_fc2_quant(const b200moe_gemm_args* args, void* stream) { return b200moe::run_gemm(b200moe::EPI_FC2, args, stream); }

int b200moe_dswiglu(const b200moe_gemm_args* args, void* stream) { return b200moe::run_gemm(b200moe::EPI_DSWIGLU, args, stream); }

int b200moe_wgrad(const b200moe_gemm_args* args, void* stream) { return b200moe::run_wgrad(args, stream); }

int64_t b200moe_workspace_bytes(int32_t num_experts, int32_t mode) {
  if (num_experts <= 0) return 0;
  int64_t bytes = 0;
  if (mode & B200MOE_WORKSPACE_DISCRETE) bytes += (int64_t)num_experts * 256;  // one weight map and one scale-factor map per expert
  if (mode & B200MOE_WORKSPACE_DYNAMIC_SCHED) bytes += 128;                      // the tile counter
  return bytes;
}

const char* b200moe_last_error(void) { return b200moe::tl_error; }

int b200moe_device_status(int clear) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, b200moe::g_device_status, sizeof(int)) != cudaSuccess) return -1;
  if (clear) {
    int z = 0;
    cudaMemcpyToSymbol(b200moe::g_device_status, &z, sizeof(int));
  }
  return v;
}

int b200moe_abi_version(void) { return 7; }

}  // extern "C"
