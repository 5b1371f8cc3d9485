/*
 * b200moe.h - C ABI of the B200-native MoE grouped-GEMM hot path.
 *
 * One shared library (libb200moe.so) built for sm_100a only.  Every entry point takes
 * plain device pointers, sizes and a CUDA stream (passed as void*) and never throws.  The
 * compute entry points (GEMMs, quantiser, routing and row movers) launch their kernels
 * asynchronously on that stream, never synchronise and never allocate device memory; the only
 * calls that allocate, map or free device memory are b200moe_peer_alloc / _open / _close /
 * _free, and b200moe_device_status synchronises the device.  Return value: 0 = launched, < 0 = argument error (B200MOE_E_*),
 * > 0 = CUDA runtime / driver error code.  b200moe_last_error() returns a thread-local
 * human-readable description of the last non-zero return.
 *
 * The entry points stand in for the reference's JIT-compiled CuTe-DSL kernels; each
 * comment names the reference interface it replaces (path inside NVIDIA/cudnn-frontend).
 */
#ifndef B200MOE_H_
#define B200MOE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200MOE_OK 0
#define B200MOE_E_NULL (-1)        /* a required pointer is NULL                        */
#define B200MOE_E_SHAPE (-2)       /* a size is out of range / violates a divisibility  */
#define B200MOE_E_ALIGN (-3)       /* a pointer or pitch is not 16-byte aligned          */
#define B200MOE_E_UNSUPPORTED (-4) /* valid in the reference, not built here             */
#define B200MOE_E_WORKSPACE (-5)   /* workspace missing or too small                     */
#define B200MOE_E_DEVICE (-6)      /* not an sm_100 device / driver entry point missing  */

/* d_dtype values */
#define B200MOE_DTYPE_BF16 0
#define B200MOE_DTYPE_E4M3 1
#define B200MOE_DTYPE_F16 2
#define B200MOE_DTYPE_F32 3
#define B200MOE_DTYPE_E5M2 4
#define B200MOE_DTYPE_E2M1 5 /* FP4, two values per byte, the even element in the low nibble */

#define B200MOE_ACT_SWIGLU 0
#define B200MOE_ACT_GEGLU 1

/* flags */
#define B200MOE_FLAG_DISCRETE_COL_SFD 1 /* per-expert column scale-factor blocks */
#define B200MOE_FLAG_TILE_SINGLE 2      /* force 128 x 256 single-CTA tiles                    */
#define B200MOE_FLAG_TILE_PAIR 4        /* force 256 x 256 CTA-pair tiles (cta_group::2)       */
/* Tiles are handed out through an atomic counter instead of a fixed stride (the reference's
   use_dynamic_sched, python/cudnn/grouped_gemm/moe_persistent_scheduler.py:838-893); needs 128
   bytes of workspace (b200moe_workspace_bytes with B200MOE_WORKSPACE_DYNAMIC_SCHED).  Results are
   bit-identical to the static schedule. */
#define B200MOE_FLAG_DYNAMIC_SCHED 8
/* B is N-major: memory [E][k][n] (dense) or one [k][n] allocation per expert (discrete), the
   reference's b_major = "n" (python/cudnn/grouped_gemm/grouped_gemm_quant/api.py:288-294) */
#define B200MOE_FLAG_B_NMAJOR 16
/* The call covers a slice [e0, e0 + num_experts) of a longer expert list: padded_offsets, alpha,
   amax, b / sfb (or b_ptrs / sfb_ptrs) and bias point at expert e0's entries, padded_offsets[-1] is
   readable and is the first row of expert e0; a, sfa, prob, c, d, ... and m_rows describe the whole
   row range.  Lets a layer run its experts in chunks on the same buffers. */
#define B200MOE_FLAG_OFFSETS_HAVE_PREV 32
/* Test hook: the producer of the B side issues no loads, so the kernel's bounded waits run out,
   the kernel returns and b200moe_device_status reports which wait gave up.  Use with a small
   wait_limit_ms.  The outputs of such a launch are undefined. */
#define B200MOE_FLAG_TEST_SKIP_B_LOADS 64
/* b200moe_wgrad: add the result to d instead of overwriting it (the reference's accumulate_on_output) */
#define B200MOE_FLAG_ACCUMULATE 128

/* mode bits of b200moe_workspace_bytes */
#define B200MOE_WORKSPACE_DISCRETE 1
#define B200MOE_WORKSPACE_DYNAMIC_SCHED 2

/*
 * Arguments of one grouped GEMM launch.  All pointers are device pointers.
 *
 * Layouts (the reference's, python/cudnn/grouped_gemm/grouped_gemm_swiglu/api.py:193-247):
 *   a      [m_rows, k]  E4M3 / E5M2 (or k / 2 bytes of packed E2M1), K contiguous
 *   sfa    E8M0 (or E4M3), "128x4" swizzled layout of (m_rows, k / sf_vec_size)
 *   b      [E, n, k]    same element type as a, K contiguous (dense mode) | exactly one of
 *   sfb    E blocks, each the 128x4 layout of (n, k/32)           | (b, sfb) and
 *   b_ptrs / sfb_ptrs   int64 device arrays [E] of per-expert     | (b_ptrs, sfb_ptrs)
 *                       addresses of [n, k] / its 128x4 layout    | is non-NULL
 *   padded_offsets [E]  int32 END offsets, multiples of 128
 *   alpha  [E] f32, prob [m_rows] f32 (optional for FC1), norm_const [1] f32
 *   c      [m_rows, n]      bf16 (FC1 only; NULL = do not write it)
 *   d      [m_rows, n_out]  bf16 or E4M3 (n_out = n/2 for FC1, n for FC2)
 *   d_col  [m_rows, n_out]  E4M3 quantised with the column scales (optional)
 *   amax   [E] f32, updated with atomic max (caller initialises, e.g. to -inf)
 *   sfd_row  128x4 layout of (m_rows, n_out/32); sfd_col  128x4 layout of (n_out, m_rows/32)
 *   workspace  discrete mode and / or dynamic scheduler: b200moe_workspace_bytes(E, mode) bytes,
 *              128-B aligned
 */
typedef struct b200moe_gemm_args {
  const void* a;
  const void* sfa;
  const void* b;
  const void* sfb;
  const int64_t* b_ptrs;
  const int64_t* sfb_ptrs;
  const int32_t* padded_offsets;
  const float* alpha;
  const float* prob;
  const float* norm_const;
  void* c;
  void* d;
  void* d_col;
  float* amax;
  void* sfd_row;
  void* sfd_col;
  void* workspace;
  int64_t workspace_bytes;
  int64_t m_rows;
  int64_t n;
  int64_t k;
  int32_t num_experts;
  int32_t d_dtype;
  int32_t flags;
  int32_t sm_margin; /* SMs left free for a concurrent kernel (CUDNNFE_CLUSTER_OVERLAP_MARGIN) */
  /* optional, bf16 D only: row r of the result is stored at row d_row_map[r] of d (negative =
     the row is not stored).  Lets the layer write FC2 results straight in all-to-all order. */
  const int32_t* d_row_map;
  /* optional, with d_row_map: the destination rows live in peer-accessible buffers of G ranks.
     d_peer_ptrs = device array of G base addresses (this rank's own buffer included), every buffer
     [d_peer_slots, N_out] bf16; a map value v >= 0 then means row (v % d_peer_slots) of the buffer
     of rank (v / d_peer_slots).  The epilogue stores over NVLink, which replaces the combine
     all-to-all of an expert-parallel layer.  NULL = d_row_map indexes d. */
  const int64_t* d_peer_ptrs;
  int64_t d_peer_slots;
  /* optional fused bias, [N, E] with strides (1, N) as in the reference (element (n, e) at
     e * N + n), bf16 / f16 / f32.  FC1: C = alpha * acc + bias before the activation
     (grouped_gemm_glu/moe_blockscaled_grouped_gemm_glu_bias.py:2628-2660).  FC2:
     D = alpha * acc + bias * prob (grouped_gemm_quant/grouped_gemm_quant.py:1841-1865). */
  const void* bias;
  int32_t bias_dtype; /* B200MOE_DTYPE_BF16 / _F16 / _F32 */
  /* FC1 activation: B200MOE_ACT_SWIGLU, or B200MOE_ACT_GEGLU = the reference's GeGLU
     (gate <= 7, -7 <= up <= 7, D = (up + 1) * gate * sigmoid(1.702 gate) * prob;
     moe_blockscaled_grouped_gemm_glu_bias.py:1414-1487,2702-2716) */
  int32_t act_func;
  /* element type of A and B (both the same, as the reference demands): B200MOE_DTYPE_E4M3
     (also when left 0) or B200MOE_DTYPE_E5M2 */
  int32_t ab_dtype;
  /* element type of C: B200MOE_DTYPE_BF16 (also when left 0) or B200MOE_DTYPE_F16.  d_dtype takes
     B200MOE_DTYPE_BF16 / _F16 (16-bit D with amax) or B200MOE_DTYPE_E4M3 / _E5M2 (FP8 D and D_col
     with E8M0 scales; the block maximum maps to 448 resp. 128 as in the reference's
     get_dtype_rcp_limits, grouped_gemm_swiglu_quant.py:2996-3012). */
  int32_t c_dtype;
  /* limit of every wait inside the kernel in milliseconds (0 = the default, 4000): a wait that runs
     out records a code in the device status word and the kernel returns */
  int32_t wait_limit_ms;
  /* tile schedule: experts with at most this many row tiles are treated as weight-streaming and
     their tiles are interleaved with those of the larger experts (0 = the library's default,
     -1 = no interleaving: experts in order) */
  int32_t sched_light_m_tiles;
  /* weight tiles of experts with at most this many row tiles are read with an evict-first L2 hint:
     they are used once or twice and should not displace activations and shared weight tiles
     (0 = the library's default, -1 = no hints) */
  int32_t l2_stream_m_tiles;
  /* Block scaling of A and B (python/cudnn/grouped_gemm/grouped_gemm_swiglu/api.py:249-352).  sf_vec_size:
     elements of K per scale factor, 32 (also when left 0) or 16; sf_dtype: 0 = E8M0, B200MOE_DTYPE_E4M3 =
     E4M3 read as unsigned (sf_vec_size 16 only).  8-bit operands (ab_dtype E4M3 / E5M2) take E8M0 per 32
     (MXFP8).  ab_dtype B200MOE_DTYPE_E2M1: a and b hold k / 2 bytes per row and k counts elements; E8M0
     per 32 (MXFP4), E8M0 per 16, or E4M3 per 16 (NVFP4); k must be a multiple of 64, B K-major, D bf16 /
     fp16 (with amax) or float32, no scale-factor generation (the reference's rules for FP4 operands). */
  int32_t sf_vec_size;
  int32_t sf_dtype;
  /* b200moe_dswiglu only: per-expert scale of the forward pre-activation read through `c` (NULL = 1), and the
     gradient of the gate probabilities [m_rows] f32, accumulated with atomic adds (the caller zeroes it) */
  const float* beta;
  float* dprob;
} b200moe_gemm_args;

/*
 * FC1: C = alpha_e * (A*SFA)(B_e*SFB_e)^T ; D[:, 32j:32j+32] = up_j * silu(gate_j) * prob,
 * gate/up = even/odd 32-column blocks of C; per-expert amax (bf16 D) or row/column MXFP8
 * re-quantisation (E4M3 D).
 * Replaces the launch done by GroupedGemmSwigluSm100.execute
 * (python/cudnn/grouped_gemm/grouped_gemm_swiglu/api.py:706-771), i.e. the kernel
 * BlockScaledContiguousGroupedGemmKernel
 * (python/cudnn/grouped_gemm/grouped_gemm_swiglu/grouped_gemm_swiglu_quant.py:1241-2636),
 * and, with b_ptrs/sfb_ptrs, DiscreteGroupedGemmSwigluSm100.execute
 * (python/cudnn/discrete_grouped_gemm/discrete_grouped_gemm_swiglu/api.py:710-795).
 */
int b200moe_fc1_swiglu(const b200moe_gemm_args* args, void* stream);

/*
 * Discrete-weight FC1 that allocates nothing and needs no workspace.  It has no counterpart in
 * the reference.  It is b200moe_fc1_swiglu in discrete mode (b_ptrs / sfb_ptrs; args->workspace is
 * ignored) with the per-expert descriptor table kept in a fixed device array inside the library
 * (B200MOE_NOALLOC_SCRATCH_BYTES per GPU, held from library load to process exit) instead of in
 * caller memory.  Meant for callers that cannot obtain device memory at call time: code that runs
 * after the host application has given all free GPU memory to its own arena, plugins that receive
 * tensors but no allocator, and loops that must never trigger cudaMalloc (it synchronises the
 * device).  Limits and rules:
 *   - at most B200MOE_NOALLOC_MAX_EXPERTS experts; more returns B200MOE_E_SHAPE;
 *   - the first call on each device looks up the array's device address (cudaGetSymbolAddress,
 *     with that device current); make that first call outside any stream capture;
 *   - every call on a device uses the same array: calls that overlap on the GPU (different
 *     streams) race with each other; calls ordered on one stream are safe.
 */
#define B200MOE_NOALLOC_MAX_EXPERTS 256
#define B200MOE_NOALLOC_SCRATCH_BYTES (B200MOE_NOALLOC_MAX_EXPERTS * 256)
int b200moe_fc1_swiglu_discrete_noalloc(const b200moe_gemm_args* args, void* stream);

/*
 * FC2: D = quant(alpha_e * acc * prob); bf16 D + per-expert amax, or E4M3 D + row/column
 * E8M0 scale factors.
 * Replaces GroupedGemmQuantSm100.execute
 * (python/cudnn/grouped_gemm/grouped_gemm_quant/api.py:974-1089), kernel
 * BlockScaledMoEGroupedGemmQuantKernel
 * (python/cudnn/grouped_gemm/grouped_gemm_quant/grouped_gemm_quant.py:1073-1985).
 */
int b200moe_fc2_quant(const b200moe_gemm_args* args, void* stream);

/*
 * Backward of FC1's activation: G = alpha_e^2 * (A*SFA)(B_e*SFB_e)^T is the gradient of the SwiGLU output
 * [m_rows, n]; `c` is an INPUT here, the forward pre-activation [m_rows, 2n] (c_dtype bf16 / fp16 / E4M3 / E5M2;
 * gate / up = even / odd 32-column blocks), scaled by beta_e.  D and D_col are [m_rows, 2n]:
 *   D[:, 64j:64j+32]    = G_j * prob * up_j * sig_j * (1 + gate_j * (1 - sig_j))     (gradient of the gate block)
 *   D[:, 64j+32:64j+64] = G_j * prob * gate_j * sig_j                                (gradient of the up block)
 *   dprob[r]           += sum over columns of G * gate * sig * up
 * with sig = sigmoid(gate).  Outputs as for FC2: E4M3 / E5M2 D and D_col with row and column E8M0 scale factors,
 * or a 16-bit / float32 D with amax, which is [E][2] here (gate gradient, up gradient).
 * Replaces GroupedGemmDswigluSm100.execute
 * (python/cudnn/grouped_gemm/grouped_gemm_dswiglu/api.py:621-695), kernel BlockScaledContiguousGroupedGemmKernel of
 * python/cudnn/grouped_gemm/grouped_gemm_dswiglu/grouped_gemm_dswiglu_quant.py (epilogue :2590-3095).
 */
int b200moe_dswiglu(const b200moe_gemm_args* args, void* stream);

/*
 * Weight gradient of a grouped GEMM: the experts partition the contraction dimension.  Fields of the argument
 * struct are read as follows:
 *   a  [m_rows, k] and b [n, k]: both contiguous along k = the total number of tokens (k / 2 bytes per row with
 *      E2M1 operands); expert e owns tokens [padded_offsets[e-1], padded_offsets[e]), a multiple of 32 each (an expert
 *      whose range is not gets a zero result and status 202 in b200moe_device_status);
 *   sfa, sfb: per expert the 128x4 layout of (m_rows, tokens_e / sf_vec) resp. (n, tokens_e / sf_vec), the experts'
 *      blocks one after the other (the layout torch's scaled_grouped_mm takes for its 2D-2D case);
 *   alpha, beta: optional per-expert scales (the reference's global_scale_a and global_scale_b), NULL = 1;
 *   d: [E, m_rows, n] bf16 / fp16 / float32 (d_dtype), d[e] = alpha_e beta_e (A_e SFA_e)(B_e SFB_e)^T, added to the existing
 *      contents with B200MOE_FLAG_ACCUMULATE; or (the reference's discrete output mode) d_peer_ptrs = int64 device array
 *      of E addresses of per-expert [m_rows, n] allocations, 16-byte aligned, and d may be NULL.  Everything else in
 *      the struct is ignored.
 * Replaces GroupedGemmWgradSm100.execute (python/cudnn/grouped_gemm/grouped_gemm_wgrad/api.py), kernel
 * BlockScaledMoEGroupedGemmWgradKernel (python/cudnn/grouped_gemm/grouped_gemm_wgrad/moe_blockscaled_grouped_gemm_wgrad.py).
 */
int b200moe_wgrad(const b200moe_gemm_args* args, void* stream);

/*
 * Bytes of caller-owned workspace a launch needs.  mode = B200MOE_WORKSPACE_DISCRETE (two 128-byte
 * tensor-map slots per expert) | B200MOE_WORKSPACE_DYNAMIC_SCHED (128 bytes for the tile counter);
 * 0 for a dense launch with the static schedule.  Mirrors the workspace the reference allocates in
 * compile() (python/cudnn/grouped_gemm/grouped_gemm_quant/grouped_gemm_quant.py:425-445: descriptors
 * plus a 4-byte counter).
 */
int64_t b200moe_workspace_bytes(int32_t num_experts, int32_t mode);

/*
 * Activation quantiser: x [rows, cols] bf16 (row pitch ld_elems) -> q [rows, cols] E4M3
 * + E8M0 scales per 32 elements along cols, written in the 128x4 layout of (rows, cols/32).
 * sf must hold ceil(rows/128) * ceil(cols/128) * 512 bytes.  No reference counterpart
 * (the reference's tests delegate input quantisation to TransformerEngine,
 * test/python/sdpa/mxfp8.py:137-187); the arithmetic is the row-quantisation formula of
 * grouped_gemm_swiglu_quant.py:1067-1139 with norm_const = 1.
 */
int b200moe_quantize_mxfp8(const void* x, int64_t rows, int64_t cols, int64_t ld_elems,
                           void* q, void* sf, void* stream);

/*
 * Routing helpers (no reference counterpart; the reference's tests build offsets on the
 * host, test/python/fe_api/test_grouped_gemm_swiglu_utils.py:270-312).
 *
 * b200moe_route: expert_ids [num_rows] int32 (expert of every routed row, token-major) ->
 *   counts [E] int32, padded_offsets [E] int32 END offsets with each group rounded up to
 *   m_aligned (1 = compact; the GEMMs need a multiple of 128), dst_row [num_rows] int32 = row of the expert-grouped padded buffer (stable:
 *   rows of one expert keep their order).  scratch: (E + 1) int32, caller-owned.
 * b200moe_scatter_rows: out[dst_row[r], :] = in[r / rows_per_src, :]  (bf16, cols % 8 == 0);
 *   also out_prob[dst_row[r]] = in_prob[r] when both are non-NULL.
 * b200moe_dispatch_quantize: fused dispatch-side pass.  For token t the bf16 row x[t, :] is read
 *   once, quantised to MXFP8 (same arithmetic as b200moe_quantize_mxfp8) and written to rows
 *   send_pos[t*topk + j] (j < topk; negative = skip) of q [R, cols] (E4M3), sf [R, cols/32] (E8M0,
 *   row-major: this buffer is for transport, not for the GEMM) and prob_out [R].
 * b200moe_place_quantized_rows: receive-side pass.  Arrival-order row i of (q_in, sf_in, prob_in)
 *   goes to row dst_row[i] of the GEMM operand: q_out [M, cols], sf_out in the 128x4 layout of
 *   (M, cols/32), prob_out [M].
 * b200moe_gather_rows: out[r, :] = in[src_row[r], :] (bf16; a negative index gives a zero row).
 * b200moe_combine_rows: out[t, :] = sum_j in[dst_row[t*topk + j], :] (bf16 in, f32 accumulate,
 *   bf16 out).
 */
int b200moe_route(const int32_t* expert_ids, int64_t num_rows, int32_t num_experts,
                  int32_t m_aligned, int32_t* counts, int32_t* padded_offsets, int32_t* dst_row,
                  int32_t* scratch, void* stream);
int64_t b200moe_route_scratch_bytes(int64_t num_rows, int32_t num_experts);
int b200moe_zero_pad_rows(void* buf, const int32_t* counts, const int32_t* padded_offsets,
                          int32_t num_experts, int64_t cols, float* prob, void* stream);
int b200moe_scatter_rows(const void* in, const int32_t* dst_row, int64_t num_rows,
                         int32_t rows_per_src, int64_t cols, void* out, const float* in_prob,
                         float* out_prob, void* stream);
int b200moe_dispatch_quantize(const void* x, const int32_t* send_pos, const float* topk_prob,
                              int64_t num_tokens, int32_t topk, int64_t cols, void* q, void* sf,
                              float* prob_out, void* stream);
int b200moe_place_quantized_rows(const void* q_in, const void* sf_in, const float* prob_in,
                                 const int32_t* dst_row, int64_t num_rows, int64_t cols, void* q_out,
                                 void* sf_out, float* prob_out, void* stream);
int b200moe_gather_rows(const void* in, const int32_t* src_row, int64_t num_rows, int64_t cols,
                        void* out, void* stream);
int b200moe_combine_rows(const void* in, const int32_t* dst_row, int64_t num_tokens, int32_t topk,
                         int64_t cols, void* out, void* stream);

/*
 * Expert-parallel dispatch over peer memory (no reference counterpart: the reference has no
 * multi-GPU code).  Replaces quantise + all-to-all + regroup by one kernel that stores over NVLink.
 *
 * b200moe_dispatch_quantize_peer: for token t the bf16 row x[t, :] is read once and quantised to
 *   MXFP8; for every slot j < topk with expert e = expert_ids[t*topk + j] the row goes to rank
 *   e / experts_per_rank, at row  r = delta[e] + local_row[t*topk + j]  of that rank's expert-grouped
 *   GEMM operand: E4M3 bytes to peer_q[rank] + r*cols as one bulk copy, and one record of
 *   b200moe_dispatch_record_pitch(cols) bytes to peer_rec[rank] + r*pitch as a second one:
 *   [cols/32 E8M0 bytes | padding | f32 gate probability | i32 return address
 *   my_rank*slot_capacity + t*topk + j].  The destination resets its records to all-ones before the
 *   step (return address -1 = padding row) and, after all ranks finished the kernel,
 *   b200moe_unpack_dispatch_records turns the first m_rows records into the swizzled 128x4 scale
 *   tensor, the prob vector and the d_row_map of its FC2.
 *   local_row = b200moe_route(..., m_aligned = 1) of this rank's rows; delta[e] = first row this rank
 *   owns inside expert e's group on the destination, minus this rank's compact start of e.
 *   peer_* are device arrays of G addresses.  Rows r outside [0, row_capacity) are not written and
 *   raise device status 301.  The caller orders the ranks (all ranks finish this kernel, then a
 *   barrier, then unpack and the GEMMs) -- the kernel itself never waits for a peer.
 *
 * b200moe_peer_alloc / _open / _close / _free: device buffers that other processes of this node can
 *   map (CUDA IPC).  alloc returns the pointer and a 64-byte handle to hand to the peers; open maps a
 *   peer's handle (peer access is enabled on first use) and close unmaps it.
 */
int b200moe_dispatch_quantize_peer(const void* x, const int32_t* expert_ids, const int32_t* local_row,
                                   const int32_t* delta, const float* topk_prob, int64_t num_tokens,
                                   int32_t topk, int64_t cols, int32_t experts_per_rank,
                                   int32_t num_ranks, int32_t my_rank, int64_t slot_capacity,
                                   int64_t row_capacity, const int64_t* peer_q,
                                   const int64_t* peer_rec, void* stream);
/* as above for one chunk of the destination rows only: row_bounds [num_ranks][num_chunks + 1] int32
   (device) holds, for every rank, the first row of each of its chunks (and its row count at the end);
   only slots whose destination row r on rank d has row_bounds[d][chunk] <= r < row_bounds[d][chunk + 1]
   are moved (NULL = all rows).  A layer that runs its rows in chunks dispatches chunk by chunk.
   max_blocks > 0 bounds the grid (the blocks then walk the tokens), so that the kernel can run beside a
   GEMM that owns most SMs. */
int b200moe_dispatch_quantize_peer_chunk(const void* x, const int32_t* expert_ids, const int32_t* local_row,
                                         const int32_t* delta, const float* topk_prob, int64_t num_tokens,
                                         int32_t topk, int64_t cols, int32_t experts_per_rank,
                                         int32_t num_ranks, int32_t my_rank, int64_t slot_capacity,
                                         int64_t row_capacity, const int64_t* peer_q,
                                         const int64_t* peer_rec, const int32_t* row_bounds,
                                         int32_t num_chunks, int32_t chunk, int32_t max_blocks, void* stream);
int b200moe_dispatch_record_pitch(int64_t cols);
/* count asynchronous device-to-device copies on one stream: segment i moves bytes[i] bytes from
   address src[i] to address dst[i] (HOST arrays of device addresses; peer-mapped buffers included).
   The copy engines do the work, no SM is used: this is how a layer returns result rows to the
   ranks they came from while its GEMMs keep running.  No reference counterpart. */
int b200moe_copy_segments(int32_t count, const int64_t* dst, const int64_t* src, const int64_t* bytes,
                          void* stream);
int b200moe_unpack_dispatch_records(const void* rec, int64_t m_rows, int64_t cols, void* sfa,
                                    float* prob, int32_t* row_map, void* stream);
int b200moe_peer_alloc(int64_t bytes, void** ptr, void* handle64);
int b200moe_peer_open(const void* handle64, void** ptr);
int b200moe_peer_close(void* ptr);
int b200moe_peer_free(void* ptr);

/* Last error text of the calling thread ("" if none).  Never NULL. */
const char* b200moe_last_error(void);

/*
 * Device-side status word of the current device: 0, or the code of the first bounded wait
 * that gave up inside a kernel (the kernel then returns early instead of hanging).  Reading
 * it synchronises the device; clear = 1 resets it.
 */
int b200moe_device_status(int clear);

/* ABI version of this header. */
int b200moe_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* B200MOE_H_ */
