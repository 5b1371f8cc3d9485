// Routing helpers of the MoE layer: stable grouping of routed rows by expert, the padded
// per-expert END offsets the grouped GEMMs consume, row scatter (dispatch side) and the
// top-k combine.  All integer results are exact and deterministic (no float atomics, no
// order-dependent placement): rows of one expert keep their original order.
#include <algorithm>

#include "b200moe.h"
#include "common.cuh"

namespace b200moe {

constexpr int ROUTE_CHUNK = 1024;  // routed rows ranked by one warp

// per-chunk histogram: hist[chunk][e] = rows of expert e inside the chunk
__global__ void __launch_bounds__(256)
    route_hist_kernel(const int32_t* __restrict__ ids, int64_t num_rows, int num_experts, int32_t* __restrict__ hist) {
  extern __shared__ int s_hist[];
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x) s_hist[e] = 0;
  __syncthreads();
  const int64_t base = (int64_t)blockIdx.x * ROUTE_CHUNK;
  for (int i = threadIdx.x; i < ROUTE_CHUNK; i += blockDim.x) {
    const int64_t r = base + i;
    if (r < num_rows) {
      const int e = ids[r];
      if (e >= 0 && e < num_experts) atomicAdd(&s_hist[e], 1);
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x) hist[(int64_t)blockIdx.x * num_experts + e] = s_hist[e];
}

// one block: exclusive scan over chunks per expert (in place), counts, padded END offsets,
// group starts (scratch tail)
__global__ void __launch_bounds__(1024)
    route_scan_kernel(int32_t* __restrict__ hist, int num_chunks, int num_experts, int m_aligned,
                      int32_t* __restrict__ counts, int32_t* __restrict__ padded_offsets, int32_t* __restrict__ starts) {
  __shared__ int s_pad[1024];
  const int e = threadIdx.x;
  int run = 0;
  if (e < num_experts) {
    for (int c = 0; c < num_chunks; ++c) {
      const int v = hist[(int64_t)c * num_experts + e];
      hist[(int64_t)c * num_experts + e] = run;
      run += v;
    }
    counts[e] = run;
  }
  const int padded = e < num_experts ? ((run + m_aligned - 1) / m_aligned) * m_aligned : 0;
  s_pad[e] = padded;
  __syncthreads();
  // inclusive Hillis-Steele scan over up to 1024 experts
  for (int d = 1; d < 1024; d <<= 1) {
    const int t = e >= d ? s_pad[e - d] : 0;
    __syncthreads();
    s_pad[e] += t;
    __syncthreads();
  }
  if (e < num_experts) {
    padded_offsets[e] = s_pad[e];
    starts[e] = s_pad[e] - padded;
  }
}

// one warp per chunk: rows are visited in order, 32 at a time; lanes holding the same
// expert are ranked by lane index, so the placement is the stable sort order
__global__ void __launch_bounds__(32)
    route_place_kernel(const int32_t* __restrict__ ids, int64_t num_rows, int num_experts,
                       const int32_t* __restrict__ hist, const int32_t* __restrict__ starts,
                       int32_t* __restrict__ dst_row) {
  extern __shared__ int s_cnt[];
  const int lane = threadIdx.x;
  for (int e = lane; e < num_experts; e += 32)
    s_cnt[e] = starts[e] + hist[(int64_t)blockIdx.x * num_experts + e];
  __syncwarp();
  const int64_t base = (int64_t)blockIdx.x * ROUTE_CHUNK;
  for (int i = 0; i < ROUTE_CHUNK; i += 32) {
    const int64_t r = base + i + lane;
    const bool valid = r < num_rows;
    int e = valid ? ids[r] : -1;
    if (e < 0 || e >= num_experts) e = -1;
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    const int rank = __popc(peers & ((1u << lane) - 1));
    int slot = 0;
    if (e >= 0) slot = s_cnt[e] + rank;
    __syncwarp();
    if (e >= 0 && rank == 0) s_cnt[e] += __popc(peers);
    __syncwarp();
    if (valid) dst_row[r] = e >= 0 ? slot : -1;
  }
}

// out[dst_row[r], :] = in[r / rows_per_src, :], 16 bytes per thread per step
__global__ void __launch_bounds__(128)
    scatter_rows_kernel(const uint4* __restrict__ in, const int32_t* __restrict__ dst_row, int rows_per_src,
                        int vec_per_row, uint4* __restrict__ out, const float* __restrict__ in_prob,
                        float* __restrict__ out_prob) {
  const int64_t r = blockIdx.x;
  const int d = dst_row[r];
  if (d < 0) return;
  const uint4* src = in + (r / rows_per_src) * vec_per_row;
  uint4* dst = out + (int64_t)d * vec_per_row;
  for (int i = threadIdx.x; i < vec_per_row; i += blockDim.x) dst[i] = __ldg(src + i);
  if (threadIdx.x == 0 && in_prob && out_prob) out_prob[d] = in_prob[r];
}

// out[r, :] = in[src_row[r], :]
__global__ void __launch_bounds__(128)
    gather_rows_kernel(const uint4* __restrict__ in, const int32_t* __restrict__ src_row, int vec_per_row,
                       uint4* __restrict__ out) {
  const int64_t r = blockIdx.x;
  const int s = src_row[r];
  uint4* dst = out + r * vec_per_row;
  if (s < 0) {
    for (int i = threadIdx.x; i < vec_per_row; i += blockDim.x) dst[i] = make_uint4(0, 0, 0, 0);
    return;
  }
  const uint4* src = in + (int64_t)s * vec_per_row;
  for (int i = threadIdx.x; i < vec_per_row; i += blockDim.x) dst[i] = __ldg(src + i);
}

// Dispatch side, fused: one block per token reads the bf16 row once, quantises it to MXFP8 and
// writes the E4M3 row, its E8M0 scales (row-major, cols / 32 bytes per row) and the gate
// probability to each of the token's `topk` positions of the send buffers.
__global__ void __launch_bounds__(128)
    dispatch_quantize_kernel(const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ send_pos,
                             const float* __restrict__ topk_prob, int topk, int cols, uint8_t* __restrict__ q,
                             uint8_t* __restrict__ sf, float* __restrict__ prob_out) {
  const int64_t t = blockIdx.x;
  const int lane = threadIdx.x & 31;
  const int sf_cols = cols / 32;
  __shared__ int s_dst[16];
  if (threadIdx.x < topk) {
    const int d = send_pos[t * topk + threadIdx.x];
    s_dst[threadIdx.x] = d;
    if (d >= 0 && prob_out) prob_out[d] = topk_prob ? topk_prob[t * topk + threadIdx.x] : 1.0f;
  }
  __syncthreads();
  for (int v = threadIdx.x; v < cols / 8; v += blockDim.x) {
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(x + t * cols) + v);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
    float f[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 p2 = __bfloat1622float2(h[j]);
      f[2 * j] = p2.x;
      f[2 * j + 1] = p2.y;
    }
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(f[j]));
    // the four lanes of one 32-element block are consecutive lanes of one warp (cols % 32 == 0)
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    const uint32_t sfb = e8m0_from_float(amax * (1.0f / 448.0f));
    const float scale = quant_scale(1.0f, e8m0_to_float(sfb));
    uint2 o;
    o.x = e4m3x4_from_float(f[0] * scale, f[1] * scale, f[2] * scale, f[3] * scale);
    o.y = e4m3x4_from_float(f[4] * scale, f[5] * scale, f[6] * scale, f[7] * scale);
    for (int j = 0; j < topk; ++j) {
      const int d = s_dst[j];
      if (d < 0) continue;
      reinterpret_cast<uint2*>(q + (int64_t)d * cols)[v] = o;
      if ((lane & 3) == 0) sf[(int64_t)d * sf_cols + (v >> 2)] = (uint8_t)sfb;
    }
  }
}

// Dispatch over peer memory: as dispatch_quantize_kernel, but every slot's row goes straight into
// the expert-grouped GEMM operand of the rank that owns the expert.  The quantised row is built once
// in shared memory and leaves as one asynchronous bulk copy per slot; the row's scales travel with
// the slot's gate probability and return address as one small record per slot (a second bulk copy),
// because thousands of 4-byte stores per row are what NVLink is worst at.  Record layout
// (rec_pitch bytes, a multiple of 16): [cols / 32 scale bytes | padding | f32 prob | i32 return address].
__global__ void __launch_bounds__(128)
    dispatch_quantize_peer_kernel(const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ expert_ids,
                                  const int32_t* __restrict__ local_row, const int32_t* __restrict__ delta,
                                  const float* __restrict__ topk_prob, int64_t num_tokens, int topk, int cols, int rec_pitch,
                                  int experts_per_rank, int num_ranks, int my_rank, int64_t slot_capacity, int64_t row_capacity,
                                  const int32_t* __restrict__ row_bounds, int num_chunks, int chunk,
                                  const int64_t* __restrict__ peer_q, const int64_t* __restrict__ peer_rec) {
  extern __shared__ __align__(16) uint8_t s_dyn[];  // [cols] E4M3 row, then topk records of rec_pitch bytes
  uint8_t* const s_qrow = s_dyn;
  uint8_t* const s_rec = s_dyn + cols;
  const int lane = threadIdx.x & 31;
  __shared__ int64_t s_row[16];
  __shared__ int s_rank[16];
  __shared__ int s_any;
  // a block walks tokens blockIdx.x, blockIdx.x + gridDim.x, ...: one token per block when the grid is
  // the token count, a few persistent blocks when the kernel shares the GPU with a GEMM
  for (int64_t t = blockIdx.x; t < num_tokens; t += gridDim.x) {
    if (threadIdx.x == 0) s_any = 0;
    __syncthreads();
    if (threadIdx.x < topk) {
      const int64_t slot = t * topk + threadIdx.x;
      const int e = expert_ids[slot];
      int64_t row = -1;
      int rank = 0;
      if (e >= 0 && e < experts_per_rank * num_ranks) {
        rank = e / experts_per_rank;
        row = (int64_t)delta[e] + local_row[slot];
        if (row < 0 || row >= row_capacity) {
          atomicCAS(&g_device_status, 0, 301);  // never store outside a peer's buffer
          row = -1;
        } else if (row_bounds != nullptr) {
          // this launch moves only the rows that land in chunk `chunk` of their destination rank
          const int32_t* b = row_bounds + rank * (num_chunks + 1) + chunk;
          if (row < b[0] || row >= b[1]) row = -1;
        }
      }
      s_row[threadIdx.x] = row;
      s_rank[threadIdx.x] = rank;
      if (row >= 0) s_any = 1;
      uint8_t* rec = s_rec + threadIdx.x * rec_pitch;
      *reinterpret_cast<float*>(rec + rec_pitch - 8) = topk_prob ? topk_prob[slot] : 1.0f;
      *reinterpret_cast<int32_t*>(rec + rec_pitch - 4) = (int32_t)(my_rank * slot_capacity + slot);
    }
    __syncthreads();
    if (!s_any) continue;  // no slot of this token belongs to this launch's experts (block-uniform)
    // the row is read in batches of four 16-byte loads per thread, all issued before the first use
    const int vecs = cols / 8;
    const uint4* xrow = reinterpret_cast<const uint4*>(x + t * cols);
    for (int v0 = threadIdx.x; v0 < vecs; v0 += 4 * blockDim.x) {
      uint4 raw4[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int v = v0 + u * blockDim.x;
        raw4[u] = v < vecs ? __ldg(xrow + v) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int v = v0 + u * blockDim.x;
        // whole warps run in or out together: vecs is a multiple of 32 (host check), v - lane too
        if (v - lane >= vecs) break;
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw4[u]);
        float f[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 p2 = __bfloat1622float2(h[j]);
          f[2 * j] = p2.x;
          f[2 * j + 1] = p2.y;
        }
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(f[j]));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        const uint32_t sfb = e8m0_from_float(amax * (1.0f / 448.0f));
        const float scale = quant_scale(1.0f, e8m0_to_float(sfb));
        uint2 o;
        o.x = e4m3x4_from_float(f[0] * scale, f[1] * scale, f[2] * scale, f[3] * scale);
        o.y = e4m3x4_from_float(f[4] * scale, f[5] * scale, f[6] * scale, f[7] * scale);
        reinterpret_cast<uint2*>(s_qrow)[v] = o;
        if ((lane & 3) == 0) {
          for (int j = 0; j < topk; ++j) s_rec[j * rec_pitch + (v >> 2)] = (uint8_t)sfb;
        }
      }
    }
    fence_proxy_async_smem();  // this thread's writes, for the bulk copies below
    __syncthreads();
    if (threadIdx.x < topk) {
      const int64_t row = s_row[threadIdx.x];
      if (row >= 0) {
        const int rank = s_rank[threadIdx.x];
        bulk_store(reinterpret_cast<uint8_t*>(peer_q[rank]) + row * cols, smem_u32(s_qrow), (uint32_t)cols);
        bulk_store(reinterpret_cast<uint8_t*>(peer_rec[rank]) + row * rec_pitch, smem_u32(s_rec + threadIdx.x * rec_pitch),
                   (uint32_t)rec_pitch);
      }
      bulk_commit();
      bulk_wait_read0();  // shared memory must outlive the copies' reads
    }
    __syncthreads();  // the next token reuses the row and the records
  }
}

// Receive side of the peer dispatch, after the ranks' barrier: records -> scales in the swizzled
// 128x4 layout, gate probabilities and return addresses of the first m_rows rows.  A record that no
// sender wrote still holds the reset pattern (all bits set): return address -1, the row is padding.
__global__ void __launch_bounds__(256)
    unpack_dispatch_records_kernel(const uint8_t* __restrict__ rec, int64_t m_rows, int sf_cols, int rec_pitch, int rest_k,
                                   uint8_t* __restrict__ sfa, float* __restrict__ prob, int32_t* __restrict__ row_map) {
  const int words = (sf_cols + 3) / 4;  // 4 scale bytes = 4 consecutive bytes of the swizzled layout
  const int64_t total = m_rows * (words + 1);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / (words + 1);
    const int w = (int)(i - row * (words + 1));
    const uint8_t* r = rec + row * rec_pitch;
    if (w == words) {
      const int32_t ret = *reinterpret_cast<const int32_t*>(r + rec_pitch - 4);
      row_map[row] = ret;
      prob[row] = ret < 0 ? 0.f : *reinterpret_cast<const float*>(r + rec_pitch - 8);
    } else if (4 * w + 4 <= sf_cols) {
      *reinterpret_cast<uint32_t*>(sfa + sf_offset(row, 4 * w, rest_k)) = *reinterpret_cast<const uint32_t*>(r + 4 * w);
    } else {
      for (int kb = 4 * w; kb < sf_cols; ++kb) sfa[sf_offset(row, kb, rest_k)] = r[kb];
    }
  }
}

// Receive side: row i of the arrival-order buffers goes to row dst_row[i] of the expert-grouped
// operand; its scales are written into the 128x4 swizzled layout the GEMM reads.
__global__ void __launch_bounds__(128)
    place_quantized_rows_kernel(const uint8_t* __restrict__ q_in, const uint8_t* __restrict__ sf_in,
                                const float* __restrict__ prob_in, const int32_t* __restrict__ dst_row, int cols,
                                int rest_k, uint8_t* __restrict__ q_out, uint8_t* __restrict__ sf_out,
                                float* __restrict__ prob_out) {
  const int64_t i = blockIdx.x;
  const int d = dst_row[i];
  if (d < 0) return;
  const uint4* src = reinterpret_cast<const uint4*>(q_in + i * cols);
  uint4* dst = reinterpret_cast<uint4*>(q_out + (int64_t)d * cols);
  for (int v = threadIdx.x; v < cols / 16; v += blockDim.x) dst[v] = __ldg(src + v);
  const int sf_cols = cols / 32;
  for (int kb = threadIdx.x; kb < sf_cols; kb += blockDim.x) sf_out[sf_offset(d, kb, rest_k)] = sf_in[i * sf_cols + kb];
  if (threadIdx.x == 0 && prob_in && prob_out) prob_out[d] = prob_in[i];
}

// rows [start_e + count_e, end_e) of every expert group are set to zero
__global__ void __launch_bounds__(128)
    zero_pad_rows_kernel(uint4* __restrict__ buf, const int32_t* __restrict__ counts,
                         const int32_t* __restrict__ padded_offsets, int vec_per_row, float* __restrict__ prob) {
  const int e = blockIdx.x;
  const int end = padded_offsets[e];
  const int start = e == 0 ? 0 : padded_offsets[e - 1];
  for (int row = start + counts[e] + blockIdx.y; row < end; row += gridDim.y) {
    uint4* dst = buf + (int64_t)row * vec_per_row;
    for (int i = threadIdx.x; i < vec_per_row; i += blockDim.x) dst[i] = make_uint4(0, 0, 0, 0);
    if (prob && threadIdx.x == 0) prob[row] = 0.f;
  }
}

// out[t, :] = sum_j in[dst_row[t * topk + j], :], float32 accumulation in slot order
__global__ void __launch_bounds__(128)
    combine_rows_kernel(const uint4* __restrict__ in, const int32_t* __restrict__ dst_row, int topk, int vec_per_row,
                        uint4* __restrict__ out) {
  const int64_t t = blockIdx.x;
  for (int i = threadIdx.x; i < vec_per_row; i += blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int j = 0; j < topk; ++j) {
      const int d = dst_row[t * topk + j];
      if (d < 0) continue;
      const uint4 v = __ldg(in + (int64_t)d * vec_per_row + i);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = __bfloat1622float2(h[q]);
        acc[2 * q] += f.x;
        acc[2 * q + 1] += f.y;
      }
    }
    uint4 o;
    o.x = bf16x2_from_float(acc[0], acc[1]);
    o.y = bf16x2_from_float(acc[2], acc[3]);
    o.z = bf16x2_from_float(acc[4], acc[5]);
    o.w = bf16x2_from_float(acc[6], acc[7]);
    out[t * vec_per_row + i] = o;
  }
}

}  // namespace b200moe

extern "C" {

int64_t b200moe_route_scratch_bytes(int64_t num_rows, int32_t num_experts) {
  const int64_t chunks = (num_rows + b200moe::ROUTE_CHUNK - 1) / b200moe::ROUTE_CHUNK;
  return (chunks * num_experts + num_experts) * (int64_t)sizeof(int32_t);
}

int b200moe_route(const int32_t* expert_ids, int64_t num_rows, int32_t num_experts, int32_t m_aligned, int32_t* counts,
                  int32_t* padded_offsets, int32_t* dst_row, int32_t* scratch, void* stream_v) {
  using namespace b200moe;
  cudaStream_t stream = (cudaStream_t)stream_v;
  if (num_experts <= 0 || num_experts > 1024) return fail(B200MOE_E_SHAPE, "route: num_experts must be in [1, 1024], got %d", num_experts);
  if (m_aligned <= 0) return fail(B200MOE_E_SHAPE, "route: m_aligned must be positive");
  if (num_rows < 0 || num_rows > (1ll << 30)) return fail(B200MOE_E_SHAPE, "route: bad num_rows");
  if (!counts || !padded_offsets || !scratch || (num_rows > 0 && (!expert_ids || !dst_row)))
    return fail(B200MOE_E_NULL, "route: null pointer");
  const int chunks = (int)((num_rows + ROUTE_CHUNK - 1) / ROUTE_CHUNK);
  int32_t* hist = scratch;
  int32_t* starts = scratch + (int64_t)chunks * num_experts;
  if (chunks > 0) {
    route_hist_kernel<<<chunks, 256, num_experts * sizeof(int), stream>>>(expert_ids, num_rows, num_experts, hist);
    B200_CUDA_CHECK(cudaGetLastError());
  }
  route_scan_kernel<<<1, 1024, 0, stream>>>(hist, chunks, num_experts, m_aligned, counts, padded_offsets, starts);
  B200_CUDA_CHECK(cudaGetLastError());
  if (chunks > 0) {
    route_place_kernel<<<chunks, 32, num_experts * sizeof(int), stream>>>(expert_ids, num_rows, num_experts, hist, starts, dst_row);
    B200_CUDA_CHECK(cudaGetLastError());
  }
  return B200MOE_OK;
}

int b200moe_scatter_rows(const void* in, const int32_t* dst_row, int64_t num_rows, int32_t rows_per_src, int64_t cols,
                         void* out, const float* in_prob, float* out_prob, void* stream) {
  using namespace b200moe;
  if (num_rows == 0) return B200MOE_OK;
  if (!in || !dst_row || !out) return fail(B200MOE_E_NULL, "scatter_rows: null pointer");
  if (cols <= 0 || cols % 8 != 0 || rows_per_src <= 0 || num_rows < 0 || num_rows > 0x7fffffffll)
    return fail(B200MOE_E_SHAPE, "scatter_rows: cols must be a positive multiple of 8");
  if (((uintptr_t)in | (uintptr_t)out) & 15) return fail(B200MOE_E_ALIGN, "scatter_rows: 16-byte alignment required");
  scatter_rows_kernel<<<(unsigned)num_rows, 128, 0, (cudaStream_t)stream>>>((const uint4*)in, dst_row, rows_per_src,
                                                                           (int)(cols / 8), (uint4*)out, in_prob, out_prob);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200MOE_OK;
}

int b200moe_gather_rows(const void* in, const int32_t* src_row, int64_t num_rows, int64_t cols, void* out, void* stream) {
  using namespace b200moe;
  if (num_rows == 0) return B200MOE_OK;
  if (!in || !src_row || !out) return fail(B200MOE_E_NULL, "gather_rows: null pointer");
  if (cols <= 0 || cols % 8 != 0 || num_rows < 0 || num_rows > 0x7fffffffll)
    return fail(B200MOE_E_SHAPE, "gather_rows: cols must be a positive multiple of 8");
  if (((uintptr_t)in | (uintptr_t)out) & 15) return fail(B200MOE_E_ALIGN, "gather_rows: 16-byte alignment required");
  gather_rows_kernel<<<(unsigned)num_rows, 128, 0, (cudaStream_t)stream>>>((const uint4*)in, src_row, (int)(cols / 8), (uint4*)out);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200MOE_OK;
}

int b200moe_dispatch_quantize(const void* x, const int32_t* send_pos, const float* topk_prob, int64_t num_tokens,
                              int32_t topk, int64_t cols, void* q, void* sf, float* prob_out, void* stream) {
  using namespace b200moe;
  if (num_tokens == 0) return B200MOE_OK;
  if (!x || !send_pos || !q || !sf) return fail(B200MOE_E_NULL, "dispatch_quantize: null pointer");
  if (cols <= 0 || cols % 32 != 0 || topk <= 0 || topk > 16 || num_tokens < 0 || num_tokens > 0x7fffffffll)
    return fail(B200MOE_E_SHAPE, "dispatch_quantize: cols must be a positive multiple of 32 and topk in [1, 16]");
  if (((uintptr_t)x | (uintptr_t)q) & 15) return fail(B200MOE_E_ALIGN, "dispatch_quantize: 16-byte alignment required");
  dispatch_quantize_kernel<<<(unsigned)num_tokens, 128, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, send_pos, topk_prob, topk, (int)cols, (uint8_t*)q, (uint8_t*)sf, prob_out);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200MOE_OK;
}

int b200moe_dispatch_record_pitch(int64_t cols) { return (int)(((cols / 32 + 8) + 15) / 16 * 16); }

int b200moe_dispatch_quantize_peer_chunk(const void* x, const int32_t* expert_ids, const int32_t* local_row, const int32_t* delta,
                                         const float* topk_prob, int64_t num_tokens, int32_t topk, int64_t cols,
                                         int32_t experts_per_rank, int32_t num_ranks, int32_t my_rank, int64_t slot_capacity,
                                         int64_t row_capacity, const int64_t* peer_q, const int64_t* peer_rec,
                                         const int32_t* row_bounds, int32_t num_chunks, int32_t chunk, int32_t max_blocks,
                                         void* stream) {
  using namespace b200moe;
  if (num_tokens == 0) return B200MOE_OK;
  if (!x || !expert_ids || !local_row || !delta || !peer_q || !peer_rec)
    return fail(B200MOE_E_NULL, "dispatch_quantize_peer: null pointer");
  // whole warps only (full-mask shuffles inside the row loop): 32 lanes x 8 columns
  if (cols <= 0 || cols % 256 != 0 || topk <= 0 || topk > 16 || num_tokens < 0 || num_tokens > 0x7fffffffll)
    return fail(B200MOE_E_SHAPE, "dispatch_quantize_peer: cols must be a positive multiple of 256 and topk in [1, 16]");
  if (experts_per_rank <= 0 || num_ranks <= 0 || my_rank < 0 || my_rank >= num_ranks || slot_capacity < num_tokens * topk ||
      (int64_t)num_ranks * slot_capacity > 0x7fffffffll || row_capacity <= 0)
    return fail(B200MOE_E_SHAPE, "dispatch_quantize_peer: bad rank layout or capacities");
  if (max_blocks < 0) return fail(B200MOE_E_SHAPE, "dispatch_quantize_peer: negative block limit");
  if (row_bounds && (num_chunks <= 0 || chunk < 0 || chunk >= num_chunks))
    return fail(B200MOE_E_SHAPE, "dispatch_quantize_peer: chunk %d outside [0, %d)", chunk, num_chunks);
  if ((uintptr_t)x & 15) return fail(B200MOE_E_ALIGN, "dispatch_quantize_peer: 16-byte alignment required");
  const int rec_pitch = b200moe_dispatch_record_pitch(cols);
  const size_t smem = (size_t)cols + (size_t)topk * rec_pitch;
  if (smem > 48 * 1024) return fail(B200MOE_E_SHAPE, "dispatch_quantize_peer: a row and its records must fit 48 KiB of shared memory");
  const int64_t blocks = max_blocks > 0 ? std::min<int64_t>(max_blocks, num_tokens) : num_tokens;
  dispatch_quantize_peer_kernel<<<(unsigned)blocks, 128, smem, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, expert_ids, local_row, delta, topk_prob, num_tokens, topk, (int)cols, rec_pitch, experts_per_rank,
      num_ranks, my_rank, slot_capacity, row_capacity, row_bounds, num_chunks, chunk, peer_q, peer_rec);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200MOE_OK;
}

int b200moe_dispatch_quantize_peer(const void* x, const int32_t* expert_ids, const int32_t* local_row, const int32_t* delta,
                                   const float* topk_prob, int64_t num_tokens, int32_t topk, int64_t cols,
                                   int32_t experts_per_rank, int32_t num_ranks, int32_t my_rank, int64_t slot_capacity,
                                   int64_t row_capacity, const int64_t* peer_q, const int64_t* peer_rec, void* stream) {
  return b200moe_dispatch_quantize_peer_chunk(x, expert_ids, local_row, delta, topk_prob, num_tokens, topk, cols, experts_per_rank,
                                              num_ranks, my_rank, slot_capacity, row_capacity, peer_q, peer_rec, nullptr, 0, 0, 0, stream);
}

int b200moe_copy_segments(int32_t count, const int64_t* dst, const int64_t* src, const int64_t* bytes, void* stream) {
  using namespace b200moe;
  if (count < 0 || (count > 0 && (!dst || !src || !bytes))) return fail(B200MOE_E_NULL, "copy_segments: null table");
  for (int i = 0; i < count; ++i) {
    if (bytes[i] < 0 || (bytes[i] > 0 && (!dst[i] || !src[i]))) return fail(B200MOE_E_NULL, "copy_segments: segment %d is null or negative", i);
  }
  // one asynchronous device-to-device copy per segment (copy engines: no SM takes part)
  for (int i = 0; i < count; ++i) {
    if (bytes[i] == 0) continue;
    B200_CUDA_CHECK(cudaMemcpyAsync(reinterpret_cast<void*>(dst[i]), reinterpret_cast<const void*>(src[i]), (size_t)bytes[i],
                                    cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
  }
  return B200MOE_OK;
}

int b200moe_unpack_dispatch_records(const void* rec, int64_t m_rows, int64_t cols, void* sfa, float* prob, int32_t* row_map,
                                    void* stream) {
  using namespace b200moe;
  if (m_rows == 0) return B200MOE_OK;
  if (!rec || !sfa || !prob || !row_map) return fail(B200MOE_E_NULL, "unpack_dispatch_records: null pointer");
  if (cols <= 0 || cols % 32 != 0 || m_rows < 0 || m_rows > 0x7fffffffll)
    return fail(B200MOE_E_SHAPE, "unpack_dispatch_records: cols must be a positive multiple of 32");
  const int sf_cols = (int)(cols / 32);
  const int rest_k = (sf_cols + 3) / 4;
  const int64_t total = m_rows * ((sf_cols + 3) / 4 + 1);
  const unsigned blocks = (unsigned)std::min<int64_t>((total + 255) / 256, 148 * 32);
  unpack_dispatch_records_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(
      (const uint8_t*)rec, m_rows, sf_cols, b200moe_dispatch_record_pitch(cols), rest_k, (uint8_t*)sfa, prob, row_map);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200MOE_OK;
}

int b200moe_peer_alloc(int64_t bytes, void** ptr, void* handle64) {
  using namespace b200moe;
  if (!ptr || !handle64 || bytes <= 0) return fail(B200MOE_E_NULL, "peer_alloc: null pointer or empty size");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  B200_CUDA_CHECK(cudaMalloc(ptr, (size_t)bytes));
  cudaIpcMemHandle_t h;
  const cudaError_t e = cudaIpcGetMemHandle(&h, *ptr);
  if (e != cudaSuccess) {
    cudaFree(*ptr);
    *ptr = nullptr;
    B200_CUDA_CHECK(e);
  }
  memcpy(handle64, &h, 64);
  return B200MOE_OK;
}

int b200moe_peer_open(const void* handle64, void** ptr) {
  using namespace b200moe;
  if (!ptr || !handle64) return fail(B200MOE_E_NULL, "peer_open: null pointer");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  B200_CUDA_CHECK(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return B200MOE_OK;
}

int b200moe_peer_close(void* ptr) {
  using namespace b200moe;
  if (ptr) B200_CUDA_CHECK(cudaIpcCloseMemHandle(ptr));
  return B200MOE_OK;
}

int b200moe_peer_free(void* ptr) {
  using namespace b200moe;
  if (ptr) B200_CUDA_CHECK(cudaFree(ptr));
  return B200MOE_OK;
}

int b200moe_place_quantized_rows(const void* q_in, const void* sf_in, const float* prob_in, const int32_t* dst_row,
                                 int64_t num_rows, int64_t cols, void* q_out, void* sf_out, float* prob_out, void* stream) {
  using namespace b200moe;
  if (num_rows == 0) return B200MOE_OK;
  if (!q_in || !sf_in || !dst_row || !q_out || !sf_out) return fail(B200MOE_E_NULL, "place_quantized_rows: null pointer");
  if (cols <= 0 || cols % 32 != 0 || num_rows < 0 || num_rows > 0x7fffffffll)
    return fail(B200MOE_E_SHAPE, "place_quantized_rows: cols must be a positive multiple of 32");
  if (((uintptr_t)q_in | (uintptr_t)q_out) & 15) return fail(B200MOE_E_ALIGN, "place_quantized_rows: 16-byte alignment required");
  const int rest_k = (int)((cols / 32 + 3) / 4);
  place_quantized_rows_kernel<<<(unsigned)num_rows, 128, 0, (cudaStream_t)stream>>>(
      (const uint8_t*)q_in, (const uint8_t*)sf_in, prob_in, dst_row, (int)cols, rest_k, (uint8_t*)q_out, (uint8_t*)sf_out, prob_out);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200MOE_OK;
}

int b200moe_zero_pad_rows(void* buf, const int32_t* counts, const int32_t* padded_offsets, int32_t num_experts,
                          int64_t cols, float* prob, void* stream) {
  using namespace b200moe;
  if (num_experts == 0) return B200MOE_OK;
  if (!buf || !counts || !padded_offsets) return fail(B200MOE_E_NULL, "zero_pad_rows: null pointer");
  if (cols <= 0 || cols % 8 != 0) return fail(B200MOE_E_SHAPE, "zero_pad_rows: cols must be a positive multiple of 8");
  dim3 grid((unsigned)num_experts, 8);
  zero_pad_rows_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>((uint4*)buf, counts, padded_offsets, (int)(cols / 8), prob);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200MOE_OK;
}

int b200moe_combine_rows(const void* in, const int32_t* dst_row, int64_t num_tokens, int32_t topk, int64_t cols, void* out,
                         void* stream) {
  using namespace b200moe;
  if (num_tokens == 0) return B200MOE_OK;
  if (!in || !dst_row || !out) return fail(B200MOE_E_NULL, "combine_rows: null pointer");
  if (cols <= 0 || cols % 8 != 0 || topk <= 0 || num_tokens < 0 || num_tokens > 0x7fffffffll)
    return fail(B200MOE_E_SHAPE, "combine_rows: cols must be a positive multiple of 8");
  if (((uintptr_t)in | (uintptr_t)out) & 15) return fail(B200MOE_E_ALIGN, "combine_rows: 16-byte alignment required");
  combine_rows_kernel<<<(unsigned)num_tokens, 128, 0, (cudaStream_t)stream>>>((const uint4*)in, dst_row, topk, (int)(cols / 8),
                                                                             (uint4*)out);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200MOE_OK;
}

}  // extern "C"
