// MXFP8 activation quantiser: bf16 [rows, cols] -> E4M3 [rows, cols] + one E8M0 scale per 32
// consecutive elements of a row, written in the 128x4 swizzled scale layout that the
// block-scaled tensor-core instruction consumes.
//
// HBM-bound: 2 B read + 1 B + 1/32 B written per element.  One CTA handles 128 rows x 256
// columns.  A warp reads one 512-byte row segment per instruction (16 B per lane, eight bf16),
// reduces |x| over the four lanes that share a 32-element block with two shuffles, converts
// and writes 8 B per lane (256 B per warp instruction).  The tile's 2 x 512 scale bytes are
// staged in shared memory in their final order and written with 16-byte stores.
#include "b200moe.h"
#include "common.cuh"

namespace b200moe {

constexpr int QT_ROWS = 128;
constexpr int QT_COLS = 256;
constexpr int QT_THREADS = 256;
// independent 16-byte loads in flight per lane: 4 gave 5.05 TB/s, 8 gives 6.28 TB/s, 16 spills (2.7 TB/s)
#ifndef QT_UNROLL
#define QT_UNROLL 8
#endif

__global__ void __launch_bounds__(QT_THREADS)
    quantize_mxfp8_kernel(const __nv_bfloat16* __restrict__ x, int64_t rows, int64_t cols,
                          int64_t ld, uint8_t* __restrict__ q, uint8_t* __restrict__ sf,
                          int rest_k) {
  __shared__ __align__(16) uint8_t s_sf[2][512];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row0 = (int64_t)blockIdx.y * QT_ROWS;
  const int64_t col0 = (int64_t)blockIdx.x * QT_COLS;
  const int64_t col = col0 + lane * 8;
  const bool col_ok = col < cols;  // cols is a multiple of 16, so a lane is all-in or all-out

  // rows beyond the tensor still get a (zero) scale so that the 128-row block is defined
  for (int i = threadIdx.x; i < 2 * 512 / 4; i += QT_THREADS) reinterpret_cast<uint32_t*>(s_sf)[i] = 0;
  __syncthreads();

  constexpr int ROWS_PER_WARP = QT_ROWS / (QT_THREADS / 32);  // 16
  constexpr int UNROLL = QT_UNROLL;  // independent 16-byte loads in flight per lane
#pragma unroll 1
  for (int rb = 0; rb < ROWS_PER_WARP; rb += UNROLL) {
    uint4 v[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int r = warp + (rb + u) * (QT_THREADS / 32);
      const int64_t row = row0 + r;
      v[u] = make_uint4(0, 0, 0, 0);
      if (col_ok && row < rows) v[u] = __ldg(reinterpret_cast<const uint4*>(x + row * ld + col));
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int r = warp + (rb + u) * (QT_THREADS / 32);
      const int64_t row = row0 + r;
      float f[8];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[u]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 t = __bfloat1622float2(h[j]);
        f[2 * j] = t.x;
        f[2 * j + 1] = t.y;
      }
      float amax = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(f[j]));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      // same operation order as the GEMM epilogue: amax * (1/448) * norm_const, norm_const = 1
      const float pv = amax * (1.0f / 448.0f);
      const uint32_t sfb = e8m0_from_float(pv);
      const float scale = quant_scale(1.0f, e8m0_to_float(sfb));
      uint2 o;
      o.x = e4m3x4_from_float(f[0] * scale, f[1] * scale, f[2] * scale, f[3] * scale);
      o.y = e4m3x4_from_float(f[4] * scale, f[5] * scale, f[6] * scale, f[7] * scale);
      if (col_ok && row < rows) *reinterpret_cast<uint2*>(q + row * cols + col) = o;
      if ((lane & 3) == 0 && col_ok) {
        const int kb = lane >> 2;  // 0..7 inside the tile
        s_sf[kb >> 2][(r & 31) * 16 + (r >> 5) * 4 + (kb & 3)] = (uint8_t)sfb;
      }
    }
  }
  __syncthreads();
  // two 512-byte chunks: K group (col0/128) and (col0/128 + 1) of row block blockIdx.y
  if (threadIdx.x < 64) {
    const int chunk = threadIdx.x >> 5;
    const int64_t kg = col0 / 128 + chunk;
    if (kg < rest_k) {
      uint8_t* dst = sf + ((int64_t)blockIdx.y * rest_k + kg) * 512 + (threadIdx.x & 31) * 16;
      *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(&s_sf[chunk][(threadIdx.x & 31) * 16]);
    }
  }
}

}  // namespace b200moe

extern "C" int b200moe_quantize_mxfp8(const void* x, int64_t rows, int64_t cols, int64_t ld_elems,
                                      void* q, void* sf, void* stream) {
  using namespace b200moe;
  if (rows == 0 || cols == 0) return B200MOE_OK;
  if (!x || !q || !sf) return fail(B200MOE_E_NULL, "quantize_mxfp8: null pointer");
  if (rows < 0 || cols < 0 || cols % 16 != 0 || ld_elems < cols || ld_elems % 8 != 0)
    return fail(B200MOE_E_SHAPE, "quantize_mxfp8: cols (%lld) must be a multiple of 16 and ld (%lld) >= cols, multiple of 8",
                (long long)cols, (long long)ld_elems);
  if (((uintptr_t)x | (uintptr_t)q | (uintptr_t)sf) & 15)
    return fail(B200MOE_E_ALIGN, "quantize_mxfp8: pointers must be 16-byte aligned");
  const int64_t row_blocks = (rows + QT_ROWS - 1) / QT_ROWS;
  const int64_t col_blocks = (cols + QT_COLS - 1) / QT_COLS;
  if (row_blocks > 65535) return fail(B200MOE_E_SHAPE, "quantize_mxfp8: too many rows (%lld)", (long long)rows);
  const int rest_k = (int)(((cols + 31) / 32 + 3) / 4);
  dim3 grid((unsigned)col_blocks, (unsigned)row_blocks);
  quantize_mxfp8_kernel<<<grid, QT_THREADS, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, rows, cols, ld_elems, (uint8_t*)q, (uint8_t*)sf, rest_k);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200MOE_OK;
}
