// Shared device helpers: PTX wrappers for mbarrier, TMA, tcgen05 (sm_100a) and number formats.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200moe {

// ---------------------------------------------------------------------------------------
// Host-side error plumbing (thread-local text, int status codes across the C ABI)
// ---------------------------------------------------------------------------------------
void set_error(const char* fmt, ...);
int fail(int code, const char* fmt, ...);

#define B200_CUDA_CHECK(expr)                                                        \
  do {                                                                               \
    cudaError_t _e = (expr);                                                         \
    if (_e != cudaSuccess) {                                                         \
      return ::b200moe::fail((int)_e, "%s failed: %s", #expr, cudaGetErrorString(_e)); \
    }                                                                                \
  } while (0)

// Device status word: first bounded wait that gave up records its code here.  The library is
// built as one translation unit (b200moe.cu includes every kernel file), so this is the single
// definition.
__device__ int g_device_status = 0;

// ---------------------------------------------------------------------------------------
// Small utilities
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint32_t lane_id() { return threadIdx.x & 31; }

// Asynchronous row copy shared memory -> global memory (also a peer GPU's), tracked by bulk groups.
// Both addresses 16-byte aligned, size a multiple of 16 bytes.
__device__ __forceinline__ void bulk_store(void* gdst, uint32_t smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// the issuing thread's copies have finished reading shared memory (it may be rewritten)
__device__ __forceinline__ void bulk_wait_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// the issuing thread's copies are complete
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// True in exactly one lane of a converged warp.  Unlike a `lane == 0` test, the compiler knows
// the warp stays convergent around the elected region, so descriptors and addresses of TMA and
// tcgen05 instructions can live in uniform registers.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      "elect.sync _|P, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t"
      "}"
      : "=r"(pred));
  return pred != 0;
}

// ---------------------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done;
}

// Bounded wait.  Spins on the barrier phase; after `limit_ns` without progress it records
// `code` in the device status word, raises the CTA's abort flag and returns false so the
// caller can leave its loop and fall through to the kernel's teardown.  A raised abort flag
// makes every other waiter of the CTA give up quickly as well.
constexpr uint64_t kWaitLimitNs = 4000000000ull;  // default limit, 4 s: far above any legitimate wait

struct WaitCtx {
  volatile int* abort_flag;
  uint64_t limit_ns;
};

// kCluster: acquire at cluster scope (the data guarded by the barrier was written by the other CTA
// of the pair)
template <bool kCluster = false>
__device__ __forceinline__ uint32_t mbar_try_wait_scoped(uint32_t bar, uint32_t parity) {
  if constexpr (!kCluster) {
    return mbar_try_wait(bar, parity);
  } else {
    uint32_t done;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done;
  }
}

// The same test with a suspend-time hint: the thread may sleep up to `hint_ns` for the phase to complete
// instead of returning at once, so a long wait costs a few instructions instead of a busy loop.
template <bool kCluster = false>
__device__ __forceinline__ uint32_t mbar_try_wait_hint(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t done;
  if constexpr (!kCluster) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(done)
        : "r"(bar), "r"(parity), "r"(hint_ns)
        : "memory");
  } else {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(done)
        : "r"(bar), "r"(parity), "r"(hint_ns)
        : "memory");
  }
  return done;
}

constexpr uint32_t kWaitHintNs = 20000;

// The part of a wait that runs when the phase has not completed yet: kept out of line, so that a wait costs its
// caller a test and a branch and the loops of the producer, issuer and epilogue warps stay short.
template <bool kCluster>
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int* abort_flag, uint64_t limit_ns, int code) {
#pragma unroll 1
  for (int i = 0; i < 64; ++i) {
    if (mbar_try_wait_hint<kCluster>(bar, parity, kWaitHintNs)) return true;
  }
  const uint64_t t0 = global_timer_ns();
#pragma unroll 1
  while (true) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      if (mbar_try_wait_hint<kCluster>(bar, parity, kWaitHintNs)) return true;
    }
    if (*abort_flag) return false;
    if (global_timer_ns() - t0 > limit_ns) {
      atomicCAS(&g_device_status, 0, code);
      *abort_flag = 1;
      return false;
    }
  }
}

template <bool kCluster = false>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const WaitCtx& w, int code) {
  if (mbar_try_wait_scoped<kCluster>(bar, parity)) return true;
  return mbar_wait_slow<kCluster>(bar, parity, w.abort_flag, w.limit_ns, code);
}

// ---------------------------------------------------------------------------------------
// TMA: tiled bulk tensor loads, always into the issuing CTA's own shared memory
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, uint32_t bar, int c0,
                                            int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, "
      "{%3, %4}], [%2];" ::"r"(dst),
      "l"(tmap), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const void* tmap, uint32_t bar, int c0,
                                            int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, "
      "{%3, %4, %5}], [%2];" ::"r"(dst),
      "l"(tmap), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

// Pair (cta_group::2) forms: data lands in the issuing CTA's shared memory, the transaction
// bytes are credited to an mbarrier that may live in either CTA of the pair (the leader's).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const void* tmap, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, "
      "{%3, %4}], [%2];" ::"r"(dst),
      "l"(tmap), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const void* tmap, uint32_t bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, "
      "{%3, %4, %5}], [%2];" ::"r"(dst),
      "l"(tmap), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d_pair(uint32_t dst, const void* tmap, uint32_t bar, int c0, int c1, int c2,
                                                 int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, "
      "{%3, %4, %5, %6}], [%2];" ::"r"(dst),
      "l"(tmap), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

// The same loads with an L2 eviction-priority hint.  The 64-bit policy words are the fixed encodings
// of createpolicy.fractional.L2::evict_* with fraction 1.0.
constexpr uint64_t L2_EVICT_NORMAL = 0x1000000000000000ull;
constexpr uint64_t L2_EVICT_FIRST = 0x12F0000000000000ull;
constexpr uint64_t L2_EVICT_LAST = 0x14F0000000000000ull;

__device__ __forceinline__ void tma_load_2d_hint(uint32_t dst, const void* tmap, uint32_t bar, int c0, int c1, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, "
      "{%3, %4}], [%2], %5;" ::"r"(dst),
      "l"(tmap), "r"(bar), "r"(c0), "r"(c1), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d_hint(uint32_t dst, const void* tmap, uint32_t bar, int c0, int c1, int c2,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, "
      "{%3, %4, %5}], [%2], %6;" ::"r"(dst),
      "l"(tmap), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair_hint(uint32_t dst, const void* tmap, uint32_t bar, int c0, int c1,
                                                      uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, "
      "{%3, %4}], [%2], %5;" ::"r"(dst),
      "l"(tmap), "r"(bar), "r"(c0), "r"(c1), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair_hint(uint32_t dst, const void* tmap, uint32_t bar, int c0, int c1, int c2,
                                                      uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, "
      "{%3, %4, %5}], [%2], %6;" ::"r"(dst),
      "l"(tmap), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "l"(policy)
      : "memory");
}

// Untiled bulk copy global -> shared (16-byte aligned addresses, size multiple of 16).
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes,
                                          uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(dst),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}

__device__ __forceinline__ void tensormap_fence_acquire(const void* tmap) {
  asm volatile("fence.proxy.tensormap::generic.acquire.gpu [%0], 128;" ::"l"(tmap) : "memory");
}

// request the 128-byte line at `ptr` into L2
__device__ __forceinline__ void prefetch_l2(const void* ptr) { asm volatile("prefetch.global.L2 [%0];" ::"l"(ptr)); }
__device__ __forceinline__ void prefetch_tensormap(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// ---------------------------------------------------------------------------------------
// tcgen05 (5th-generation tensor cores, TMEM)
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Arrive on an mbarrier of this CTA once every tcgen05 operation issued so far by this
// thread has completed.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar)
               : "memory");
}

// ---- CTA-pair (cta_group::2) variants -----------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `addr` (a shared::cta address of this CTA) in the CTA of rank `rank`
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
// Arrive on a barrier of any CTA of the cluster.  Relaxed on purpose: a release at cluster scope
// first waits for every earlier global store of the thread (the previous tile's output), which
// cost the epilogue about 1.9k cycles per tile.  The arrival only has to follow the thread's own
// TMEM loads, and tcgen05.wait::ld plus tcgen05.fence::before_thread_sync order those.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Releasing arrive on a barrier of any CTA of the cluster (orders this thread's earlier writes,
// remote shared-memory stores included, before the arrival).
__device__ __forceinline__ void mbar_arrive_cluster_release(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// 32-bit store into the shared memory of any CTA of the cluster
__device__ __forceinline__ void st_shared_cluster(uint32_t cluster_addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
// 0, computed from `v` in a way the compiler cannot fold: adding it to an address makes the
// instruction that uses the address wait for the load that produced `v`.
__device__ __forceinline__ uint32_t zero_after(int v) {
  uint32_t z;
  asm volatile("and.b32 %0, %1, 0;" : "=r"(z) : "r"(v));
  return z;
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// Arrive, once every tcgen05 operation issued so far by this thread has completed, on the mbarrier
// at this shared-memory offset in each CTA of the pair named by `cta_mask`.
__device__ __forceinline__ void tc_commit_pair(uint32_t bar, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
      "h"(cta_mask)
      : "memory");
}
__device__ __forceinline__ void mma_mxf8_ss_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                 uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t"
      "}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
      : "memory");
}
__device__ __forceinline__ void tmem_cp_sf_pair(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

// Shared-memory matrix descriptor (sm_100 format, version 1).
//   bits [0,14)  start address >> 4      bits [16,30) leading byte offset >> 4
//   bits [32,46) stride byte offset >> 4 bits [46,48) version = 1
//   bits [61,64) swizzle mode: 0 none, 2 = 128-byte, 4 = 64-byte, 6 = 32-byte
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes,
                                                   uint32_t sbo_bytes, uint32_t swizzle) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)swizzle << 61;
  return d;
}

// Instruction descriptor of tcgen05.mma.kind::mxf8f6f4.block_scale, E4M3 x E4M3 (K-major
// both), E8M0 scales, f32 accumulate.
//   [4,6) B scale id  [7,10) A format (0 = E4M3)  [10,13) B format  [15] A major  [16] B major
//   [17,23) N >> 3    [23] scale format (1 = E8M0) [24,29) M >> 4   [29,31) A scale id
__host__ __device__ constexpr uint32_t make_idesc_mxf8(int m, int n) {
  return ((uint32_t)(n >> 3) << 17) | (1u << 23) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ uint32_t idesc_with_sf_id(uint32_t idesc, uint32_t a_id, uint32_t b_id) {
  return idesc | (a_id << 29) | (b_id << 4);
}

__device__ __forceinline__ void mma_mxf8_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                            uint32_t idesc, uint32_t tmem_sfa, uint32_t tmem_sfb,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t"
      "}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
      : "memory");
}

// Block-scaled MMA of any of the three operand formats, one CTA or a CTA pair.
//   kFmt 0  kind::mxf8f6f4, 8-bit operands, K = 32, one scale per row and MMA (scale id = byte of the TMEM word)
//   kFmt 1  kind::mxf4, packed E2M1 operands, K = 64, two E8M0 scales per row and MMA (scale id 0 or 2)
//   kFmt 2  kind::mxf4nvf4, packed E2M1 operands, K = 64, four scales (E8M0 or UE4M3) per row and MMA
// Every form consumes 32 bytes of K per operand row.
template <int kFmt, bool kPair>
__device__ __forceinline__ void mma_block_scaled(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t tmem_sfa,
                                                 uint32_t tmem_sfb, uint32_t accumulate) {
#define B200_MMA_ASM(GROUP, KIND)                                                                               \
  asm volatile(                                                                                                 \
      "{\n\t"                                                                                                   \
      ".reg .pred p;\n\t"                                                                                       \
      "setp.ne.b32 p, %4, 0;\n\t"                                                                               \
      "tcgen05.mma.cta_group::" GROUP ".kind::" KIND " [%0], %1, %2, %3, [%5], [%6], p;\n\t"                    \
      "}" ::"r"(tmem_d),                                                                                        \
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)                         \
      : "memory")
  if constexpr (kFmt == 0) {
    if constexpr (kPair) B200_MMA_ASM("2", "mxf8f6f4.block_scale");
    else B200_MMA_ASM("1", "mxf8f6f4.block_scale");
  } else if constexpr (kFmt == 1) {
    if constexpr (kPair) B200_MMA_ASM("2", "mxf4.block_scale.scale_vec::2X");
    else B200_MMA_ASM("1", "mxf4.block_scale.scale_vec::2X");
  } else {
    if constexpr (kPair) B200_MMA_ASM("2", "mxf4nvf4.block_scale.scale_vec::4X");
    else B200_MMA_ASM("1", "mxf4nvf4.block_scale.scale_vec::4X");
  }
#undef B200_MMA_ASM
}

template <bool kPair>
__device__ __forceinline__ void tmem_cp_sf_any(uint32_t taddr, uint64_t sdesc) {
  if constexpr (kPair) asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
  else asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

// Copy 32 rows x 16 bytes of shared memory into TMEM columns [taddr, taddr+4), replicated
// into the four 32-lane quarters (the scale-factor operand format of block-scaled MMA).
__device__ __forceinline__ void tmem_cp_sf(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc)
               : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns -> 32 registers per thread (thread = lane).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, float* v) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

// Compiler-level fence on 32 registers: makes every later use of v[] depend on this point, so
// arithmetic on the results of an asynchronous tcgen05.ld cannot be scheduled above the
// tcgen05.wait::ld that precedes this call.
__device__ __forceinline__ void reg_fence32(float* v) {
  asm volatile(""
               : "+f"(v[0]), "+f"(v[1]), "+f"(v[2]), "+f"(v[3]), "+f"(v[4]), "+f"(v[5]), "+f"(v[6]), "+f"(v[7]),
                 "+f"(v[8]), "+f"(v[9]), "+f"(v[10]), "+f"(v[11]), "+f"(v[12]), "+f"(v[13]), "+f"(v[14]),
                 "+f"(v[15]), "+f"(v[16]), "+f"(v[17]), "+f"(v[18]), "+f"(v[19]), "+f"(v[20]), "+f"(v[21]),
                 "+f"(v[22]), "+f"(v[23]), "+f"(v[24]), "+f"(v[25]), "+f"(v[26]), "+f"(v[27]), "+f"(v[28]),
                 "+f"(v[29]), "+f"(v[30]), "+f"(v[31])::"memory");
}

// ---------------------------------------------------------------------------------------
// Number formats and fast math (the reference kernel's arithmetic,
// python/cudnn/grouped_gemm/utils.py:157-309, grouped_gemm_swiglu_quant.py:1067-1188)
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ float rcp_approx(float x) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ float ex2_approx(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ float fmin_nan(float a, float b) {
  float r;
  asm("min.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
// max |x| over the 32 lanes of the warp
__device__ __forceinline__ float warp_absmax(float x) {
  float r;
  asm volatile("redux.sync.max.abs.NaN.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(x));
  return r;
}

// the same, ignoring NaN inputs (fmaxf semantics)
__device__ __forceinline__ float warp_absmax_number(float x) {
  float r;
  asm volatile("redux.sync.max.abs.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(x));
  return r;
}

// float32 loads / stores at a shared-memory address (the .shared window, as smem_u32 returns it)
__device__ __forceinline__ void st_shared_f32(uint32_t addr, float v) { asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory"); }
__device__ __forceinline__ void st_shared_f32x4(uint32_t addr, float4 v) {
  asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
__device__ __forceinline__ float ld_shared_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ float4 ld_shared_f32x4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
  return v;
}

// float32 (>= 0) -> E8M0 byte: round up to a power of two, saturate to finite.
__device__ __forceinline__ uint32_t e8m0_from_float(float x) {
  uint16_t out;
  asm("cvt.rp.satfinite.ue8m0x2.f32 %0, 0f00000000, %1;" : "=h"(out) : "f"(x));
  return (uint32_t)(out & 0xFF);
}
// E8M0 byte -> float32 (2^(b-127); byte 0 = 2^-127 as a float32 denormal)
__device__ __forceinline__ float e8m0_to_float(uint32_t b) {
  return __uint_as_float(b == 0 ? 0x00400000u : (b << 23));
}
// two float32 -> packed E4M3 pair (lo in bits 0-7, hi in bits 8-15), RNE, saturating
__device__ __forceinline__ uint32_t e4m3x2_from_float(float lo, float hi) {
  uint16_t out;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(out) : "f"(hi), "f"(lo));
  return (uint32_t)out;
}
__device__ __forceinline__ uint32_t e4m3x4_from_float(float a, float b, float c, float d) {
  return e4m3x2_from_float(a, b) | (e4m3x2_from_float(c, d) << 16);
}
__device__ __forceinline__ uint32_t bf16x2_from_float(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// two float32 -> packed E5M2 pair, RNE, saturating
__device__ __forceinline__ uint32_t e5m2x2_from_float(float lo, float hi) {
  uint16_t out;
  asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(out) : "f"(hi), "f"(lo));
  return (uint32_t)out;
}
// four float32 -> four FP8 bytes in the output's format (warp-uniform choice)
__device__ __forceinline__ uint32_t fp8x4_from_float(float a, float b, float c, float d, bool e5m2) {
  return e5m2 ? (e5m2x2_from_float(a, b) | (e5m2x2_from_float(c, d) << 16)) : e4m3x4_from_float(a, b, c, d);
}
// one FP8 byte (E4M3 or E5M2) -> float32, exact
__device__ __forceinline__ float fp8_to_float(uint8_t b, bool e5m2) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw(b, e5m2 ? __NV_E5M2 : __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}
// two float32 -> packed 16-bit pair, bf16 or fp16 (warp-uniform choice)
__device__ __forceinline__ uint32_t pack16x2_from_float(float lo, float hi, bool f16) {
  if (f16) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  return bf16x2_from_float(lo, hi);
}

// Packed float32 arithmetic of sm_100: two products / sums / fused multiply-adds per instruction, each lane
// rounded to nearest even exactly like the scalar instruction, so results do not change.
__device__ __forceinline__ float2 mul2(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float2 mul2(float2 a, float b) { return __fmul2_rn(a, make_float2(b, b)); }
__device__ __forceinline__ float2 add2(float2 a, float2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ float2 add2(float2 a, float b) { return __fadd2_rn(a, make_float2(b, b)); }
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
// v[0..n) *= s, two at a time (n even)
template <int N>
__device__ __forceinline__ void scale_inplace(float* v, float s) {
  const float2 ss = make_float2(s, s);
#pragma unroll
  for (int j = 0; j < N; j += 2) {
    const float2 r = __fmul2_rn(make_float2(v[j], v[j + 1]), ss);
    v[j] = r.x;
    v[j + 1] = r.y;
  }
}

// Scale applied to a block before the E4M3 conversion: norm / sf, clamped to FLT_MAX.
__device__ __forceinline__ float quant_scale(float norm_const, float sf_value) {
  return fmin_nan(norm_const * rcp_approx(sf_value), 3.40282346638528859812e38f);
}

// Byte offset of the scale of row `mn`, K block `kb` in the "128x4" layout
// (32 x 4 x rest_mn x 4 x rest_k; test/python/fe_api/test_fe_api_utils.py:95-114).
__host__ __device__ __forceinline__ int64_t sf_offset(int64_t mn, int64_t kb, int64_t rest_k) {
  return (mn % 32) * 16 + ((mn / 32) % 4) * 4 + (kb % 4) + (kb / 4) * 512 +
         (mn / 128) * rest_k * 512;
}

}  // namespace b200moe
