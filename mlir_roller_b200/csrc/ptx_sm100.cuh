// Thin inline-PTX wrappers for the Blackwell (sm_100a) features the GEMM family uses:
// mbarrier, TMA tiled loads, tcgen05 (TMEM allocation, MMA, commit, load), cluster helpers.
// Every wait is bounded: a wait that runs out records an error code in a global status word
// and returns false, so a broken pipeline ends the kernel instead of hanging the GPU.
#pragma once

#include <cstdint>
#include <cuda.h>  // CUtensorMap (type only; the driver entry point is fetched at run time)

namespace rb200 {

// Device-side status codes written to the plan's status word (0 = no error).
enum : uint32_t {
  kDevOk = 0,
  kDevTimeoutEmpty = 1,      // TMA producer never saw a stage released
  kDevTimeoutFull = 2,       // split/relay warps never saw a stage land
  kDevTimeoutReady = 3,      // MMA issuer never saw a stage become ready
  kDevTimeoutTmemEmpty = 4,  // MMA issuer never saw an accumulator drained
  kDevTimeoutTmemFull = 5,   // epilogue never saw an accumulator completed
  kDevTimeoutTail = 6,       // producer tail wait ran out
  kDevTimeoutFixup = 7,      // split-K fix-up wait ran out
  kDevTimeoutSlot = 8,       // a worker's scratch slot was never handed back by its reader
  kDevTimeoutPeer = 9        // a flag another GPU should have raised never arrived
};

// What a bounded wait needs: where to record a failure and how long to keep trying.
struct WaitCtx {
  uint32_t* status;   // device status word shared by the whole grid (0 = no error)
  long long limit;    // clock cycles a wait may spin before it gives up
};

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---------------------------------------------------------------- cluster helpers
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\t"
               "barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Address of the same shared-memory offset in another CTA of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t cta_rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(cta_rank));
  return r;
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Arrive on the barrier at the same offset in CTA `cta_rank` of this cluster. Default
// semantics (release, CTA scope): explicit cluster-scope release/acquire on every stage cost a
// fixed ~0.6 us per k-block on B200 and serialised the CTA-pair pipeline.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar, uint32_t cta_rank) {
  const uint32_t remote = map_to_cta(bar, cta_rank);
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(remote) : "memory");
}

template <bool kClusterScope>
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  if constexpr (kClusterScope) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
  }
  return ok != 0;
}

// Bounded wait. Returns false after recording `code` when the limit runs out, or when some
// other role of the grid has already recorded an error (so a failure drains quickly).
template <bool kClusterScope = false>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const WaitCtx& ctx,
                                          uint32_t code) {
  if (mbar_try_wait<kClusterScope>(bar, parity)) return true;
  const long long t0 = clock64();
  uint32_t spins = 0;
  while (!mbar_try_wait<kClusterScope>(bar, parity)) {
    if ((++spins & 63u) == 0) {
      if (*reinterpret_cast<volatile uint32_t*>(ctx.status) != kDevOk) return false;
      if (clock64() - t0 > ctx.limit) {
        atomicCAS(ctx.status, kDevOk, code);
        return false;
      }
    }
  }
  return true;
}

// Wait used while winding a CTA down: bounded by time alone (an error recorded elsewhere does
// not cut it short, because what it waits for -- the tensor core finishing the MMAs already
// issued -- still has to happen before shared and tensor memory may be given up). Records
// nothing.
__device__ __forceinline__ bool mbar_wait_drain(uint32_t bar, uint32_t parity, long long limit) {
  if (mbar_try_wait<false>(bar, parity)) return true;
  const long long t0 = clock64();
  uint32_t spins = 0;
  while (!mbar_try_wait<false>(bar, parity)) {
    if ((++spins & 63u) == 0 && clock64() - t0 > limit) return false;
  }
  return true;
}

// Lets bulk copies and MMAs that were in flight when a role gave up finish before the CTA
// releases its shared memory: a fixed pause, far longer than any such operation takes.
__device__ __forceinline__ void abort_grace_period() {
  const long long t0 = clock64();
  while (clock64() - t0 < 200000) __nanosleep(1000);
}

// ---------------------------------------------------------------- proxies and fences
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// Orders this thread's view of what the async proxy (the TMA unit) wrote, in any state space,
// with its generic-proxy accesses that follow.
__device__ __forceinline__ void fence_proxy_async_all() {
  asm volatile("fence.proxy.async;" ::: "memory");
}

__device__ __forceinline__ void tcgen05_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tcgen05_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---------------------------------------------------------------- TMA
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* tm) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tm)) : "memory");
}

// 2-D tiled load global -> this CTA's shared memory; completion is counted in bytes on `bar`.
// c0 is the innermost (contiguous) coordinate and must keep c0 * 4 bytes 16-byte aligned.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* tm, uint32_t bar,
                                            int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(tm)), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}

// Same load issued by one CTA of a pair: the data lands in this CTA's shared memory, the byte
// count is reported to `bar_cluster`, a shared::cluster address that may name the peer's barrier.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* tm,
                                                 uint32_t bar_cluster, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(tm)), "r"(bar_cluster), "r"(c0), "r"(c1)
      : "memory");
}

// 2-D tiled store of one box from this CTA's shared memory to global memory (which may be a
// peer GPU's memory mapped into this process: the tensor map is only ever a store destination).
// c0 is the innermost coordinate (c0 * 4 bytes 16-byte aligned); elements outside the tensor
// are not written. Completion is tracked by the issuing thread's bulk async-group.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* tm, uint32_t src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(tm)),
               "r"(src), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// Until the shared-memory source of every committed store has been read (it may be rewritten).
__device__ __forceinline__ void bulk_wait_read_all() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
// Until every committed store has been performed.
__device__ __forceinline__ void bulk_wait_all() {
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

// ---------------------------------------------------------------- programmatic dependent launch
// A launch carrying the programmatic-stream-serialization attribute may start while the
// previous kernel of its stream is still running. `grid_dependency_wait` blocks until that
// kernel has completed and its writes are visible; everything before it must touch neither
// global memory the previous kernel may write nor memory it may still read.
// `grid_launch_dependents` tells the runtime that the next kernel may be scheduled once every
// CTA of this grid has said so (or exited). Both are no-ops for an ordinary launch.
__device__ __forceinline__ void grid_dependency_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void grid_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ---------------------------------------------------------------- TMEM
template <int kCtaGroup>
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  if constexpr (kCtaGroup == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
                 "r"(ncols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  } else {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
                 "r"(ncols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
}

template <int kCtaGroup>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  if constexpr (kCtaGroup == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
  } else {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
  }
}

// 32 lanes x 32 consecutive fp32 columns: thread t of the warp receives lane (base_lane + t),
// register j holds column (base_col + j).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
        "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
        "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}

// Same, 16 columns.
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---------------------------------------------------------------- UMMA descriptors
// Shared-memory matrix descriptor (64 bit): start address, leading and stride byte offsets in
// 16-byte units, descriptor version 1 (Blackwell), swizzle layout type in the top three bits.
constexpr uint64_t kLayoutSw128 = 2;        // 16-byte chunks swizzled inside 128-byte rows
constexpr uint64_t kLayoutSw128Base32 = 1;  // 32-byte chunks swizzled inside 128-byte rows

__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr, uint32_t lbo_bytes,
                                                   uint32_t sbo_bytes, uint64_t layout) {
  return static_cast<uint64_t>((addr >> 4) & 0x3FFFu) |
         (static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16) |
         (static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46) | (layout << 61);
}

// Instruction descriptor for kind::tf32 with fp32 accumulation.
// a_major / b_major: 0 = the operand tile is contiguous along k, 1 = along m (A) or n (B).
__host__ __device__ constexpr uint32_t make_idesc_tf32(int mma_m, int mma_n, uint32_t a_major,
                                                       uint32_t b_major) {
  return (1u << 4)      // D format: f32
         | (2u << 7)    // A format: tf32
         | (2u << 10)   // B format: tf32
         | (a_major << 15) | (b_major << 16)
         | (static_cast<uint32_t>(mma_n >> 3) << 17) | (static_cast<uint32_t>(mma_m >> 4) << 24);
}

template <int kCtaGroup>
__device__ __forceinline__ void umma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                          uint32_t idesc, uint32_t accumulate) {
  if constexpr (kCtaGroup == 1) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}

// Instruction descriptor for kind::f16 with fp32 accumulation; fmt: 0 = fp16, 1 = bf16 operands.
__host__ __device__ constexpr uint32_t make_idesc_f16(int mma_m, int mma_n, uint32_t a_major,
                                                      uint32_t b_major, uint32_t fmt) {
  return (1u << 4)        // D format: f32
         | (fmt << 7)     // A format
         | (fmt << 10)    // B format
         | (a_major << 15) | (b_major << 16)
         | (static_cast<uint32_t>(mma_n >> 3) << 17) | (static_cast<uint32_t>(mma_m >> 4) << 24);
}

// One MMA over 16 k of 16-bit operands.
template <int kCtaGroup>
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                         uint32_t idesc, uint32_t accumulate) {
  if constexpr (kCtaGroup == 1) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}

// Make `bar` track completion of every MMA this thread has issued so far. With a CTA pair
// the arrival is delivered to the barrier at the same offset in both CTAs.
template <int kCtaGroup>
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  if constexpr (kCtaGroup == 1) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     bar)
                 : "memory");
  } else {
    const uint16_t mask = 0x3;
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64"
        " [%0], %1;" ::"r"(bar),
        "h"(mask)
        : "memory");
  }
}

}  // namespace rb200
