// Inline-PTX wrappers for sm_100a: mbarrier, TMA (cp.async.bulk[.tensor]),
// tcgen05 {alloc, cp, mma block_scale, commit, ld, fence} and the 64-bit shared
// memory / 32-bit instruction descriptors the block-scaled MMA consumes.
//
// Everything the reference obtains from the CuTe DSL (MmaMXF4NVF4Op,
// Cp4x32x128bOp, Ld32x32bOp, PipelineTmaUmma: dual_gemm/submission.py:147-164,
// 375-378, 566-569, 672-678) is spelled out here by hand.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

// ---------------------------------------------------------------------------
// Generic helpers
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Warpgroup-wide register reallocation (all 128 threads of warps 4i..4i+3 execute it).
template <uint32_t kRegs> __device__ __forceinline__ void warpgroup_reg_inc() {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegs));
}
template <uint32_t kRegs> __device__ __forceinline__ void warpgroup_reg_dec() {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegs));
}

__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(pred));
    return pred != 0;
}

// ---------------------------------------------------------------------------
// Programmatic dependent launch: a kernel launched with the programmatic-stream-serialization
// attribute may start while the kernel before it in the stream is still running.
// ---------------------------------------------------------------------------
// Let the next kernel in the stream be scheduled as soon as every CTA of this grid has said so (or
// exited): its CTAs then start on SMs as this grid's CTAs leave them, instead of after the whole grid.
__device__ __forceinline__ void griddep_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
// Wait until the kernels this one depends on have completed and their writes are visible.  Returns at
// once when the launch carried no programmatic dependency.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// Make generic-proxy writes to shared memory visible to the async proxy (TMA,
// tcgen05) and vice versa.
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

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// try_wait that lets the hardware park the thread for up to `hint_ns` before it
// reports "not yet": far fewer barrier accesses than a tight polling loop.
__device__ __forceinline__ bool mbar_try_wait_parked(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(hint_ns)
        : "memory");
    return ok != 0;
}

// Bounded wait: gives up after about a second (kWaitTimeoutCycles SM clocks),
// ORs `code` into *status, raises the CTA-wide abort flag and returns false.
// Never traps, never spins forever.  The deadline is kept with clock64(), which
// costs a few cycles; %globaltimer is far slower to read and would sit on the
// wake-up path of every wait that does not succeed at once.
constexpr long long kWaitTimeoutCycles = 2000ll * 1000ll * 1000ll;

// What the fault-injection self-test waits instead: about a millisecond.
constexpr long long kShortWaitTimeoutCycles = 2ll * 1000ll * 1000ll;

template <bool kParked = false, long long kLimit = kWaitTimeoutCycles>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                          uint32_t* status, uint32_t code) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
#pragma unroll 1
    while (true) {
#pragma unroll 1
        for (int i = 0; i < 256; ++i)
            if (kParked ? mbar_try_wait_parked(bar, parity, 20000u) : mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > kLimit) {
            *abort_flag = 1u;
            atomicOr(status, code);
            return false;
        }
    }
}

// 3-D tiled store shared memory -> global (whole box; the bytes must have been made
// visible to the async proxy with fence_proxy_async_smem).  Joins the thread's
// current bulk group.
__device__ __forceinline__ void tma_store_3d(const void* map, uint32_t smem_src, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(map)), "r"(smem_src), "r"(c0), "r"(c1), "r"(c2)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// All of this thread's bulk groups have finished *reading* shared memory.
__device__ __forceinline__ void bulk_wait_group_read_all() {
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
// All but the newest of this thread's bulk groups have finished reading shared memory.
__device__ __forceinline__ void bulk_wait_group_read_1() {
    asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
}
// All of this thread's bulk groups are complete (their global writes performed).
__device__ __forceinline__ void bulk_wait_group_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// ---------------------------------------------------------------------------
// Thread-block clusters (CTA pairs)
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Address of this CTA's shared-memory location `addr` as seen in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
// Arrive on an mbarrier that lives in any CTA of the cluster (address from map_to_cta).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Same without release ordering: for hand-overs whose data went to tensor memory
// (ordered by tcgen05.wait / tcgen05.fence), where nothing in ordinary memory is
// published by the arrival.  A cluster-scope release otherwise waits for every
// earlier write of the thread to become visible to the partner SM.
__device__ __forceinline__ void mbar_arrive_cluster_relaxed(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_arrive() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// try_wait that also acquires arrivals made by the other CTA of the pair.
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_try_wait_cluster_parked(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(hint_ns)
        : "memory");
    return ok != 0;
}
template <bool kParked = false>
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                                  uint32_t* status, uint32_t code) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    const long long t0 = clock64();
#pragma unroll 1
    while (true) {
#pragma unroll 1
        for (int i = 0; i < 256; ++i)
            if (kParked ? mbar_try_wait_cluster_parked(bar, parity, 20000u) : mbar_try_wait_cluster(bar, parity))
                return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > kWaitTimeoutCycles) {
            *abort_flag = 1u;
            atomicOr(status, code);
            return false;
        }
    }
}

// Warp-wide bounded wait: lane 0 polls, the outcome is broadcast.  Every polling
// lane is a separate access to the barrier, and barrier traffic from waiting
// warps slows down the (single) thread that issues the MMAs on the same SM.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, int lane, volatile uint32_t* abort_flag,
                                               uint32_t* status, uint32_t code) {
    uint32_t ok = 1;
    if (lane == 0) ok = mbar_wait<true>(bar, parity, abort_flag, status, code) ? 1u : 0u;
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

// ---------------------------------------------------------------------------
// TMA
// ---------------------------------------------------------------------------
__device__ __forceinline__ void prefetch_tensormap(const void* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// Acquire a tensor map that lives in global memory before the TMA unit reads it.
__device__ __forceinline__ void tensormap_acquire(const void* map) {
    asm volatile("fence.proxy.tensormap::generic.acquire.gpu [%0], 128;" ::"l"(
                     reinterpret_cast<uint64_t>(map))
                 : "memory");
}

// 3-D tiled load, completion counted in bytes on `bar`.  c0 is the innermost
// coordinate (bytes here: always a multiple of 16).
__device__ __forceinline__ void tma_load_3d(uint32_t smem_dst, const void* map, uint32_t bar, int c0,
                                            int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

// Warp-collective forms of the producer's instructions: every lane of a converged warp executes
// the call with the same arguments and one elected lane issues.  Inside an `if (lane == 0)`
// branch each of these costs the issuing thread 100-150 cycles (five per k-tile made the producer
// the slowest role: ~750 cycles per k-tile); predicated on elect.sync in warp-uniform code the
// operands stay in uniform registers.
__device__ __forceinline__ void mbar_arrive_expect_tx_elect(uint32_t bar, uint32_t bytes) {
    asm volatile(
        "{\n\t"
        ".reg .pred e;\n\t"
        "elect.sync _|e, 0xffffffff;\n\t"
        "@e mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n\t"
        "}\n" ::"r"(bar), "r"(bytes)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d_elect(uint32_t smem_dst, const void* map, uint32_t bar, int c0, int c1,
                                                  int c2) {
    asm volatile(
        "{\n\t"
        ".reg .pred e;\n\t"
        "elect.sync _|e, 0xffffffff;\n\t"
        "@e cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5}], [%2];\n\t"
        "}\n" ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
__device__ __forceinline__ void bulk_load_elect(uint32_t smem_dst, const void* gsrc, uint32_t bytes, uint32_t bar) {
    asm volatile(
        "{\n\t"
        ".reg .pred e;\n\t"
        "elect.sync _|e, 0xffffffff;\n\t"
        "@e cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n\t"
        "}\n" ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(bar)
        : "memory");
}

// Untiled bulk copy global -> shared (16-byte aligned, size multiple of 16).
__device__ __forceinline__ void bulk_load(uint32_t smem_dst, const void* gsrc, uint32_t bytes,
                                          uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(bar)
        : "memory");
}

// ---------------------------------------------------------------------------
// tcgen05: tensor memory management
// ---------------------------------------------------------------------------
// Whole warp.  Writes the allocated base address to *smem_slot.
__device__ __forceinline__ void tmem_alloc(uint32_t smem_slot, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_slot),
                 "r"(columns)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(columns)
                 : "memory");
}

// CTA-pair variants: a warp with the same index in both CTAs executes alloc / dealloc.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_slot, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_slot),
                 "r"(columns)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t base, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(columns)
                 : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---------------------------------------------------------------------------
// Descriptors
// ---------------------------------------------------------------------------
// Shared-memory matrix descriptor, K-major operand stored as 128-byte rows with
// the 128-byte swizzle (what a TMA box of 128 bytes x rows with
// CU_TENSOR_MAP_SWIZZLE_128B writes): 8-row groups are 1024 bytes apart.
//   [0,14)  start address >> 4      [16,30) leading byte offset >> 4 (1: unused)
//   [32,46) stride byte offset >> 4 [46,48) version = 1 (sm_100)
//   [61,64) layout: 2 = SWIZZLE_128B, 0 = none
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_addr) {
    return static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4) | (1ull << 16) |
           (static_cast<uint64_t>(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

// Descriptor for a 512-byte scale-factor atom (32 rows x 16 bytes, no swizzle,
// 8-row core matrices 128 bytes apart) as the source of tcgen05.cp.32x128b.
__device__ __forceinline__ uint64_t smem_desc_sf(uint32_t smem_addr) {
    return static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4) |
           (static_cast<uint64_t>(128 >> 4) << 32) | (1ull << 46);
}

// Instruction descriptor, kind::mxf4nvf4 block-scaled, dense, K-major A and B:
//   [7,10) A format (1 = e2m1)   [10,13) B format (1 = e2m1)
//   [17,23) N >> 3               [23] scale format (0 = ue4m3)
//   [24,29) M >> 4               [4,6)/[29,31) scale-factor ids (0)   [31] K = 64
__host__ __device__ constexpr uint32_t idesc_mxf4nvf4(int m, int n) {
    return (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
           (static_cast<uint32_t>(m >> 4) << 24);
}

// ---------------------------------------------------------------------------
// tcgen05: copy, MMA, commit, load
// ---------------------------------------------------------------------------
// 32 rows x 128 bit from shared memory into 4 TMEM columns, replicated to the
// four 32-lane quadrants.  One thread issues.
__device__ __forceinline__ void tc_cp_32x128b_warpx4(uint32_t tmem_col, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_col), "l"(sdesc)
                 : "memory");
}

// D[tmem] (+)= A[smem] * B[smem] with per-16-element ue4m3 scale factors read
// from TMEM.  One thread issues.  K = 64 e2m1 elements.
__device__ __forceinline__ void tc_mma_mxf4nvf4(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                                uint32_t idesc, uint32_t tmem_sfa, uint32_t tmem_sfb,
                                                uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t"
        "}\n"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(tmem_sfa),
        "r"(tmem_sfb)
        : "memory");
}

// Same MMA, operands given as the low words of their SWIZZLE_128B descriptors (the
// high word is the same constant for every operand tile): keeps the issuing
// thread's dependent instruction chain short.
constexpr uint32_t kDescHiSw128 = (1024u >> 4) | (1u << 14) | (2u << 29);   // SBO, version, layout
__device__ __forceinline__ uint32_t smem_desc_lo(uint32_t smem_addr) {
    return ((smem_addr & 0x3FFFFu) >> 4) | (1u << 16);                       // start address, LBO = 1
}
__device__ __forceinline__ void tc_mma_mxf4nvf4_lo(uint32_t tmem_d, uint32_t adesc_lo, uint32_t bdesc_lo,
                                                   uint32_t idesc, uint32_t tmem_sfa, uint32_t tmem_sfb,
                                                   uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        ".reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %7};\n\t"
        "mov.b64 db, {%2, %7};\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], da, db, %3, [%5], [%6], p;\n\t"
        "}\n"
        ::"r"(tmem_d), "r"(adesc_lo), "r"(bdesc_lo), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb),
        "r"(kDescHiSw128)
        : "memory");
}

// The same MMA across a CTA pair (M = 256: each CTA contributes its 128 rows of A
// and its half of B's rows from the same shared-memory offsets, and receives its
// 128 rows of D in its own TMEM).  Issued by one thread of the pair's first CTA.
__device__ __forceinline__ void tc_mma_mxf4nvf4_pair_lo(uint32_t tmem_d, uint32_t adesc_lo, uint32_t bdesc_lo,
                                                        uint32_t idesc, uint32_t tmem_sfa, uint32_t tmem_sfb,
                                                        uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        ".reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %7};\n\t"
        "mov.b64 db, {%2, %7};\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.block16 [%0], da, db, %3, [%5], [%6], p;\n\t"
        "}\n"
        ::"r"(tmem_d), "r"(adesc_lo), "r"(bdesc_lo), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb),
        "r"(kDescHiSw128)
        : "memory");
}
// Warp-collective forms: every lane of a converged warp executes the call with the
// same arguments and one elected lane issues the instruction.  With the operands
// computed in warp-uniform code the issuing cost per MMA is about half of what the
// same instruction costs inside an `if (lane == 0)` branch (measured 39 vs 70 cycles).
__device__ __forceinline__ void tc_mma_mxf4nvf4_pair_lo_elect(uint32_t tmem_d, uint32_t adesc_lo, uint32_t bdesc_lo,
                                                              uint32_t idesc, uint32_t tmem_sfa, uint32_t tmem_sfb,
                                                              uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p, e;\n\t"
        ".reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %7};\n\t"
        "mov.b64 db, {%2, %7};\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "elect.sync _|e, 0xffffffff;\n\t"
        "@e tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.block16 [%0], da, db, %3, [%5], [%6], p;\n\t"
        "}\n"
        ::"r"(tmem_d), "r"(adesc_lo), "r"(bdesc_lo), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb),
        "r"(kDescHiSw128)
        : "memory");
}
// tcgen05.commit tracks the MMAs issued by the executing thread: elect.sync picks the
// same lane every time for a full mask, so the committing lane is the issuing lane.
__device__ __forceinline__ void tc_commit_pair_both_elect(uint32_t bar, uint16_t cta_mask) {
    asm volatile(
        "{\n\t"
        ".reg .pred e;\n\t"
        "elect.sync _|e, 0xffffffff;\n\t"
        "@e tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n\t"
        "}\n"
        ::"r"(bar), "h"(cta_mask)
        : "memory");
}
__device__ __forceinline__ void tc_commit_pair_elect(uint32_t cluster_bar) {
    asm volatile(
        "{\n\t"
        ".reg .pred e;\n\t"
        "elect.sync _|e, 0xffffffff;\n\t"
        "@e tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t"
        "}\n"
        ::"r"(cluster_bar)
        : "memory");
}
// Arrive on an mbarrier (cluster address: this CTA's or the partner's) once every
// MMA the pair has been given so far by this thread is done.
__device__ __forceinline__ void tc_commit_pair(uint32_t cluster_bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar)
                 : "memory");
}

// One commit that arrives on the barrier at the same shared-memory offset in every
// CTA of `cta_mask` (bit i = cluster rank i).
__device__ __forceinline__ void tc_commit_pair_both(uint32_t bar, uint16_t cta_mask) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
        ::"r"(bar), "h"(cta_mask)
        : "memory");
}

// mbarrier arrive once every tcgen05 op issued so far by this thread is done.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}

// TMEM -> registers: lane i of the warp gets 16 consecutive 32-bit columns of
// TMEM lane (taddr.lane + i).  The warp may only touch its own lane quadrant.
__device__ __forceinline__ void tc_ld_x16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
          "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
          "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}
// Same, 64 consecutive columns in one instruction (v points at 64 registers).
__device__ __forceinline__ void tc_ld_x64(uint32_t taddr, uint32_t* v) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31]), "=r"(v[32]), "=r"(v[33]), "=r"(v[34]), "=r"(v[35]), "=r"(v[36]), "=r"(v[37]), "=r"(v[38]), "=r"(v[39]), "=r"(v[40]), "=r"(v[41]), "=r"(v[42]), "=r"(v[43]), "=r"(v[44]), "=r"(v[45]), "=r"(v[46]), "=r"(v[47]), "=r"(v[48]), "=r"(v[49]), "=r"(v[50]), "=r"(v[51]), "=r"(v[52]), "=r"(v[53]), "=r"(v[54]), "=r"(v[55]), "=r"(v[56]), "=r"(v[57]), "=r"(v[58]), "=r"(v[59]), "=r"(v[60]), "=r"(v[61]), "=r"(v[62]), "=r"(v[63])
        : "r"(taddr)
        : "memory");
}
// Registers -> TMEM: lane i of the warp writes 4 consecutive 32-bit columns of
// TMEM lane (taddr.lane + i).  The warp may only touch its own lane quadrant.
__device__ __forceinline__ void tc_st_x4(uint32_t taddr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(a), "r"(b),
                 "r"(c), "r"(d)
                 : "memory");
}
__device__ __forceinline__ void tc_st_x8(uint32_t taddr, const uint32_t* v) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr),
                 "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
                 : "memory");
}
__device__ __forceinline__ void tc_st_x16(uint32_t taddr, const uint32_t* v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
        "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
        "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
        : "memory");
}
__device__ __forceinline__ void tc_wait_st() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void ld_shared_v4(uint32_t addr, uint32_t& a, uint32_t& b, uint32_t& c, uint32_t& d) {
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "r"(addr)
                 : "memory");
}
__device__ __forceinline__ void ld_shared_v2(uint32_t addr, uint32_t& a, uint32_t& b) {
    asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];" : "=r"(a), "=r"(b) : "r"(addr) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void st_global_v4(void* p, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.global.v4.b32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(a), "r"(b), "r"(c), "r"(d)
                 : "memory");
}

__device__ __forceinline__ void st_global_v4f(float* p, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.global.v4.b32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
// Load that bypasses L1 (data written by another SM during this launch).
__device__ __forceinline__ float4 ld_global_cg_v4f(const float* p) {
    float4 v;
    asm volatile("ld.global.cg.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p)
                 : "memory");
    return v;
}
__device__ __forceinline__ void st_release_gpu_u32(uint32_t* p, uint32_t v) {
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_gpu_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// Barrier among the 128 epilogue threads only (hardware barrier 1; barrier 0 is __syncthreads).
__device__ __forceinline__ void epilogue_bar_sync() {
    asm volatile("bar.sync 1, 128;" ::: "memory");
}

// Barrier among the nine warps of the pair kernel that use tensor memory (all but the producer warp;
// hardware barrier 2).
__device__ __forceinline__ void consumer_bar_sync() {
    asm volatile("bar.sync 2, 288;" ::: "memory");
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);  // round to nearest, overflow -> inf
    return *reinterpret_cast<uint32_t*>(&h);
}

// silu(x) * y with silu(x) = x / (1 + exp(-x)); x -> -inf gives -0 (never NaN).
__device__ __forceinline__ float silu_mul(float x, float y) {
    return __fdividef(x, 1.0f + __expf(-x)) * y;
}

}  // namespace b200
