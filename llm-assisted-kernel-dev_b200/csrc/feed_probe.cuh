// Measurement aid: how fast can TMA fill shared memory from L2?  The GEMM kernels take 38 KB per
// k-tile and CTA from L2; this kernel does nothing but such loads, so that the rate the memory
// system sustains can be put beside the rate the GEMMs draw.
//
// Every CTA keeps twelve 16 KiB slots in flight from a window that fits L2.  Four warps issue (one
// lane each, three slots each): one thread manages a wait + expect_tx + copy only every few hundred
// cycles, so a single issuer would measure itself.  `share` consecutive CTAs read the same sequence
// of tiles at about the same time, the way the CTAs of a GEMM wave share operand tiles.
#pragma once

#include "ptx_sm100.cuh"

namespace b200 {

constexpr int kFeedSlotBytes = 16384;   // one operand tile: 128 rows x 128 bytes
constexpr int kFeedSlots = 12;
constexpr int kFeedIssuers = 4;
constexpr int kFeedThreads = 32 * kFeedIssuers;
constexpr uint32_t kStatusFeedProbe = 0x100;

struct FeedProbe {
    CUtensorMap map;             // window as [rows][row_bytes] bytes, box 128 x 128, 128-byte swizzle
    const uint8_t* window;
    int rows, row_bytes;
    int copies_per_issuer;
    int share;                   // CTAs that read the same tiles (>= 1)
    int tiled;                   // 1: cp.async.bulk.tensor boxes, 0: contiguous cp.async.bulk copies
    unsigned long long* cycles;  // per CTA: clock64 span of its loop
    uint32_t* status;
};

__global__ void __launch_bounds__(kFeedThreads, 1) l2_feed_probe(const __grid_constant__ FeedProbe p) {
    extern __shared__ uint8_t feed_smem[];
    __shared__ uint64_t full[kFeedSlots];
    __shared__ uint32_t abort_word;
    const uint32_t base = (smem_u32(feed_smem) + 1023u) & ~1023u;
    if (threadIdx.x == 0) {
        for (int i = 0; i < kFeedSlots; ++i) mbar_init(smem_u32(&full[i]), 1);
        abort_word = 0;
        fence_mbar_init();
        fence_proxy_async_smem();
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5;
    const long long t0 = clock64();
    if ((threadIdx.x & 31) == 0) {
        volatile uint32_t* abort_flag = &abort_word;
        constexpr int kMine = kFeedSlots / kFeedIssuers;   // slots warp, warp + 4, warp + 8
        const int row_tiles = p.rows / 128, k_chunks = p.row_bytes / 128;
        const unsigned tiles = static_cast<unsigned>(row_tiles) * static_cast<unsigned>(k_chunks);
        const unsigned first = (blockIdx.x / static_cast<unsigned>(p.share)) * 131u;
        bool ok = true;
        // copy i of this issuer reuses slot (i % kMine): wait for the copy that filled it last
        for (int i = 0; ok && i < p.copies_per_issuer + kMine; ++i) {
            const int s = warp + (i % kMine) * kFeedIssuers;
            const int use = i / kMine;
            const uint32_t bar = smem_u32(&full[s]);
            if (use > 0) ok = mbar_wait<false>(bar, static_cast<uint32_t>(use - 1) & 1u, abort_flag, p.status, kStatusFeedProbe);
            if (!ok || i >= p.copies_per_issuer) continue;   // the last kMine turns only drain
            const unsigned g = (first + (static_cast<unsigned>(i) * kFeedIssuers + warp) * 17u) % tiles;
            mbar_arrive_expect_tx(bar, kFeedSlotBytes);
            if (p.tiled)
                tma_load_3d(base + s * kFeedSlotBytes, &p.map, bar, static_cast<int>(g / row_tiles) * 128,
                            static_cast<int>(g % row_tiles) * 128, 0);
            else
                bulk_load(base + s * kFeedSlotBytes, p.window + static_cast<size_t>(g) * kFeedSlotBytes, kFeedSlotBytes, bar);
        }
        if (!ok)
            for (int i = 0; i < 64; ++i) __nanosleep(2000);   // a wait ran out: let copies in flight land before the CTA ends
    }
    __syncthreads();
    if (threadIdx.x == 0) p.cycles[blockIdx.x] = static_cast<unsigned long long>(clock64() - t0);
}

}  // namespace b200
