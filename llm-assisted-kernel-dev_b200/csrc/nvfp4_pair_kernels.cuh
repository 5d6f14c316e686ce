// GEMMs on CTA pairs (tcgen05 cta_group::2): two CTAs on the two SMs of a TPC share
// one 256-row output tile.  Dual GEMM: 256 x 128 outputs of C = silu(A.B1^T) * (A.B2^T)
// (merged B = the B1 tile in the first CTA, the B2 tile in the second).  Grouped GEMM:
// 256 x 256 outputs of one group's C = A.B^T (merged B = 256 consecutive rows of B, 128
// in each CTA); rows past the group's M are zero-filled by TMA and never stored.
//
// Why: in the one-CTA kernel a 128x256x64 MMA reads 12 KB of operands from shared
// memory (A 4 KB + merged B 8 KB) every 130 cycles, the TMA fills add 54 KB per
// k-tile and the scale-factor warps read another 24 KB: about 126 KB per k-tile on
// a 128 B/clk shared memory is ~1000 cycles, twice the 520 the four MMAs need.  In
// a pair each CTA holds its own 128 rows of A and *half* of the merged B (CTA 0 the
// B1 tile, CTA 1 the B2 tile): per CTA the MMAs read 32 KB per k-tile, the TMA
// fills 38 KB, the scale-factor warps 24 KB.
//
// Division of labour (same ten warps per CTA as the one-CTA kernel):
//   producer          each CTA loads its own A tile, its B tile, its SFA chunk and
//                     both SFB chunks; signals its own `full` barrier
//   scale factors     each CTA's four warps fill their own TMEM (SFA of the CTA's
//                     rows, SFB of all 256 merged-B rows); they arrive on the
//                     *first* CTA's hand-over barrier (eight arrivals per k-tile)
//   MMA               one thread of the first CTA issues every MMA for the pair;
//                     it commits to both CTAs' `empty` and `acc_full` barriers
//   epilogue          each CTA drains its own 128 accumulator rows; both hand the
//                     buffer back on the first CTA's `acc_release` barrier
// No load carries a cluster-multicast qualifier; the partner is only ever signalled
// through mbarrier arrivals.
#pragma once

#include "nvfp4_gemm_kernels.cuh"
#include "nvfp4_quantize.cuh"

namespace b200 {

// One pipeline stage of a CTA: its 128 rows of A, its kBRows rows of the merged B and the three
// 2 KiB scale-factor chunks (SFA of its rows, SFB of both CTAs' B rows).
template <int kBRows> struct PairStageT {
    static constexpr uint32_t kOffA = 0;
    static constexpr uint32_t kOffB = kOperandTileBytes;                 // this CTA's half of merged B
    static constexpr uint32_t kOffSfA = kOperandTileBytes + kBRows * 128u;
    static constexpr uint32_t kOffSfB1 = kOffSfA + kSfChunkBytes;
    static constexpr uint32_t kOffSfB2 = kOffSfB1 + kSfChunkBytes;
    static constexpr uint32_t kBytes = kOffSfB2 + kSfChunkBytes;        // 38 KiB (128 rows) / 30 KiB (64 rows)
    static_assert(kBytes % 1024 == 0, "stages keep the 1024-byte alignment of the swizzle atoms");
};
constexpr uint32_t kPairStagingBytes = 4u * 8192u;   // per epilogue warp: two boxes of 32 rows x 128 bytes
template <typename S> constexpr uint32_t pair_smem_bytes() {
    return 1024u + S::kStages * PairStageT<S::kBRows>::kBytes + kPairStagingBytes + sizeof(ControlBlock);
}
constexpr uint32_t kStatusPairWait = 0x80;

// Stream-k scratch of one pair: the fp32 accumulator of a 256 x 256 pair tile, laid out
// [CTA rank][warp][4-column group][lane][4 floats] so that a warp's stores and loads are 512
// contiguous bytes, and eight flag words (one per writing warp) per pair.
constexpr size_t kStreamKSlotFloats = 2u * 4u * 64u * 32u * 4u;            // 65536 floats = 256 KiB
constexpr size_t kStreamKFlagWords = 8;

// One piece of work of a pair: k-tiles [kt_begin, kt_begin + kt_count) of pair tile `tile`.
//   kind 0  the whole k range: ordinary epilogue
//   kind 1  the tail of the k range (first piece of this pair's stream-k range): the fp32
//           accumulator goes to the pair's scratch slot, nothing is stored to C
//   kind 2  the head of the k range (last piece of the range): the next pair's slot is added
//           to the accumulator before the epilogue
struct PairPiece {
    int tile, kt_begin, kt_count, kind;
};

// Scheduling policies: work of one CTA (cluster rank) of the pair for pair tile `tile`.
//   kBRows   rows of the merged B that each CTA holds (the MMA's N is 2 * kBRows)
//   kStages  pipeline depth that fits the shared memory beside the staging area
//   TM       tensor-memory map (accumulator buffers, scale-factor ring)
struct PairDual {
    using Params = DenseProblem;
    using TM = TmemMap<Mode::Dual>;           // 256 accumulator columns per buffer, buffers overlap
    static constexpr const char* kName = "nvfp4_gemm_pair<PairDual>";
    static constexpr bool kGrouped = false;
    static constexpr bool kQuantOut = false;
    static constexpr bool kStreamK = false;
    static constexpr bool kGather = false;
    static constexpr int kBRows = 128;
    static constexpr int kMmaN = 256;
    static constexpr int kStages = 5;
    __device__ static int total(const Params& p) { return (p.m_tiles / 2) * p.n_tiles * p.batches; }
    __device__ static int k_tiles(const Params& p, int /*tile*/, int& /*cursor*/) { return p.k_tiles; }
    __device__ static int sfb_half(const Params& /*p*/, int /*tile*/) { return 0; }
    // rows of A/C are those of the CTA's rank, the B tile is B1 for rank 0 and B2 for rank 1
    __device__ static Work get(const Params& p, int tile, uint32_t rank, int& /*cursor*/) {
        const int m_pairs = p.m_tiles / 2;
        const int m_pair = tile % m_pairs;
        const int t = tile / m_pairs;
        const int n_blk = t % p.n_tiles;
        const int b = t / p.n_tiles;
        const int m_blk = 2 * m_pair + static_cast<int>(rank);
        Work w;
        w.map_a = &p.map_a;
        w.map_blo = rank == 0 ? static_cast<const void*>(&p.map_b1) : static_cast<const void*>(&p.map_b2);
        w.map_bhi = w.map_blo;
        w.a_row = m_blk * kTileM;
        w.blo_row = w.bhi_row = n_blk * 128;
        w.batch = b;
        const long long sf_row = static_cast<long long>(p.sf_k_atoms) * kSfAtomBytes;
        w.sfa = p.sfa + b * p.sfa_batch + m_blk * sf_row;
        w.sfblo = p.sfb1 + b * p.sfb_batch + n_blk * sf_row;
        w.sfbhi = p.sfb2 + b * p.sfb_batch + n_blk * sf_row;
        w.ldc = p.ldc;
        w.c = p.c + b * p.c_batch + static_cast<long long>(m_blk) * kTileM * p.ldc + n_blk * 128;
        w.rows_valid = kTileM;
        w.cols_valid = 128;
        w.k_tile_begin = 0;
        w.k_tile_count = p.k_tiles;
        w.group = 0;
        w.tile = tile;
        w.split = 0;
        return w;
    }
};

// The same tiles with a stream-k tail (DenseProblem::sk_tiles > 0): a kernel of its own so that
// the partial-sum code does not weigh on the registers of the plain one.
struct PairDualStreamK : PairDual {
    static constexpr const char* kName = "nvfp4_gemm_pair<PairDualStreamK>";
    static constexpr bool kStreamK = true;
};

// Column shard of a dual GEMM whose epilogue stores every tile into the full C of every rank of the
// node (its own and, over NVLink, the peers'): GEMM and all-gather of the shards in one kernel.
struct PairDualGather : PairDual {
    static constexpr const char* kName = "nvfp4_gemm_pair<PairDualGather>";
    static constexpr bool kGather = true;
};

// Dual GEMM whose epilogue re-quantises its fp16 result to NVFP4 (packed e2m1 + e4m3
// scale factors in the reordered layout), ready to be the A operand of the next GEMM.
struct PairDualQuant : PairDual {
    static constexpr const char* kName = "nvfp4_gemm_pair<PairDualQuant>";
    static constexpr bool kQuantOut = true;
};

// Dual GEMM on 256 x 64 output tiles for shapes with few tiles (the reference task's
// benchmark shapes have 48-128 tiles of 128 x 128 for 148 SMs): each CTA holds 64 rows of
// B1 (rank 0) or of B2 (rank 1), the MMA is 256 x 128 x 64, accumulator columns [0,64) =
// A.B1^T and [64,128) = A.B2^T.  Twice as many pair tiles as PairDual, 30 KiB instead of
// 38 KiB of loads and 24 KiB instead of 32 KiB of MMA operand reads per k-tile and CTA.
// The scale factors of 64 B rows are half of a 128-row atom: the whole atom is loaded and
// the scale-factor warps pick the two 32-row groups of their tile (`sfb_half`).
struct PairDualNarrow {
    using Params = DenseProblem;
    using TM = TmemMap<Mode::Group128>;       // two disjoint 128-column accumulators
    static constexpr const char* kName = "nvfp4_gemm_pair<PairDualNarrow>";
    static constexpr bool kGrouped = false;
    static constexpr bool kQuantOut = false;
    static constexpr bool kStreamK = false;
    static constexpr int kBRows = 64;
    static constexpr int kMmaN = 128;
#ifdef B200_NARROW_STAGES
    static constexpr int kStages = B200_NARROW_STAGES;
#else
    static constexpr int kStages = 6;
#endif
    __device__ static int total(const Params& p) { return (p.m_tiles / 2) * p.n_tiles * 2 * p.batches; }
    __device__ static int k_tiles(const Params& p, int /*tile*/, int& /*cursor*/) { return p.k_tiles; }
    __device__ static int n_blk64(const Params& p, int tile) { return (tile / (p.m_tiles / 2)) % (p.n_tiles * 2); }
    __device__ static int sfb_half(const Params& p, int tile) { return n_blk64(p, tile) & 1; }
    __device__ static Work get(const Params& p, int tile, uint32_t rank, int& /*cursor*/) {
        const int m_pairs = p.m_tiles / 2;
        const int m_pair = tile % m_pairs;
        const int t = tile / m_pairs;
        const int n64 = t % (p.n_tiles * 2);
        const int b = t / (p.n_tiles * 2);
        const int m_blk = 2 * m_pair + static_cast<int>(rank);
        Work w;
        w.map_a = &p.map_a;
        w.map_blo = rank == 0 ? static_cast<const void*>(&p.map_b1n) : static_cast<const void*>(&p.map_b2n);
        w.map_bhi = w.map_blo;
        w.a_row = m_blk * kTileM;
        w.blo_row = w.bhi_row = n64 * 64;
        w.batch = b;
        const long long sf_row = static_cast<long long>(p.sf_k_atoms) * kSfAtomBytes;
        w.sfa = p.sfa + b * p.sfa_batch + m_blk * sf_row;
        w.sfblo = p.sfb1 + b * p.sfb_batch + (n64 >> 1) * sf_row;
        w.sfbhi = p.sfb2 + b * p.sfb_batch + (n64 >> 1) * sf_row;
        w.ldc = p.ldc;
        w.c = p.c + b * p.c_batch + static_cast<long long>(m_blk) * kTileM * p.ldc + n64 * 64;
        w.rows_valid = kTileM;
        w.cols_valid = 64;
        w.k_tile_begin = 0;
        w.k_tile_count = p.k_tiles;
        w.group = 0;
        w.tile = tile;
        w.split = 0;
        return w;
    }
};

// Grouped: the host fills GroupEntry::m_tiles with the number of 256-row pair tiles
// and n_tiles with n / 256; tiles are walked m-fastest inside a group like in the
// one-CTA kernel, `cursor` remembers the group of the previous tile.
struct PairGrouped {
    using Params = GroupedProblem;
    using TM = TmemMap<Mode::Group256>;
    static constexpr const char* kName = "nvfp4_gemm_pair<PairGrouped>";
    static constexpr bool kGrouped = true;
    static constexpr bool kStoreByTma = true;     // C leaves through GroupEntry::map_c, which clips rows past the group's M
    static constexpr bool kQuantOut = false;
    static constexpr bool kStreamK = false;
    static constexpr int kBRows = 128;
    static constexpr int kMmaN = 256;
    static constexpr int kStages = 5;
    __device__ static int total(const Params& p) { return p.total_tiles_dev ? *p.total_tiles_dev : p.total_tiles; }
    __device__ static int sfb_half(const Params& /*p*/, int /*tile*/) { return 0; }
    __device__ static const GroupEntry* find(const Params& p, int tile, int& cursor) {
        int g = cursor;
        const GroupEntry* e = p.groups + g;
        while (g + 1 < p.num_groups && tile >= e->tile_begin + e->m_tiles * e->n_tiles) {
            ++g;
            ++e;
        }
        cursor = g;
        return e;
    }
    __device__ static int k_tiles(const Params& p, int tile, int& cursor) { return find(p, tile, cursor)->k_tiles; }
    __device__ static Work get(const Params& p, int tile, uint32_t rank, int& cursor) {
        const GroupEntry* e = find(p, tile, cursor);
        const int local = tile - e->tile_begin;
        const int m_pair = local % e->m_tiles;
        const int n_blk = local / e->m_tiles;              // 256 columns
        const int m_blk = 2 * m_pair + static_cast<int>(rank);
        Work w;
        w.map_a = &e->map_a;
        w.map_blo = w.map_bhi = &e->map_b;
        w.a_row = e->a_row0 + m_blk * kTileM;              // may lie past the group's rows (zeros, or another group's)
        w.blo_row = w.bhi_row = n_blk * 256 + static_cast<int>(rank) * 128;
        w.batch = 0;
        const long long sf_row = static_cast<long long>(e->sf_k_atoms) * kSfAtomBytes;
        const int sfa_blocks = (e->m + kTileM - 1) / kTileM;   // the buffer is padded to whole 128-row blocks
        w.sfa = e->sfa + (m_blk < sfa_blocks ? m_blk : 0) * sf_row;
        w.sfblo = e->sfb + (2 * n_blk) * sf_row;
        w.sfbhi = e->sfb + (2 * n_blk + 1) * sf_row;
        w.ldc = e->ldc;
        w.c = e->c + static_cast<long long>(m_blk) * kTileM * e->ldc + n_blk * 256;
        w.map_c = &e->map_c;
        const int left = e->m - m_blk * kTileM;
        w.rows_valid = left < 0 ? 0 : (left > kTileM ? kTileM : left);
        w.cols_valid = 256;
        w.k_tile_begin = 0;
        w.k_tile_count = e->k_tiles;
        w.group = cursor;
        w.tile = tile;
        w.split = 0;
        return w;
    }
};

// Groups whose C tiles live in one shared buffer (the MoE layer's y): rows of a tile past a group's count
// belong to the next group, so the epilogue stores row by row, predicated, instead of by TMA.
struct PairGroupedShared : PairGrouped {
    static constexpr const char* kName = "nvfp4_gemm_pair<PairGroupedShared>";
    static constexpr bool kStoreByTma = false;
};

// The sequence of pieces of one pair, the same in every role of both CTAs.  Whole tiles are
// dealt round-robin (tile = pair, pair + pairs, ...).  With a stream-k tail (PairDual,
// sk_tiles > 0) only the first total - sk_tiles tiles are dealt that way (a whole number of
// rounds); the k-tiles of the last sk_tiles tiles form one line of sk_tiles * k_tiles units
// that is cut into `pairs` equal ranges, so every pair gets the same amount of work to the
// k-tile.  A range is at least one tile long (the host guarantees sk_tiles >= pairs), so a
// tile is shared by at most two neighbouring pairs: pair i runs its head (k-tiles from 0) at the
// end of its range, pair i + 1 its tail at the start of its own.  The tail's accumulator goes
// through pair i + 1's scratch slot, long before pair i asks for it.
template <typename S> struct PairWalk {
    int pairs, dp_tiles, next_dp, k_tiles;
    long long u, u_end;
    __device__ PairWalk(const typename S::Params& p, int pair, int pairs_) : pairs(pairs_), k_tiles(1), u(0), u_end(0) {
        const int total = S::total(p);
        dp_tiles = total;
        next_dp = pair;
        if constexpr (S::kStreamK) {
            if (p.sk_tiles > 0) {
                dp_tiles = total - p.sk_tiles;
                k_tiles = p.k_tiles;
                const long long units = static_cast<long long>(p.sk_tiles) * p.k_tiles;
                u = units * pair / pairs;
                u_end = units * (pair + 1) / pairs;
            }
        }
    }
    __device__ bool next(const typename S::Params& p, int& cursor, PairPiece& out) {
        if (next_dp < dp_tiles) {
            out.tile = next_dp;
            out.kt_begin = 0;
            out.kt_count = S::k_tiles(p, next_dp, cursor);
            out.kind = 0;
            next_dp += pairs;
            return true;
        }
        if constexpr (S::kStreamK) {
            if (u < u_end) {
                const int t = static_cast<int>(u / k_tiles);
                const int kt0 = static_cast<int>(u - static_cast<long long>(t) * k_tiles);
                const long long left = u_end - u;
                const int cnt = (k_tiles - kt0) < left ? (k_tiles - kt0) : static_cast<int>(left);
                out.tile = dp_tiles + t;
                out.kt_begin = kt0;
                out.kt_count = cnt;
                out.kind = kt0 > 0 ? 1 : (cnt < k_tiles ? 2 : 0);
                u += cnt;
                return true;
            }
        }
        return false;
    }
};

// Grouped epilogue of one warp: 32 rows x 256 columns of fp16, no activation.  The
// accumulator columns shared with the other buffer are fetched first and the buffer is
// handed back; then 64 columns at a time go through a 4 KB staging box (128-byte-swizzle
// layout) so that the global stores are whole 128-byte lines: one instruction writes
// four rows x 128 bytes instead of 32 rows x 16 bytes.  Rows past the group's M are
// predicated off.
template <int kBuf>
__device__ __forceinline__ void epilogue_tile_grouped_pair(const Work& w, uint32_t tmem_base, int quad, int lane,
                                                           uint32_t release_bar, uint32_t staging, bool store) {
    using TM = TmemMap<Mode::Group256>;
    constexpr int kEarly = TM::kEarlyChunks;
    constexpr int kSharedRel = (kBuf == 0) ? TM::kSharedBegin : 0;
    const uint32_t acc = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + kBuf * TM::kAccStride;
    uint32_t early[kEarly][16];
    static_assert(kEarly == 9, "the shared columns are fetched as 64 + 64 + 16");
    tc_ld_x64(acc + kSharedRel, &early[0][0]);
    tc_ld_x64(acc + kSharedRel + 64, &early[4][0]);
    tc_ld_x16(acc + kSharedRel + 128, early[8]);
    tc_wait_ld();
    tc_fence_before_sync();
    __syncwarp();
    if (lane == 0) mbar_arrive_cluster_relaxed(release_bar);   // barrier of the pair's first CTA
    const int rows_here = w.rows_valid - quad * 32;            // rows of this warp that exist
    const uint32_t wr_base = staging + lane * 128;
    const uint32_t swz = static_cast<uint32_t>(lane & 7);
    __half* out = w.c + static_cast<long long>(quad * 32) * w.ldc;
#pragma unroll
    for (int chunk = 0; chunk < 16; ++chunk) {
        const int col = chunk * 16;
        const bool is_early = col >= kSharedRel && col < kSharedRel + kEarly * 16;
        uint32_t x[16];
        if (!is_early) {
            tc_ld_x16(acc + col, x);
            tc_wait_ld();
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) x[i] = early[(col - kSharedRel) / 16][i];
        }
        uint32_t packed[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) packed[i] = pack_half2(__uint_as_float(x[2 * i]), __uint_as_float(x[2 * i + 1]));
        const uint32_t u0 = static_cast<uint32_t>((chunk & 3) * 2);
        st_shared_v4(wr_base + ((u0 ^ swz) << 4), packed[0], packed[1], packed[2], packed[3]);
        st_shared_v4(wr_base + (((u0 + 1) ^ swz) << 4), packed[4], packed[5], packed[6], packed[7]);
        if ((chunk & 3) == 3) {
            __syncwarp();
            // lane l: 16-byte unit l % 8 of rows 4j + l / 8
            const int unit = lane & 7;
            __half* dst = out + (chunk >> 2) * 64 + unit * 8;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int r = 4 * j + (lane >> 3);
                uint32_t a, b, c, d;
                ld_shared_v4(staging + r * 128 + ((static_cast<uint32_t>(unit) ^ static_cast<uint32_t>(r & 7)) << 4), a, b,
                             c, d);
                if (store && r < rows_here) st_global_v4(dst + static_cast<long long>(r) * w.ldc, a, b, c, d);
            }
            __syncwarp();
        }
    }
}

// The same tile leaving through TMA stores (policies with kStoreByTma): each 64-column slice of the warp's 32 rows is
// converted into one of the warp's two 4 KB staging boxes and handed to the TMA unit, which clips the rows past the
// group's M (the store map's extent) by itself.  No shared-memory read-back and no global store instruction runs on
// the SM's load/store path, which the scale-factor warps and the MMAs' operand reads share with this epilogue.
template <int kBuf>
__device__ __forceinline__ void epilogue_tile_grouped_pair_tma(const Work& w, uint32_t tmem_base, int quad, int lane,
                                                               uint32_t release_bar, uint32_t staging, int c_col, int c_row,
                                                               bool store) {
    using TM = TmemMap<Mode::Group256>;
    constexpr int kEarly = TM::kEarlyChunks;
    constexpr int kSharedRel = (kBuf == 0) ? TM::kSharedBegin : 0;
    const uint32_t acc = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + kBuf * TM::kAccStride;
    uint32_t early[kEarly][16];
    static_assert(kEarly == 9, "the shared columns are fetched as 64 + 64 + 16");
    tc_ld_x64(acc + kSharedRel, &early[0][0]);
    tc_ld_x64(acc + kSharedRel + 64, &early[4][0]);
    tc_ld_x16(acc + kSharedRel + 128, early[8]);
    tc_wait_ld();
    tc_fence_before_sync();
    __syncwarp();
    if (lane == 0) mbar_arrive_cluster_relaxed(release_bar);   // barrier of the pair's first CTA
    const bool rows_exist = w.rows_valid - quad * 32 > 0;       // else every row of this warp lies past the group's M
    const uint32_t row_base = staging + lane * 128;
    const uint32_t swz = static_cast<uint32_t>(lane & 7);
#pragma unroll
    for (int chunk = 0; chunk < 16; ++chunk) {
        const int col = chunk * 16;
        const bool is_early = col >= kSharedRel && col < kSharedRel + kEarly * 16;
        uint32_t x[16];
        if (!is_early) {
            tc_ld_x16(acc + col, x);
            tc_wait_ld();
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) x[i] = early[(col - kSharedRel) / 16][i];
        }
        if ((chunk & 3) == 0) {
            // the box about to be rewritten was handed to the TMA unit two slices ago (or by the previous tile)
            if (lane == 0) bulk_wait_group_read_1();
            __syncwarp();
        }
        uint32_t packed[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) packed[i] = pack_half2(__uint_as_float(x[2 * i]), __uint_as_float(x[2 * i + 1]));
        const uint32_t box = row_base + static_cast<uint32_t>((chunk >> 2) & 1) * 4096u;
        const uint32_t u0 = static_cast<uint32_t>((chunk & 3) * 2);
        st_shared_v4(box + ((u0 ^ swz) << 4), packed[0], packed[1], packed[2], packed[3]);
        st_shared_v4(box + (((u0 + 1) ^ swz) << 4), packed[4], packed[5], packed[6], packed[7]);
        if ((chunk & 3) == 3) {
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                if (store && rows_exist)
                    tma_store_3d(w.map_c, staging + static_cast<uint32_t>((chunk >> 2) & 1) * 4096u, c_col + (chunk >> 2) * 64,
                                 c_row, 0);
                bulk_commit_group();      // an empty group keeps the count of groups per tile at four
            }
        }
    }
}

// Epilogue of the quantised-output dual GEMM for one warp (32 rows x 128 columns): the
// fp16 value the plain kernel would store, silu(x) * y rounded to fp16, is quantised the
// way nvfp4_quantize does it.  A lane holds one row and a 16-column chunk is exactly one
// scale-factor block, so nothing crosses lanes: eight packed bytes per chunk go straight
// to global memory and four chunks' scale bytes make one word of the reordered layout.
// The result equals quantising the plain kernel's C byte for byte.
template <int kBuf>
__device__ __forceinline__ void epilogue_tile_quant(const DenseProblem& p, const Work& w, uint32_t tmem_base,
                                                    int quad, int lane, uint32_t release_bar, int m_blk, int n_blk,
                                                    bool store) {
    using TM = TmemMap<Mode::Dual>;
    constexpr int kEarly = TM::kEarlyChunks;
    constexpr int kSharedRel = (kBuf == 0) ? TM::kSharedBegin : 0;
    const uint32_t acc = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + kBuf * TM::kAccStride;
    uint32_t early[kEarly][16];
    static_assert(kEarly == 9, "the shared columns are fetched as 64 + 64 + 16");
    tc_ld_x64(acc + kSharedRel, &early[0][0]);
    tc_ld_x64(acc + kSharedRel + 64, &early[4][0]);
    tc_ld_x16(acc + kSharedRel + 128, early[8]);
    tc_wait_ld();
    tc_fence_before_sync();
    __syncwarp();
    if (lane == 0) mbar_arrive_cluster_relaxed(release_bar);   // barrier of the pair's first CTA
    const int n_total = p.n_tiles * 128;
    const long long row = static_cast<long long>(m_blk) * kTileM + quad * 32 + lane;
    uint8_t* q_row = p.q_out + row * (n_total / 2) + n_blk * 64;
    // scale factors of this row, columns n_blk*128 ...: k-blocks n_blk*8 + chunk of the (m, n/16) scale matrix
    uint8_t* sf_row = p.sf_out + (static_cast<long long>(m_blk) * (n_total / 64) + n_blk * 2) * 512 + lane * 16 + quad * 4;
    uint32_t sf_word = 0;
    uint2 held = make_uint2(0u, 0u);
#pragma unroll
    for (int chunk = 0; chunk < 8; ++chunk) {
        const int xcol = chunk * 16;
        const int ycol = 128 + chunk * 16;
        const bool x_early = xcol >= kSharedRel && xcol < kSharedRel + kEarly * 16;
        const bool y_early = ycol >= kSharedRel && ycol < kSharedRel + kEarly * 16;
        uint32_t x[16], y[16];
        if (!x_early) tc_ld_x16(acc + xcol, x);
        if (!y_early) tc_ld_x16(acc + ycol, y);
        if (!x_early || !y_early) tc_wait_ld();
        if (x_early) {
#pragma unroll
            for (int i = 0; i < 16; ++i) x[i] = early[(xcol - kSharedRel) / 16][i];
        }
        if (y_early) {
#pragma unroll
            for (int i = 0; i < 16; ++i) y[i] = early[(ycol - kSharedRel) / 16][i];
        }
        uint32_t h[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
            h[i] = pack_half2(silu_mul(__uint_as_float(x[2 * i]), __uint_as_float(y[2 * i])),
                              silu_mul(__uint_as_float(x[2 * i + 1]), __uint_as_float(y[2 * i + 1])));
        uint2 packed;
        const uint32_t sbyte = quantize_block<kQuantDtypeF16>(make_uint4(h[0], h[1], h[2], h[3]),
                                                              make_uint4(h[4], h[5], h[6], h[7]), packed);
        sf_word |= sbyte << (8 * (chunk & 3));
        // four chunks = 64 columns = 32 packed bytes of the row: one whole 32-byte sector, written with two 16-byte
        // stores instead of four 8-byte ones
        if ((chunk & 1) == 0) {
            held = packed;
        } else if (store) {
            st_global_v4(q_row + (chunk - 1) * 8, held.x, held.y, packed.x, packed.y);
        }
        if ((chunk & 3) == 3) {
            if (store) *reinterpret_cast<uint32_t*>(sf_row + (chunk >> 2) * 512) = sf_word;
            sf_word = 0;
        }
    }
}

// Narrow dual tile (PairDualNarrow), one warp: 32 rows x 64 output columns.  Accumulator
// columns [0,64) = x, [64,128) = y; the fp16 results go through one swizzled 4 KiB box of the
// warp's staging area and leave with one TMA store.
template <int kBuf>
__device__ __forceinline__ void epilogue_tile_narrow(const DenseProblem& p, const Work& w, uint32_t tmem_base, int quad,
                                                     int lane, uint32_t staging, int c_col, int c_row, bool store) {
    using TM = TmemMap<Mode::Group128>;
    const uint32_t acc = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + kBuf * TM::kAccStride;
    if (lane == 0) bulk_wait_group_read_all();      // the previous tile's box has left the staging area
    __syncwarp();
    const uint32_t row_base = staging + lane * 128;
    const uint32_t swz = static_cast<uint32_t>(lane & 7);
#pragma unroll
    for (int chunk = 0; chunk < 4; ++chunk) {
        uint32_t x[16], y[16];
        tc_ld_x16(acc + chunk * 16, x);
        tc_ld_x16(acc + 64 + chunk * 16, y);
        tc_wait_ld();
        uint32_t packed[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
            packed[i] = pack_half2(silu_mul(__uint_as_float(x[2 * i]), __uint_as_float(y[2 * i])),
                                   silu_mul(__uint_as_float(x[2 * i + 1]), __uint_as_float(y[2 * i + 1])));
        const uint32_t u0 = static_cast<uint32_t>(chunk * 2);
        st_shared_v4(row_base + ((u0 ^ swz) << 4), packed[0], packed[1], packed[2], packed[3]);
        st_shared_v4(row_base + (((u0 + 1) ^ swz) << 4), packed[4], packed[5], packed[6], packed[7]);
    }
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0 && store) {
        tma_store_3d(&p.map_c, staging, c_col, c_row, w.batch);
        bulk_commit_group();
    }
}

// Stream-k, tail piece: this warp's 32 rows x 256 accumulator columns go to the pair's scratch
// slot as fp32; nothing is stored to C.  The columns shared with the other accumulator buffer
// are read first and the buffer is handed back before the rest is copied.
template <int kBuf>
__device__ __forceinline__ void epilogue_partial_store(const DenseProblem& p, uint32_t tmem_base, uint32_t rank,
                                                       int quad, int lane, uint32_t release_bar, int slot) {
    using TM = TmemMap<Mode::Dual>;
    const uint32_t acc = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + kBuf * TM::kAccStride;
    float* dst = p.splitk_ws + static_cast<size_t>(slot) * kStreamKSlotFloats +
                 static_cast<size_t>(rank * 4 + quad) * (64 * 128) + lane * 4;
    // buffer 0 shares its columns [112,256), buffer 1 its columns [0,144)
    constexpr int kFirst = (kBuf == 0) ? 112 : 0;
#pragma unroll 1
    for (int i = 0; i < 16; ++i) {
        const int col = (kFirst + i * 16) & 255;
        uint32_t v[16];
        tc_ld_x16(acc + col, v);
        tc_wait_ld();
        if (i == 8) {                              // the 144 shared columns are in registers or memory
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster_relaxed(release_bar);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j)
            st_global_v4f(dst + static_cast<size_t>(col / 4 + j) * 128, v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    }
    __threadfence();
    __syncwarp();
    if (lane == 0)
        st_release_gpu_u32(p.splitk_flags + static_cast<size_t>(slot) * kStreamKFlagWords + rank * 4 + quad,
                           p.splitk_epoch);
}

// Stream-k, head piece: wait (bounded) until the warp with the same rows in the pair that ran the
// tail of this tile has published its partial sums.
__device__ __forceinline__ bool wait_partial(const DenseProblem& p, int slot, uint32_t rank, int quad,
                                             volatile uint32_t* abort_flag) {
    const uint32_t* flag = p.splitk_flags + static_cast<size_t>(slot) * kStreamKFlagWords + rank * 4 + quad;
    bool ok = true;
    if (ld_acquire_gpu_u32(flag) != p.splitk_epoch) {
        const long long t0 = clock64();
        while (ld_acquire_gpu_u32(flag) != p.splitk_epoch) {
            if (*abort_flag || clock64() - t0 > kWaitTimeoutCycles) {
                *abort_flag = 1u;
                atomicOr(p.status, kStatusSplitKWait);
                ok = false;
                break;
            }
            __nanosleep(200);
        }
    }
    return __all_sync(0xffffffffu, ok);
}

constexpr int kPairThreads = 352;   // eleven warps: 0-3 epilogue, 4 MMA, 5 operand loads, 6-9 scale factors, 10 scale-factor loads

template <typename S, bool kTimingProbes = false>
__global__ void __launch_bounds__(kPairThreads, 1)
nvfp4_gemm_pair(const __grid_constant__ typename S::Params p, int flags) {
    using TM = typename S::TM;
    using Stage = PairStageT<S::kBRows>;
    constexpr int kStages = S::kStages;
    constexpr int kWordsPerBlock = TM::kSlotCols;          // scale-factor words per 64-k block and lane
    static_assert(kWordsPerBlock == 4 + S::kMmaN / 32, "scale-factor slot = SFA 4 columns + SFB N/32 columns");
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    ControlBlock* ctl = reinterpret_cast<ControlBlock*>(smem_raw + (smem_base - smem_u32(smem_raw)) +
                                                        kStages * Stage::kBytes + kPairStagingBytes);
    const uint32_t staging_base = smem_base + kStages * Stage::kBytes;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_cta_rank();          // 0: issues the MMAs, 1: partner
    const int pair = blockIdx.x >> 1;
    const int pairs = gridDim.x >> 1;
    const long long launch_t0 = clock64();
    griddep_launch_dependents();   // the next launch may move onto SMs as this grid's CTAs leave them

    if constexpr (!S::kGrouped) {
        // the descriptors the first loads need: fetched while the CTA sets itself up
        if (threadIdx.x == 160) {
            int cursor0 = 0;
            const Work w0 = S::get(p, pair, rank, cursor0);
            prefetch_tensormap(w0.map_a);
            prefetch_tensormap(w0.map_blo);
            if (!S::kQuantOut) prefetch_tensormap(&p.map_c);
        }
    }
    // Barriers: one initialising thread per stage, one for the rest.
    if (threadIdx.x < kStages) {
        const int s = threadIdx.x;
        mbar_init(smem_u32(&ctl->full[s]), 2);    // the two producer warps, each with its own byte count
        mbar_init(smem_u32(&ctl->empty[s]), 1);
        // one hand-over barrier per stage: a slot is reused only after the MMA thread
        // passed its previous use (the stage had to be freed in between); used in CTA 0
        mbar_init(smem_u32(&ctl->sf_ready[s]), 8);
        fence_mbar_init();
        fence_proxy_async_smem();
    } else if (threadIdx.x == 32) {
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&ctl->acc_full[b]), 1);
            mbar_init(smem_u32(&ctl->acc_release[b]), 8);   // four epilogue warps in each CTA (used in CTA 0)
        }
        mbar_init(smem_u32(&ctl->aux[0]), 1);
        ctl->abort_flag = 0;
        fence_mbar_init();
        fence_proxy_async_smem();
    }
    __syncthreads();       // this CTA's barriers exist
    cluster_arrive();      // every thread arrives now; who needs the partner's barriers waits below
    uint32_t tmem_base = 0;
    volatile uint32_t* abort_flag = &ctl->abort_flag;
    if (warp != 5 && warp != 10) {
        // The two producer warps need neither tensor memory nor the partner: they start loading while
        // the other nine warps allocate tensor memory and meet the partner CTA.
        if (warp == 4) {
            tmem_alloc_pair(smem_u32(&ctl->tmem_base), kTmemColumns);
            tmem_relinquish_pair();
        }
        tc_fence_before_sync();
        consumer_bar_sync();   // the tensor-memory base address is published
        tc_fence_after_sync();
        tmem_base = ctl->tmem_base;
        cluster_wait();        // the partner's barriers exist before anybody signals them
    }
    // Everything above touched only this CTA's own resources; from here on global memory is read and
    // written, which must wait for the kernels before this one in the stream.
    griddep_wait();

    if (warp >= 6 && warp <= 9) {
        // ------------------------------ scale factors: own shared memory -> own TMEM
        const uint32_t quad_lane = static_cast<uint32_t>((warp & 3) * 32) << 16;
        constexpr uint32_t kUnitsPerKTile = kKBlocks / TM::kGranule;
        constexpr int kUnitWords = TM::kGranule * kWordsPerBlock;   // 24 (N = 256) or 32 (N = 128)
        uint32_t s = 0, ph = 0, kt = 0, buf = 0, units = 0, retired = 0, rs = 0, rph = 0;
        bool ok = true;
        int cursor = 0;
        Tracer trace(kTimingProbes && lane == 0 && warp == 6 ? p.trace : nullptr, 5);
        PairWalk<S> walk(p, pair, pairs);
        PairPiece pc;
        while (ok && walk.next(p, cursor, pc)) {
            const uint32_t half_off = static_cast<uint32_t>(S::sfb_half(p, pc.tile)) * 8u;
            for (int i = 0; ok && i < pc.kt_count; ++i) {
                if (!mbar_wait<true>(smem_u32(&ctl->full[s]), ph, abort_flag, p.status, kStatusSfWait)) {
                    ok = false;
                    break;
                }
                trace(1);   // operands landed
                uint32_t v[kKBlocks * kWordsPerBlock];
                const uint32_t src = smem_base + s * Stage::kBytes + lane * 16;
                if (!(kTimingProbes && (flags & kFlagSkipBHi)))   // timing probe (bit reused): no scale-factor reads
#pragma unroll
                for (int kb = 0; kb < kKBlocks; ++kb) {
                    uint32_t* d = v + kb * kWordsPerBlock;
                    ld_shared_v4(src + Stage::kOffSfA + kb * kSfAtomBytes, d[0], d[1], d[2], d[3]);
                    if constexpr (S::kMmaN == 256) {
                        ld_shared_v4(src + Stage::kOffSfB1 + kb * kSfAtomBytes, d[4], d[5], d[6], d[7]);
                        ld_shared_v4(src + Stage::kOffSfB2 + kb * kSfAtomBytes, d[8], d[9], d[10], d[11]);
                    } else {
                        // 64 B rows per CTA: two of the atom's four 32-row groups
                        ld_shared_v2(src + Stage::kOffSfB1 + kb * kSfAtomBytes + half_off, d[4], d[5]);
                        ld_shared_v2(src + Stage::kOffSfB2 + kb * kSfAtomBytes + half_off, d[6], d[7]);
                    }
                }
                trace(4);   // scale factors in registers
                // ring units of this k-tile were last read by k-tile (units + 1 - kBuffers) / kUnitsPerKTile
                const uint32_t last_unit = units + kUnitsPerKTile - 1;
                const bool probe_skip = kTimingProbes && (flags & kFlagSkipSfCopy) && kt >= 2;   // timing probe
                if (!probe_skip && last_unit >= static_cast<uint32_t>(TM::kBuffers)) {
                    const uint32_t need = (last_unit - TM::kBuffers) / kUnitsPerKTile;
                    if (retired <= need) {
                        while (retired < need) {
                            ++retired;
                            if (++rs == kStages) { rs = 0; rph ^= 1u; }
                        }
                        // arrived on by the first CTA's tcgen05.commit
                        ok = mbar_wait<false>(smem_u32(&ctl->empty[rs]), rph, abort_flag, p.status, kStatusSfWait);
                        ++retired;
                        if (++rs == kStages) { rs = 0; rph ^= 1u; }
                        if (!ok) break;
                        tc_fence_after_sync();
                    }
                }
                trace(5);   // ring units free
                if (!probe_skip) {
#pragma unroll
                    for (int gr = 0; gr < static_cast<int>(kUnitsPerKTile); ++gr) {
                        uint32_t b = buf + gr;
                        if (b >= static_cast<uint32_t>(TM::kBuffers)) b -= TM::kBuffers;
                        const uint32_t dst = tmem_base + quad_lane + TM::sfa_col(b * TM::kGranule);
                        tc_st_x16(dst, v + gr * kUnitWords);
                        if constexpr (kUnitWords == 24) tc_st_x8(dst + 16, v + gr * kUnitWords + 16);
                        else tc_st_x16(dst + 16, v + gr * kUnitWords + 16);
                    }
                    trace(6);   // stores issued
                    tc_wait_st();
                    trace(7);   // stores complete
                }
                units += kUnitsPerKTile;
                buf += kUnitsPerKTile;
                if (buf >= static_cast<uint32_t>(TM::kBuffers)) buf -= TM::kBuffers;
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster_relaxed(map_to_cta(smem_u32(&ctl->sf_ready[s]), 0));
                trace(3);   // handed to the MMA warp
                ++kt;
                if (++s == kStages) { s = 0; ph ^= 1u; }
            }
        }
    } else if (warp == 5 || warp == 10) {
        // ------------------------------ TMA producers (each CTA for itself)
        // Two warps share a k-tile's instructions, each of which costs its issuing warp 80-100 cycles:
        // warp 5 loads the two operand tiles, warp 10 the three scale-factor chunks; each arrives on
        // the stage's barrier (count 2) with the byte count of its own copies before it issues them.
        // Whole warps run the loop in lock step on warp-uniform values; one elected lane issues.
        {
            const bool operands = warp == 5;
            uint32_t s = 0, ph = 0;
            bool ok = true;
            int cursor = 0, last_group = -1;
            Tracer trace(kTimingProbes && lane == 0 && operands ? p.trace : nullptr, 4);
            PairWalk<S> walk(p, pair, pairs);
            PairPiece pc;
            trace(10);   // producer starts
            while (ok && walk.next(p, cursor, pc)) {
                const Work w = S::get(p, pc.tile, rank, cursor);
                if (S::kGrouped && operands && w.group != last_group) {   // tensor maps of a new group, written by the host
                    tensormap_acquire(w.map_a);
                    tensormap_acquire(w.map_blo);
                    last_group = w.group;
                }
                for (int i = 0; i < pc.kt_count; ++i) {
                    if (!__all_sync(0xffffffffu, mbar_wait<true>(smem_u32(&ctl->empty[s]), ph ^ 1u, abort_flag, p.status,
                                                                 kStatusProducerWait))) {
                        ok = false;
                        break;
                    }
                    const uint32_t stage = smem_base + s * Stage::kBytes;
                    const uint32_t bar = smem_u32(&ctl->full[s]);
                    if (kTimingProbes && (flags & kFlagSkipLoads)) {   // timing probe
                        if (lane == 0) mbar_arrive(bar);
                        if (++s == kStages) { s = 0; ph ^= 1u; }
                        continue;
                    }
                    const int kt_index = pc.kt_begin + i;
                    if (operands) {
                        mbar_arrive_expect_tx_elect(bar, Stage::kOffSfA);              // A tile + B tile
                        tma_load_3d_elect(stage + Stage::kOffA, w.map_a, bar, kt_index * 128, w.a_row, w.batch);
                        tma_load_3d_elect(stage + Stage::kOffB, w.map_blo, bar, kt_index * 128, w.blo_row, w.batch);
                    } else {
                        const long long sf_off = static_cast<long long>(kt_index) * kSfChunkBytes;
                        mbar_arrive_expect_tx_elect(bar, 3 * kSfChunkBytes);
                        bulk_load_elect(stage + Stage::kOffSfA, w.sfa + sf_off, kSfChunkBytes, bar);
                        bulk_load_elect(stage + Stage::kOffSfB1, w.sfblo + sf_off, kSfChunkBytes, bar);
                        bulk_load_elect(stage + Stage::kOffSfB2, w.sfbhi + sf_off, kSfChunkBytes, bar);
                    }
                    trace(1);   // k-tile's loads issued
                    if (++s == kStages) { s = 0; ph ^= 1u; }
                }
            }
            if (!ok)
                for (int i = 0; i < 64; ++i) __nanosleep(2000);   // error path: let copies in flight land
        }
        __syncwarp();
        cluster_wait();    // completes the start-up cluster barrier this warp only arrived on
    } else if (warp == 4) {
        // ------------------------------ MMA issuer (first CTA of the pair only)
        // The whole warp runs the loop in lock step (waits included) so that descriptors and
        // addresses are warp-uniform values; one elected lane issues each MMA and commit.
        if (rank == 0) {
            constexpr uint32_t kUnitCols = TM::kGranule * TM::kSlotCols;
            const uint32_t desc_lo_base = smem_desc_lo(smem_base + Stage::kOffA);
            const uint32_t sf_ready_bar = smem_u32(&ctl->sf_ready[0]);
            const uint32_t empty_mine = smem_u32(&ctl->empty[0]);
            const uint32_t sf_base = tmem_base + TM::kSfBase;
            uint32_t s = 0, ph = 0, a_lo = desc_lo_base, buf = 0;
            int it = 0;
            bool failed = false;
            Tracer trace(kTimingProbes && lane == 0 ? p.trace : nullptr, 0);
            const long long kernel_t0 = clock64();
            int cursor = 0;
            PairWalk<S> walk(p, pair, pairs);
            PairPiece pc;
            for (; !failed && walk.next(p, cursor, pc); ++it) {
                const int k_tiles = pc.kt_count;
                trace(8);
                // the first k-tile's scale factors are normally in place long before the
                // accumulator comes back: pass that barrier first, off the hand-back path
                if (!__all_sync(0xffffffffu, mbar_wait<true>(sf_ready_bar + s * 8u, ph, abort_flag, p.status, kStatusMmaWaitFull))) {
                    failed = true;
                    break;
                }
                if (it > 0) {
                    const int r = it - 1;
                    if (!__all_sync(0xffffffffu, mbar_wait<true>(smem_u32(&ctl->acc_release[r & 1]), (r >> 1) & 1, abort_flag,
                                                           p.status, kStatusMmaWaitAcc))) {
                        failed = true;
                        break;
                    }
                }
                tc_fence_after_sync();   // orders the MMAs below after both barriers
                trace(9);   // accumulator buffer available
                const uint32_t acc_addr = tmem_base + (it & 1) * TM::kAccStride;
#pragma unroll 1
                for (int i = 0; i < k_tiles; ++i) {
                    // eight arrivals: both CTAs' scale factors are in TMEM; the arriving warps
                    // waited for their CTA's operands first
                    if (i > 0) {
                        if (!__all_sync(0xffffffffu, mbar_wait<true>(sf_ready_bar + s * 8u, ph, abort_flag, p.status, kStatusMmaWaitFull))) {
                            failed = true;
                            break;
                        }
                        tc_fence_after_sync();
                    }
                    trace(1);   // k-tile ready
                    uint32_t b = buf;
                    if (!(kTimingProbes && (flags & kFlagSkipMma) && (i & 3)))   // timing probe: MMAs of every fourth k-tile only
#pragma unroll
                    for (int kb = 0; kb < kKBlocks; ++kb) {
                        if (kb > 0 && kb % TM::kGranule == 0) b = (b + 1 == TM::kBuffers) ? 0u : b + 1;
                        const uint32_t sfa = sf_base + b * kUnitCols + (kb % TM::kGranule) * TM::kSlotCols;
                        tc_mma_mxf4nvf4_pair_lo_elect(acc_addr, a_lo + 2 * kb, a_lo + (Stage::kOffB >> 4) + 2 * kb,
                                                      idesc_mxf4nvf4(256, S::kMmaN), sfa, sfa + 4,
                                                      (kb > 0 || i > 0) ? 1u : 0u);
                    }
                    tc_commit_pair_both_elect(empty_mine + s * 8, 3);   // both CTAs' `empty` barriers
                    trace(2);   // k-tile issued
                    buf += kKBlocks / TM::kGranule;
                    if (buf >= static_cast<uint32_t>(TM::kBuffers)) buf -= TM::kBuffers;
                    ++s;
                    a_lo += Stage::kBytes >> 4;
                    if (s == kStages) { s = 0; ph ^= 1u; a_lo = desc_lo_base; }
                }
                if (failed) break;
                tc_commit_pair_both_elect(smem_u32(&ctl->acc_full[it & 1]), 3);
            }
            tc_commit_pair_elect(smem_u32(&ctl->aux[0]));
            mbar_wait<true>(smem_u32(&ctl->aux[0]), 0, abort_flag, p.status, kStatusMmaWaitAcc);
            if (kTimingProbes && lane == 0 && p.trace && blockIdx.x == 0) p.trace[8 * 1024 - 1] = static_cast<unsigned long long>(clock64() - kernel_t0);
        }
        __syncwarp();
    } else if (warp < 4) {
        // ------------------------------ epilogue (each CTA its own 128 rows)
        int it = 0, cursor = 0, epi_group = -1;
        Tracer trace(kTimingProbes && lane == 0 && blockIdx.x == 0 ? p.trace : nullptr, warp == 0 ? 7 : warp);
        Tracer* tr = kTimingProbes ? &trace : nullptr;
        PairWalk<S> walk(p, pair, pairs);
        PairPiece pc;
        for (; walk.next(p, cursor, pc); ++it) {
            const Work w = S::get(p, pc.tile, rank, cursor);
            const uint32_t release_bar = map_to_cta(smem_u32(&ctl->acc_release[it & 1]), 0);
            if constexpr (!TM::kOverlapped) {
                // disjoint buffers: hand-back number `it` says "tile it - 1 is drained"
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster_relaxed(release_bar);
            }
            if (!mbar_wait<true>(smem_u32(&ctl->acc_full[it & 1]), (it >> 1) & 1, abort_flag, p.status,
                                 kStatusEpilogueWait))
                break;
            tc_fence_after_sync();
            trace(1);   // accumulator complete
            const bool store = !(kTimingProbes && (flags & kFlagSkipStores));   // timing probe
            const uint32_t staging = staging_base + static_cast<uint32_t>(warp) * 8192u;
            if constexpr (S::kQuantOut) {
                const int m_blk = w.a_row / kTileM, n_blk = w.blo_row / 128;
                if (it & 1)
                    epilogue_tile_quant<1>(p, w, tmem_base, warp, lane, release_bar, m_blk, n_blk, store);
                else
                    epilogue_tile_quant<0>(p, w, tmem_base, warp, lane, release_bar, m_blk, n_blk, store);
            } else if constexpr (S::kGrouped) {
                if constexpr (S::kStoreByTma) {
                    if (w.group != epi_group) {       // store map of a new group, written by the host
                        if (lane == 0) tensormap_acquire(w.map_c);
                        epi_group = w.group;
                    }
                    const int c_col = w.blo_row - static_cast<int>(rank) * 128, c_row = w.a_row + warp * 32;
                    if (it & 1)
                        epilogue_tile_grouped_pair_tma<1>(w, tmem_base, warp, lane, release_bar, staging, c_col, c_row, store);
                    else
                        epilogue_tile_grouped_pair_tma<0>(w, tmem_base, warp, lane, release_bar, staging, c_col, c_row, store);
                } else {
                    if (it & 1)
                        epilogue_tile_grouped_pair<1>(w, tmem_base, warp, lane, release_bar, staging, store);
                    else
                        epilogue_tile_grouped_pair<0>(w, tmem_base, warp, lane, release_bar, staging, store);
                }
            } else if constexpr (S::kMmaN == 128) {
                const int c_col = w.blo_row, c_row = w.a_row + warp * 32;
                if (it & 1)
                    epilogue_tile_narrow<1>(p, w, tmem_base, warp, lane, staging, c_col, c_row, store);
                else
                    epilogue_tile_narrow<0>(p, w, tmem_base, warp, lane, staging, c_col, c_row, store);
            } else {
                const int c_col = w.blo_row, c_row = w.a_row + warp * 32;
                bool done = false;
                if constexpr (S::kStreamK) {
                    if (pc.kind == 1) {
                        if (it & 1) epilogue_partial_store<1>(p, tmem_base, rank, warp, lane, release_bar, pair);
                        else epilogue_partial_store<0>(p, tmem_base, rank, warp, lane, release_bar, pair);
                        done = true;
                    } else if (pc.kind == 2) {
                        // partial sums of this warp's rows, published by the next pair
                        const float* partial = p.splitk_ws + static_cast<size_t>(pair + 1) * kStreamKSlotFloats +
                                               static_cast<size_t>(rank * 4 + warp) * (64 * 128) + lane * 4;
                        if (!wait_partial(p, pair + 1, rank, warp, abort_flag)) break;
                        if (it & 1)
                            epilogue_tile_staged<1, true>(p, w, tmem_base, warp, lane, release_bar, staging, c_col,
                                                          c_row, store, tr, partial);
                        else
                            epilogue_tile_staged<0, true>(p, w, tmem_base, warp, lane, release_bar, staging, c_col,
                                                          c_row, store, tr, partial);
                        done = true;
                    }
                }
                if (done) {
                } else if (it & 1) {
                    epilogue_tile_staged<1, false, S::kGather>(p, w, tmem_base, warp, lane, release_bar, staging, c_col,
                                                               c_row, store, tr);
                } else {
                    epilogue_tile_staged<0, false, S::kGather>(p, w, tmem_base, warp, lane, release_bar, staging, c_col,
                                                               c_row, store, tr);
                }
            }
            trace(2);   // tile stored
            tc_fence_before_sync();
        }
        // the staging area must outlive the TMA unit's reads; the stores themselves are
        // complete at the latest when the grid is
        if (!S::kQuantOut && lane == 0) bulk_wait_group_read_all();
        __syncwarp();
    }
    // Nobody leaves while the partner may still signal its barriers or while MMAs
    // issued by the first CTA still run on this SM.
    tc_fence_before_sync();
    __syncthreads();
    cluster_arrive();
    cluster_wait();
    if (warp == 4) {
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, kTmemColumns);
    }
    if (blockIdx.x == 0 && threadIdx.x == 0 && p.cycles) *p.cycles = static_cast<unsigned long long>(clock64() - launch_t0);
    if (kTimingProbes && blockIdx.x == 0 && threadIdx.x == 0 && p.trace) {
        p.trace[8 * 1024 - 2] = static_cast<unsigned long long>(launch_t0);
        p.trace[8 * 1024 - 3] = static_cast<unsigned long long>(clock64());
    }
}

}  // namespace b200
