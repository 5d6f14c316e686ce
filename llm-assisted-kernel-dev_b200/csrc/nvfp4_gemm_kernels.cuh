// NVFP4 block-scaled GEMM kernels for sm_100a.
//
// One kernel body serves three "modes":
//   Dual      C = silu(A.B1^T) * (A.B2^T)   (reference kernels K1/K2:
//             dual_gemm/submission.py:45-612, dual_gemm/dual_gemm_opt_cute.py:940-2107)
//   Group128  C_g = A_g.B_g^T, 128x128 output tiles      (reference K5:
//   Group256  C_g = A_g.B_g^T, 128x256 output tiles       group_gemm/group_gemm_cute5_v2.py:713-1747)
//
// Data path per 256-wide k-tile: TMA (128-byte-swizzled boxes of packed e2m1
// bytes) + bulk copies of 2 KiB scale-factor chunks -> shared memory ring ->
// tcgen05.cp (scale factors into TMEM) -> tcgen05.mma kind::mxf4nvf4.block_scale,
// fp32 accumulator in TMEM -> tcgen05.ld -> epilogue -> st.global.
//
// In Dual mode the B1 and B2 tiles sit back to back in one stage, so a single
// N=256 MMA per 64-k block produces both products (A and its scale factors are
// staged once): accumulator columns [0,128) = A.B1^T, [128,256) = A.B2^T.
#pragma once

#include "ptx_sm100.cuh"

namespace b200 {

constexpr int kTileM = 128;
constexpr int kTileK = 256;                     // e2m1 elements per k-tile (128 bytes per row)
constexpr int kKBlocks = 4;                     // 64-element MMA k-blocks per k-tile
constexpr uint32_t kOperandTileBytes = 128 * 128;  // 128 rows x 128 bytes
constexpr uint32_t kSfChunkBytes = 2048;        // 128 rows x 16 scale factors (4 atoms of 512 B)
constexpr uint32_t kSfAtomBytes = 512;
constexpr uint32_t kTmemColumns = 512;

// Status bits ORed into the status word when a bounded wait gives up.
constexpr uint32_t kStatusProducerWait = 0x1;
constexpr uint32_t kStatusMmaWaitFull = 0x2;
constexpr uint32_t kStatusMmaWaitAcc = 0x4;
constexpr uint32_t kStatusEpilogueWait = 0x8;
constexpr uint32_t kStatusSerialWait = 0x10;
constexpr uint32_t kStatusSplitKWait = 0x20;
constexpr uint32_t kStatusSfWait = 0x40;

enum class Mode { Dual, Group128, Group256 };

// Bits of the kernels' `flags` argument.  Bit 0 selects two N=128 MMAs per
// k-block instead of one N=256 MMA.  The others switch parts of the data path
// off for timing experiments (results are then wrong by design); they are only
// honoured by kernels instantiated with kTimingProbes = true.
constexpr int kFlagTwoMma = 1;
constexpr int kFlagSkipSfCopy = 2;     // scale factors copied to TMEM only for a tile's first k-tile
constexpr int kFlagSkipMma = 4;        // only the first k-block of every k-tile is multiplied
constexpr int kFlagSkipBHi = 8;        // second B tile (and its scale factors) not loaded
constexpr int kFlagSkipStores = 16;    // epilogue drains TMEM but stores nothing
constexpr int kFlagSkipLoads = 32;     // producer signals stages full without loading anything
constexpr int kFlagNoSfWarps = 64;     // scale-factor warps idle, the MMA warp does not wait for them
constexpr int kFlagNoEpilogue = 128;   // epilogue warps idle, the MMA warp does not wait for them

// Event log for the timing-probe kernels: CTA 0 appends (code << 56 | clock64)
// to its role's 1024-entry strip.
struct Tracer {
    unsigned long long* base;
    int n;
    __device__ Tracer(unsigned long long* trace, int role, unsigned cta = 0)
        : base(trace ? trace + role * 1024 : nullptr), n(0) {
        if (blockIdx.x != cta) base = nullptr;
    }
    __device__ __forceinline__ void operator()(unsigned code) {
        if (base && n < 1024) base[n++] = (static_cast<unsigned long long>(code) << 56) |
                                          (static_cast<unsigned long long>(clock64()) & 0x00FFFFFFFFFFFFFFull);
    }
};
template <Mode M> struct ModeTraits;
template <> struct ModeTraits<Mode::Dual> {
    static constexpr int kMmaN = 256;       // accumulator columns
    static constexpr int kOutCols = 128;    // output columns per tile
    static constexpr bool kSilu = true;
    static constexpr bool kHasBHi = true;
};
template <> struct ModeTraits<Mode::Group128> {
    static constexpr int kMmaN = 128;
    static constexpr int kOutCols = 128;
    static constexpr bool kSilu = false;
    static constexpr bool kHasBHi = false;
};
template <> struct ModeTraits<Mode::Group256> {
    static constexpr int kMmaN = 256;
    static constexpr int kOutCols = 256;
    static constexpr bool kSilu = false;
    static constexpr bool kHasBHi = true;
};

// ---------------------------------------------------------------------------
// Problem descriptions
// ---------------------------------------------------------------------------
// Dual GEMM: lives in kernel parameter space (tensor maps need 64-byte alignment).
struct alignas(64) DenseProblem {
    CUtensorMap map_a, map_b1, map_b2;   // 3-D {k/2 bytes, rows, batch}, box {128, 128, 1}
    CUtensorMap map_c;                   // 3-D {n, m, batch} fp16, box {64, 32, 1}, 128-byte swizzle (pair kernel)
    CUtensorMap map_b1n, map_b2n;        // B1 / B2 with 64-row boxes (narrow pair tiles only)
    CUtensorMap map_c_rank[8];           // gather variant: the full C of every rank of the node (own and peers')
    const uint8_t* sfa;
    const uint8_t* sfb1;
    const uint8_t* sfb2;
    __half* c;
    uint8_t* q_out;                      // quantised-output variant: packed e2m1 [m, n/2] instead of c ...
    uint8_t* sf_out;                     // ... and its e4m3 scale factors in the reordered layout
    long long ldc, c_batch;              // elements
    long long sfa_batch, sfb_batch;      // bytes
    float* splitk_ws;                    // fp32 partial sums (split-k variant only)
    unsigned long long* trace;           // timing probes only: per-role clock64 event log of CTA 0
    uint32_t* splitk_flags;              // eight epoch words per output tile (one per unit)
    uint32_t splitk_epoch;               // value that marks "written during this launch"
    int m_tiles, n_tiles, k_tiles, batches;
    int total_tiles;                     // m_tiles * n_tiles * batches
    int sf_k_atoms;                      // k / 64
    int k_splits;                        // 1 unless split-k
    int sk_tiles;                        // pair kernel: pair tiles in the stream-k tail (0 = none)
    int gather_world, gather_col0;       // gather variant: number of ranks, this shard's first column in the full C
    uint32_t* status;
    unsigned long long* cycles;          // CTA 0 stores its clock64 span here (one store per launch)
};

// Grouped GEMM: one entry per group in device memory (the workspace).
struct alignas(128) GroupEntry {
    CUtensorMap map_a, map_b;            // 3-D {k/2 bytes, rows, 1}
    CUtensorMap map_c;                   // fp16 C of the group for TMA stores (box 64 columns x 32 rows); rows = m, so
                                         // a box that reaches past the group's last row is clipped by the TMA unit
    const uint8_t* sfa;
    const uint8_t* sfb;
    __half* c;
    long long ldc;
    int m, n, k_tiles, m_tiles;
    int n_tiles, tile_begin, sf_k_atoms, sfb_row_atoms;
    int a_row0;                          // first row of this group in map_a (groups that share one A buffer)
    int pad[7];
};
static_assert(sizeof(GroupEntry) == 512, "GroupEntry layout");

struct GroupedProblem {
    const GroupEntry* groups;
    const int* total_tiles_dev;          // non-NULL: the tile count is read from device memory (table built on the device)
    int num_groups;
    int total_tiles;
    uint32_t* status;
    unsigned long long* trace;           // timing probes only
    unsigned long long* cycles;          // CTA 0 stores its clock64 span here (one store per launch)
};

// One unit of work: a 128-row output tile.
struct Work {
    const void* map_a;
    const void* map_blo;
    const void* map_bhi;
    const uint8_t* sfa;      // first 2 KiB chunk (k-tile 0) of this row block
    const uint8_t* sfblo;
    const uint8_t* sfbhi;
    __half* c;               // &C(m0, n0)
    const void* map_c = nullptr;   // grouped CTA-pair tiles: the group's store map
    long long ldc;
    int a_row, blo_row, bhi_row, batch;
    int rows_valid, cols_valid;
    int k_tile_begin, k_tile_count;
    int group;               // grouped modes: index of the group (for tensor-map acquire)
    int tile;                // linear output-tile index (split-k bookkeeping)
    int split;               // which k-split this unit is
};

template <Mode M> struct Scheduler;

template <> struct Scheduler<Mode::Dual> {
    using Params = DenseProblem;
    __device__ static int total_units(const Params& p) { return p.total_tiles * p.k_splits; }
    // Units are ordered split-major inside a tile so the CTAs that share a tile
    // run in the same wave; tiles are ordered m-fastest inside an n panel.
    __device__ static Work get(const Params& p, int unit, int& /*cursor*/) {
        Work w;
        const int split = unit % p.k_splits;
        const int tile = unit / p.k_splits;
        const int m_blk = tile % p.m_tiles;
        const int t = tile / p.m_tiles;
        const int n_blk = t % p.n_tiles;
        const int b = t / p.n_tiles;
        w.map_a = &p.map_a;
        w.map_blo = &p.map_b1;
        w.map_bhi = &p.map_b2;
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
        const int per = (p.k_tiles + p.k_splits - 1) / p.k_splits;
        w.k_tile_begin = split * per;
        w.k_tile_count = min(per, p.k_tiles - w.k_tile_begin);
        w.group = 0;
        w.tile = tile;
        w.split = split;
        return w;
    }
};

template <Mode M> struct GroupScheduler {
    using Params = GroupedProblem;
    static constexpr int kBN = ModeTraits<M>::kOutCols;
    __device__ static int total_units(const Params& p) {
        return p.total_tiles_dev ? *p.total_tiles_dev : p.total_tiles;
    }
    // `cursor` remembers the group of the previous (smaller) tile id so the
    // search is a short forward scan; groups with zero tiles are stepped over.
    __device__ static Work get(const Params& p, int unit, int& cursor) {
        int g = cursor;
        const GroupEntry* e = p.groups + g;
        while (g + 1 < p.num_groups && unit >= e->tile_begin + e->m_tiles * e->n_tiles) {
            ++g;
            ++e;
        }
        cursor = g;
        const int local = unit - e->tile_begin;
        const int m_blk = local % e->m_tiles;   // m fastest: neighbours share a B panel
        const int n_blk = local / e->m_tiles;
        Work w;
        w.map_a = &e->map_a;
        w.map_blo = w.map_bhi = &e->map_b;
        w.a_row = e->a_row0 + m_blk * kTileM;
        w.blo_row = n_blk * kBN;
        w.bhi_row = n_blk * kBN + 128;
        w.batch = 0;
        const long long sf_row = static_cast<long long>(e->sf_k_atoms) * kSfAtomBytes;
        const int lo_atom = n_blk * (kBN / 128);
        const int hi_atom = min(lo_atom + 1, e->sfb_row_atoms - 1);
        w.sfa = e->sfa + m_blk * sf_row;
        w.sfblo = e->sfb + lo_atom * sf_row;
        w.sfbhi = e->sfb + hi_atom * sf_row;
        w.ldc = e->ldc;
        w.c = e->c + static_cast<long long>(m_blk) * kTileM * e->ldc + n_blk * kBN;
        w.rows_valid = min(kTileM, e->m - m_blk * kTileM);
        w.cols_valid = min(kBN, e->n - n_blk * kBN);
        w.k_tile_begin = 0;
        w.k_tile_count = e->k_tiles;
        w.group = g;
        w.tile = unit;
        w.split = 0;
        return w;
    }
};
template <> struct Scheduler<Mode::Group128> : GroupScheduler<Mode::Group128> {};
template <> struct Scheduler<Mode::Group256> : GroupScheduler<Mode::Group256> {};

// ---------------------------------------------------------------------------
// Shared-memory stage and TMEM column maps
// ---------------------------------------------------------------------------
template <Mode M> struct StageLayout {
    using T = ModeTraits<M>;
    static constexpr uint32_t kOffA = 0;
    static constexpr uint32_t kOffBLo = kOperandTileBytes;
    static constexpr uint32_t kOffBHi = 2 * kOperandTileBytes;   // directly after BLo: one descriptor spans 256 rows
    static constexpr uint32_t kOffSfA = (T::kHasBHi ? 3 : 2) * kOperandTileBytes;
    static constexpr uint32_t kOffSfBLo = kOffSfA + kSfChunkBytes;
    static constexpr uint32_t kOffSfBHi = kOffSfBLo + kSfChunkBytes;
    static constexpr uint32_t kBytes = kOffSfBLo + (T::kHasBHi ? 2 : 1) * kSfChunkBytes;  // multiple of 1024
    static constexpr uint32_t kTxBytes = kBytes;
};

// TMEM columns (512 per SM).
// N=256 accumulators: two buffers at columns 0 and 112 that share columns
// [112,256); the epilogue first pulls the shared columns into registers and
// hands them back, so the next tile's MMAs overlap with the rest of the epilogue.
// N=128 accumulators: two disjoint buffers at 0 and 128.
// Scale factors: a ring of slots, one per 64-k block (SFA 4 columns + SFB
// kMmaN/32 columns), handed over kGranule slots at a time.  In the persistent
// kernel they are written by four dedicated warps with tcgen05.st (shared memory
// -> registers -> TMEM, one warp per 32-lane quadrant, which gives the 4x
// replication the MMA expects for free).  A tcgen05.cp costs the tensor pipe
// 30-60 cycles whatever its size, and NVFP4 needs twelve of them per four MMAs,
// so copying through the tensor pipe caps it near half of its peak; the serial
// bring-up kernel still uses tcgen05.cp.  The ring must cover the latency of the
// hand-back loop (MMA retires -> commit seen by the scale-factor warps -> store
// -> MMA warp sees the arrival, 500-1000 cycles): it holds three k-tiles (with 2.5 the
// writers of k-tile j had to wait for the MMAs of k-tile j-2).
template <Mode M> struct TmemMap {
    using T = ModeTraits<M>;
    static constexpr bool kOverlapped = (T::kMmaN == 256);
    static constexpr uint32_t kAccStride = kOverlapped ? 112 : 128;
    static constexpr uint32_t kSharedBegin = kAccStride;               // buffer 0's first column that buffer 1 also uses
    static constexpr uint32_t kSfBase = kOverlapped ? 368 : 256;
    static constexpr uint32_t kSfBCols = T::kMmaN / 32;
    static constexpr uint32_t kSlotCols = 4 + kSfBCols;
    static constexpr int kGranule = kOverlapped ? 2 : 4;              // 64-k blocks per hand-over
    static constexpr int kBuffers = kOverlapped ? 6 : 4;              // hand-over units in the ring
    static constexpr int kSlots = kGranule * kBuffers;
    static constexpr int kEarlyChunks = kOverlapped ? 9 : 0;          // 144 shared columns / 16
    static_assert(kSfBase + kSlots * kSlotCols <= kTmemColumns, "TMEM budget");
    static_assert(kKBlocks % kGranule == 0 && kBuffers <= 8, "ring shape");
    __device__ static constexpr uint32_t sfa_col(int slot) { return kSfBase + slot * kSlotCols; }
    __device__ static constexpr uint32_t sfb_col(int slot) { return kSfBase + slot * kSlotCols + 4; }
};

struct ControlBlock {
    uint64_t full[8];
    uint64_t empty[8];
    uint64_t acc_full[2];
    uint64_t acc_release[2];
    uint64_t sf_ready[8];     // scale factors of a k-tile are in TMEM (slot: k-tile mod 4, or its stage)
    uint64_t aux[2];
    uint32_t tmem_base;
    volatile uint32_t abort_flag;
};

template <Mode M, int kStages> constexpr uint32_t smem_bytes_persistent() {
    return 1024u + kStages * StageLayout<M>::kBytes + sizeof(ControlBlock);
}

// ---------------------------------------------------------------------------
// Role bodies shared by the persistent and the serial kernel
// ---------------------------------------------------------------------------
// kElect: called by every lane of a converged warp with the same arguments, one elected lane
// issues each instruction (see tma_load_3d_elect); otherwise called by one thread.
template <Mode M, bool kTimingProbes = false, bool kElect = false>
__device__ __forceinline__ void issue_stage_loads(const Work& w, int kt, uint32_t stage, uint32_t bar,
                                                  int flags = 0) {
    using L = StageLayout<M>;
    bool load_hi = ModeTraits<M>::kHasBHi;
    if constexpr (kTimingProbes) {
        if (flags & kFlagSkipLoads) {
            if (!kElect || (threadIdx.x & 31) == 0) mbar_arrive(bar);
            return;
        }
        if (flags & kFlagSkipBHi) load_hi = false;
    }
    const uint32_t tx = load_hi || !ModeTraits<M>::kHasBHi ? L::kTxBytes : L::kTxBytes - kOperandTileBytes - kSfChunkBytes;
    const int kbyte = kt * 128;
    const long long sf_off = static_cast<long long>(kt) * kSfChunkBytes;
    if constexpr (kElect) {
        mbar_arrive_expect_tx_elect(bar, tx);
        tma_load_3d_elect(stage + L::kOffA, w.map_a, bar, kbyte, w.a_row, w.batch);
        tma_load_3d_elect(stage + L::kOffBLo, w.map_blo, bar, kbyte, w.blo_row, w.batch);
        if (load_hi) tma_load_3d_elect(stage + L::kOffBHi, w.map_bhi, bar, kbyte, w.bhi_row, w.batch);
        bulk_load_elect(stage + L::kOffSfA, w.sfa + sf_off, kSfChunkBytes, bar);
        bulk_load_elect(stage + L::kOffSfBLo, w.sfblo + sf_off, kSfChunkBytes, bar);
        if (load_hi) bulk_load_elect(stage + L::kOffSfBHi, w.sfbhi + sf_off, kSfChunkBytes, bar);
    } else {
        mbar_arrive_expect_tx(bar, tx);
        tma_load_3d(stage + L::kOffA, w.map_a, bar, kbyte, w.a_row, w.batch);
        tma_load_3d(stage + L::kOffBLo, w.map_blo, bar, kbyte, w.blo_row, w.batch);
        if (load_hi) tma_load_3d(stage + L::kOffBHi, w.map_bhi, bar, kbyte, w.bhi_row, w.batch);
        bulk_load(stage + L::kOffSfA, w.sfa + sf_off, kSfChunkBytes, bar);
        bulk_load(stage + L::kOffSfBLo, w.sfblo + sf_off, kSfChunkBytes, bar);
        if (load_hi) bulk_load(stage + L::kOffSfBHi, w.sfbhi + sf_off, kSfChunkBytes, bar);
    }
}

// Scale factors of k-block `kb` of the k-tile in `stage`: shared memory -> TMEM slot.
template <Mode M>
__device__ __forceinline__ void issue_sf_copy(uint32_t stage, uint32_t tmem_base, int kb, int slot) {
    using L = StageLayout<M>;
    using TM = TmemMap<M>;
    tc_cp_32x128b_warpx4(tmem_base + TM::sfa_col(slot), smem_desc_sf(stage + L::kOffSfA + kb * kSfAtomBytes));
    tc_cp_32x128b_warpx4(tmem_base + TM::sfb_col(slot), smem_desc_sf(stage + L::kOffSfBLo + kb * kSfAtomBytes));
    if constexpr (ModeTraits<M>::kHasBHi)
        tc_cp_32x128b_warpx4(tmem_base + TM::sfb_col(slot) + 4,
                             smem_desc_sf(stage + L::kOffSfBHi + kb * kSfAtomBytes));
}

// The MMA of k-block `kb` (64 e2m1 elements = 32 bytes along k: +2 in the
// descriptor's address field inside the 128-byte swizzle atom).
// `two_mma`: two N=128 MMAs (B-lo, B-hi) instead of one N=256 MMA.
template <Mode M>
__device__ __forceinline__ void issue_mma(uint32_t stage, uint32_t tmem_base, uint32_t acc_col, int kb, int slot,
                                          uint32_t accumulate, bool two_mma) {
    using L = StageLayout<M>;
    using T = ModeTraits<M>;
    using TM = TmemMap<M>;
    const uint64_t adesc = smem_desc_sw128(stage + L::kOffA) + 2 * kb;
    const uint64_t bdesc = smem_desc_sw128(stage + L::kOffBLo) + 2 * kb;
    const uint32_t sfa = tmem_base + TM::sfa_col(slot);
    const uint32_t sfb = tmem_base + TM::sfb_col(slot);
    if (T::kHasBHi && two_mma) {
        const uint64_t bdesc_hi = smem_desc_sw128(stage + L::kOffBHi) + 2 * kb;
        tc_mma_mxf4nvf4(tmem_base + acc_col, adesc, bdesc, idesc_mxf4nvf4(128, 128), sfa, sfb, accumulate);
        tc_mma_mxf4nvf4(tmem_base + acc_col + 128, adesc, bdesc_hi, idesc_mxf4nvf4(128, 128), sfa, sfb + 4,
                        accumulate);
    } else {
        tc_mma_mxf4nvf4(tmem_base + acc_col, adesc, bdesc, idesc_mxf4nvf4(128, T::kMmaN), sfa, sfb, accumulate);
    }
}

// Convert + store one 16-column chunk held by this thread (one output row).
template <bool kSilu>
__device__ __forceinline__ void store_chunk(__half* row_ptr, int chunk, const uint32_t (&x)[16],
                                            const uint32_t (&y)[16]) {
    uint32_t packed[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        float a = __uint_as_float(x[2 * i]), b = __uint_as_float(x[2 * i + 1]);
        if constexpr (kSilu) {
            a = silu_mul(a, __uint_as_float(y[2 * i]));
            b = silu_mul(b, __uint_as_float(y[2 * i + 1]));
        }
        packed[i] = pack_half2(a, b);
    }
    __half* dst = row_ptr + chunk * 16;
    st_global_v4(dst, packed[0], packed[1], packed[2], packed[3]);
    st_global_v4(dst + 8, packed[4], packed[5], packed[6], packed[7]);
}

// Epilogue of one tile for one warp (TMEM lane quadrant `quad`).  When the
// accumulator buffers overlap, the 144 shared columns are pulled into registers
// first and `release` is signalled before any math; their partner columns (the
// other product of the dual GEMM) are not shared and are read later.
//   buffer 0 (columns 0-255):   shared = its columns 112-255
//   buffer 1 (columns 112-367): shared = its columns 0-143
template <Mode M, int kBuf, bool kReleaseInCluster = false>
__device__ __forceinline__ void epilogue_tile(const Work& w, uint32_t tmem_base, int quad, int lane,
                                              uint32_t release_bar, bool store = true) {
    using T = ModeTraits<M>;
    using TM = TmemMap<M>;
    constexpr int kChunks = T::kOutCols / 16;
    constexpr int kEarly = TM::kEarlyChunks;
    constexpr int kSharedRel = (kBuf == 0) ? TM::kSharedBegin : 0;    // first shared column, buffer-relative
    const uint32_t acc = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + kBuf * TM::kAccStride;
    const int row = quad * 32 + lane;
    const bool row_ok = store && row < w.rows_valid;
    __half* row_ptr = w.c + static_cast<long long>(row) * w.ldc;

    uint32_t early[kEarly > 0 ? kEarly : 1][16];
    if constexpr (kEarly > 0) {
#pragma unroll
        for (int i = 0; i < kEarly; ++i) tc_ld_x16(acc + kSharedRel + i * 16, early[i]);
        tc_wait_ld();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
            if constexpr (kReleaseInCluster) mbar_arrive_cluster_relaxed(release_bar);   // barrier of the pair's first CTA
            else mbar_arrive(release_bar);
        }
    }
    // Which buffer-relative 16-column group feeds x (and y) of output chunk c,
    // and whether that group sits in `early`.
#pragma unroll
    for (int chunk = 0; chunk < kChunks; ++chunk) {
        constexpr int kYBase = 128;                      // dual: second product starts at column 128
        const int xcol = chunk * 16;
        const int ycol = kYBase + chunk * 16;
        const bool x_early = kEarly > 0 && xcol >= kSharedRel && xcol < kSharedRel + kEarly * 16;
        const bool y_early = T::kSilu && kEarly > 0 && ycol >= kSharedRel && ycol < kSharedRel + kEarly * 16;
        uint32_t x[16], y[16];
        if (!x_early) tc_ld_x16(acc + xcol, x);
        if (T::kSilu && !y_early) tc_ld_x16(acc + ycol, y);
        if (!x_early || (T::kSilu && !y_early)) tc_wait_ld();
        if (x_early) {
#pragma unroll
            for (int i = 0; i < 16; ++i) x[i] = early[(xcol - kSharedRel) / 16][i];
        }
        if (y_early) {
#pragma unroll
            for (int i = 0; i < 16; ++i) y[i] = early[(ycol - kSharedRel) / 16][i];
        }
        if (row_ok && chunk * 16 < w.cols_valid) store_chunk<T::kSilu>(row_ptr, chunk, x, T::kSilu ? y : x);
    }
}

// Dual-GEMM epilogue that leaves through shared memory and TMA stores (CTA-pair
// kernel).  With one output row per TMEM lane a thread's direct global stores are
// 16 bytes at a 2*ldc-byte pitch: every warp-wide store touches 32 different lines
// and occupies the SM's load/store path (which it shares with shared memory) for 32
// cycles instead of 4.  Here each warp converts its 32 rows x 128 columns into an
// 8 KB staging area (two boxes of 32 rows x 128 bytes in the 128-byte-swizzle layout,
// conflict-free for the 16-byte stores) and one lane hands each box to the TMA unit
// as soon as its 64 columns are done.  `staging` is the warp's own area (1024-byte
// aligned); a box is only rewritten after the previous tile's store has read it.
// kAddPartial (stream-k head piece): `partial` points at this lane's slice of the fp32 partial
// sums another CTA pair computed over the rest of the k range, laid out [4-column group][lane][4];
// they are added to the accumulator values before the activation.
// kGather (column shard whose result every rank of a node wants): each box is stored `gather_world`
// times, once into every rank's full C (its own and, through peer-mapped addresses over NVLink, the
// others'), at this shard's column offset.  Plain TMA stores, no multicast.
template <int kBuf, bool kAddPartial = false, bool kGather = false>
__device__ __forceinline__ void epilogue_tile_staged(const DenseProblem& p, const Work& w, uint32_t tmem_base,
                                                     int quad, int lane, uint32_t release_bar, uint32_t staging,
                                                     int c_col, int c_row, bool store, Tracer* tr = nullptr,
                                                     const float* partial = nullptr) {
    using TM = TmemMap<Mode::Dual>;
    constexpr int kEarly = TM::kEarlyChunks;
    constexpr int kSharedRel = (kBuf == 0) ? TM::kSharedBegin : 0;
    const uint32_t acc = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + kBuf * TM::kAccStride;
    uint32_t early[kEarly][16];
    static_assert(kEarly == 9, "the shared columns are fetched as 64 + 64 + 16");
    tc_ld_x64(acc + kSharedRel, &early[0][0]);
    tc_ld_x64(acc + kSharedRel + 64, &early[4][0]);
    tc_ld_x16(acc + kSharedRel + 128, early[8]);
    if (tr) (*tr)(5);
    tc_wait_ld();
    if (tr) (*tr)(6);
    tc_fence_before_sync();
    __syncwarp();
    if (lane == 0) {
        mbar_arrive_cluster_relaxed(release_bar);   // barrier of the pair's first CTA
        if (tr) (*tr)(7);
        bulk_wait_group_read_all();                  // the previous tile's boxes have left the staging area
    }
    __syncwarp();
    const uint32_t row_base = staging + lane * 128;
    const uint32_t swz = static_cast<uint32_t>(lane & 7);
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
        if constexpr (kAddPartial) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float4 px = ld_global_cg_v4f(partial + static_cast<size_t>(xcol / 4 + j) * 128);
                const float4 py = ld_global_cg_v4f(partial + static_cast<size_t>(ycol / 4 + j) * 128);
                x[4 * j] = __float_as_uint(__uint_as_float(x[4 * j]) + px.x);
                x[4 * j + 1] = __float_as_uint(__uint_as_float(x[4 * j + 1]) + px.y);
                x[4 * j + 2] = __float_as_uint(__uint_as_float(x[4 * j + 2]) + px.z);
                x[4 * j + 3] = __float_as_uint(__uint_as_float(x[4 * j + 3]) + px.w);
                y[4 * j] = __float_as_uint(__uint_as_float(y[4 * j]) + py.x);
                y[4 * j + 1] = __float_as_uint(__uint_as_float(y[4 * j + 1]) + py.y);
                y[4 * j + 2] = __float_as_uint(__uint_as_float(y[4 * j + 2]) + py.z);
                y[4 * j + 3] = __float_as_uint(__uint_as_float(y[4 * j + 3]) + py.w);
            }
        }
        uint32_t packed[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
            packed[i] = pack_half2(silu_mul(__uint_as_float(x[2 * i]), __uint_as_float(y[2 * i])),
                                   silu_mul(__uint_as_float(x[2 * i + 1]), __uint_as_float(y[2 * i + 1])));
        // box = chunk / 4 (64 columns each); inside it this chunk is 16-byte units 2*(chunk%4), +1
        const uint32_t box = row_base + static_cast<uint32_t>(chunk >> 2) * 4096u;
        const uint32_t u0 = static_cast<uint32_t>((chunk & 3) * 2);
        st_shared_v4(box + ((u0 ^ swz) << 4), packed[0], packed[1], packed[2], packed[3]);
        st_shared_v4(box + (((u0 + 1) ^ swz) << 4), packed[4], packed[5], packed[6], packed[7]);
        if ((chunk & 3) == 3) {
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0 && store) {
                const uint32_t box_addr = staging + static_cast<uint32_t>(chunk >> 2) * 4096u;
                if constexpr (kGather) {
                    for (int r = 0; r < p.gather_world; ++r)
                        tma_store_3d(&p.map_c_rank[r], box_addr, p.gather_col0 + c_col + (chunk >> 2) * 64, c_row, 0);
                } else {
                    tma_store_3d(&p.map_c, box_addr, c_col + (chunk >> 2) * 64, c_row, w.batch);
                }
                bulk_commit_group();
            }
        }
    }
}

// Split-k epilogue (dual GEMM with few output tiles): a tile's k range is cut into
// `k_splits` units that run on different CTAs at the same time (the host never
// launches more units than there are SMs, one CTA per SM).  Output column chunk c
// (16 columns) is finished by unit c % k_splits: every unit writes the fp32
// partial sums of the chunks it does not own to the workspace, publishes a flag,
// waits (bounded) for its peers' flags and adds their partial sums of its own
// chunks to its accumulator in unit order, so the result does not depend on
// timing.  Each unit runs 1/k_splits of the silu*mul epilogue.
// Workspace: flags[tile][8] (uint32, written with the launch's epoch, never reset)
// then per (tile, unit) 128 KiB laid out [chunk][x|y][quarter][row][4 floats] so
// that a warp's stores and loads are contiguous.
template <int kBuf>
__device__ __forceinline__ bool epilogue_tile_splitk(const DenseProblem& p, const Work& w, uint32_t tmem_base,
                                                     int quad, int lane, uint32_t release_bar,
                                                     volatile uint32_t* abort_flag) {
    using TM = TmemMap<Mode::Dual>;
    const uint32_t acc = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + kBuf * TM::kAccStride;
    const int row = quad * 32 + lane;
    const int splits = p.k_splits;
    const size_t unit_floats = static_cast<size_t>(kTileM) * 256;
    float* tile_ws = p.splitk_ws + static_cast<size_t>(w.tile) * splits * unit_floats;
    float* mine = tile_ws + static_cast<size_t>(w.split) * unit_floats + row * 4;
    uint32_t* flags = p.splitk_flags + static_cast<size_t>(w.tile) * 8;
    // ---- send the chunks other units own
#pragma unroll 1
    for (int chunk = 0; chunk < 8; ++chunk) {
        if (chunk % splits == w.split) continue;
        uint32_t x[16], y[16];
        tc_ld_x16(acc + chunk * 16, x);
        tc_ld_x16(acc + 128 + chunk * 16, y);
        tc_wait_ld();
        float* dst = mine + static_cast<size_t>(chunk) * 8 * (kTileM * 4);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            st_global_v4f(dst + q * (kTileM * 4), x[4 * q], x[4 * q + 1], x[4 * q + 2], x[4 * q + 3]);
            st_global_v4f(dst + (4 + q) * (kTileM * 4), y[4 * q], y[4 * q + 1], y[4 * q + 2], y[4 * q + 3]);
        }
    }
    __threadfence();
    epilogue_bar_sync();
    if (threadIdx.x == 0) st_release_gpu_u32(flags + w.split, p.splitk_epoch);
    // ---- wait for the peers (every lane polls: a single polling lane followed by a
    // shuffle wakes the warp up measurably later; bounded)
    bool ok = true;
    {
        const long long t0 = clock64();
        for (int peer = 0; peer < splits && ok; ++peer) {
            if (peer == w.split) continue;
            while (ld_acquire_gpu_u32(flags + peer) != p.splitk_epoch) {
                if (*abort_flag || clock64() - t0 > kWaitTimeoutCycles) {
                    *abort_flag = 1u;
                    atomicOr(p.status, kStatusSplitKWait);
                    ok = false;
                    break;
                }
            }
        }
    }
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
        __half* row_ptr = w.c + static_cast<long long>(row) * w.ldc;
#pragma unroll 1
        for (int chunk = w.split; chunk < 8; chunk += splits) {
            uint32_t xb[16], yb[16];
            tc_ld_x16(acc + chunk * 16, xb);
            tc_ld_x16(acc + 128 + chunk * 16, yb);
            float x[16], y[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) x[i] = y[i] = 0.0f;
            bool own_added = false;
            for (int unit = 0; unit < splits; ++unit) {
                if (unit == w.split) {
                    tc_wait_ld();
#pragma unroll
                    for (int i = 0; i < 16; ++i) { x[i] += __uint_as_float(xb[i]); y[i] += __uint_as_float(yb[i]); }
                    own_added = true;
                    continue;
                }
                const float* src = tile_ws + static_cast<size_t>(unit) * unit_floats + row * 4 +
                                   static_cast<size_t>(chunk) * 8 * (kTileM * 4);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float4 a = ld_global_cg_v4f(src + q * (kTileM * 4));
                    const float4 b = ld_global_cg_v4f(src + (4 + q) * (kTileM * 4));
                    x[4 * q] += a.x; x[4 * q + 1] += a.y; x[4 * q + 2] += a.z; x[4 * q + 3] += a.w;
                    y[4 * q] += b.x; y[4 * q + 1] += b.y; y[4 * q + 2] += b.z; y[4 * q + 3] += b.w;
                }
            }
            if (!own_added) tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 16; ++i) { xb[i] = __float_as_uint(x[i]); yb[i] = __float_as_uint(y[i]); }
            store_chunk<true>(row_ptr, chunk, xb, yb);
        }
    }
    tc_fence_before_sync();
    __syncwarp();
    if (lane == 0) mbar_arrive(release_bar);       // accumulator drained: the MMA warp may reuse it
    return ok;
}

// ---------------------------------------------------------------------------
// Persistent warp-specialised kernel: 10 warps.
//   warps 0-3  epilogue (TMEM lane quadrants 0-3)
//   warp 4     TMEM allocation + first MMA issuer (one lane)
//   warp 5     TMA producer (one lane)
//   warps 6-9  scale factors shared memory -> TMEM (quadrants 2, 3, 0, 1)
// CTA b walks work units b, b+grid, b+2*grid, ...
// ---------------------------------------------------------------------------
// MMA-issuing threads.  Two issuers (warps 4 and 10, taking turns k-tile by k-tile)
// were measured and bring nothing: the limit is not the issuing thread.
constexpr int kIssuers = 1;
// Sets of four scale-factor warps that take turns k-tile by k-tile.  Two sets (16
// warps, registers rebalanced per warpgroup with setmaxnreg) were measured: the
// scale-factor hand-over gets faster but loads, epilogue and launch overhead get
// slower by more.
constexpr int kSfSets = 1;
constexpr int kFirstSfWarp = kSfSets == 2 ? 8 : 6;
constexpr int kPersistentThreads = 32 * (kFirstSfWarp + 4 * kSfSets);

template <Mode M, int kStages, bool kTimingProbes = false, bool kInjectLostLoad = false>
__global__ void __launch_bounds__(kPersistentThreads, 1)
nvfp4_gemm_persistent(const __grid_constant__ typename Scheduler<M>::Params p, int flags) {
    using L = StageLayout<M>;
    using TM = TmemMap<M>;
    using S = Scheduler<M>;
    // fault-injection self-test: the producer drops the loads of one k-tile, every wait gives up early
    constexpr long long kLimit = kInjectLostLoad ? kShortWaitTimeoutCycles : kWaitTimeoutCycles;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    ControlBlock* ctl = reinterpret_cast<ControlBlock*>(smem_raw + (smem_base - smem_u32(smem_raw)) +
                                                        kStages * L::kBytes);
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const long long launch_t0 = clock64();
    griddep_launch_dependents();   // the next launch may move onto SMs as this grid's CTAs leave them

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(smem_u32(&ctl->full[s]), 1);
            mbar_init(smem_u32(&ctl->empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&ctl->acc_full[b]), kIssuers);   // every MMA issuer commits
            mbar_init(smem_u32(&ctl->acc_release[b]), 4);
        }
        for (int i = 0; i < 4; ++i) mbar_init(smem_u32(&ctl->sf_ready[i]), 4);
        mbar_init(smem_u32(&ctl->aux[0]), 1);
        mbar_init(smem_u32(&ctl->aux[1]), 1);
        ctl->abort_flag = 0;
        fence_mbar_init();
        fence_proxy_async_smem();
    }
    if (warp == 4) {
        tmem_alloc(smem_u32(&ctl->tmem_base), kTmemColumns);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = ctl->tmem_base;
    volatile uint32_t* abort_flag = &ctl->abort_flag;
    // Everything above touched only this CTA's own resources; from here on global memory is read and
    // written, which must wait for the kernels before this one in the stream.
    griddep_wait();
    const int total = S::total_units(p);

    // Register budget per warpgroup (512 threads start with 128 each): the epilogue
    // holds 128 accumulator columns in registers, everybody else needs few.
    if constexpr (kSfSets == 2) {
        if (warp < 4) warpgroup_reg_inc<168>();
        else if (warp < 8) warpgroup_reg_dec<120>();
        else warpgroup_reg_dec<112>();
    }

    if (kTimingProbes && warp >= kFirstSfWarp && (flags & kFlagNoSfWarps)) {
        // timing probe: these warps sit the launch out
    } else if (kTimingProbes && warp < 4 && (flags & kFlagNoEpilogue)) {
        // timing probe: these warps sit the launch out
    } else if (warp >= kFirstSfWarp) {
        // ------------------------------ scale factors: shared memory -> TMEM
        // kSfSets sets of four warps (one warp per TMEM lane quadrant in each set) take
        // turns k-tile by k-tile.  One warp needs ~900 cycles per k-tile (two or three
        // barrier waits, twelve shared-memory loads, the stores, a fence, an arrival);
        // the MMAs of a k-tile take 520.
        const uint32_t sf_set = static_cast<uint32_t>(warp - kFirstSfWarp) >> 2;
        // Lane r of the warp serving quadrant q reads row r of each 512-byte atom
        // (16 bytes = the row's scale factors for four 16-k blocks of four 32-row
        // groups) and writes it to TMEM lane 32q + r, four columns per atom.  A
        // whole k-tile is read into registers as soon as its stage lands; each
        // 64-k block is then written the moment its ring slot is free.
        const uint32_t quad_lane = static_cast<uint32_t>((warp & 3) * 32) << 16;
        uint32_t s = 0, ph = 0;            // stage and its phase
        uint32_t buf = 0, use = 0;         // ring position: hand-over unit and how often it has been used
        uint32_t units = 0;                // hand-over units written so far
        uint32_t kt = 0;                   // k-tiles handed to the MMA warp so far
        uint32_t retired = 0;              // k-tiles whose MMAs are known to have retired ...
        uint32_t rs = 0, rph = 0;          // ... and the `empty` barrier that reports the next one
        constexpr uint32_t kUnitsPerKTile = kKBlocks / TM::kGranule;
        int cursor = 0;
        bool ok = true;
        const bool skip = kTimingProbes && (flags & kFlagSkipSfCopy);
        constexpr int kAtoms = ModeTraits<M>::kHasBHi ? 3 : 2;
        Tracer trace(kTimingProbes && lane == 0 && sf_set == 0 ? p.trace : nullptr,
                     warp == kFirstSfWarp ? 1 : warp - kFirstSfWarp + 3);   // roles 1, 4, 5, 6
        // v holds one k-tile's scale factors in TMEM column order: per 64-k block
        // [SFA 4 | SFB-lo 4 | SFB-hi 4] words.  The next k-tile is read into it right
        // after the current one has been handed over, so the loads are off the path
        // between "ring unit free" and "handed to the MMA warp".
        constexpr int kWordsPerBlock = TM::kSlotCols;
        uint32_t v[kKBlocks * kWordsPerBlock];
        bool loaded = false;
        auto load_k_tile = [&](uint32_t stage_index, uint32_t phase) -> bool {
            if (!mbar_wait<true, kLimit>(smem_u32(&ctl->full[stage_index]), phase, abort_flag, p.status, kStatusSfWait))
                return false;
            const uint32_t src = smem_base + stage_index * L::kBytes + lane * 16;
#pragma unroll
            for (int kb = 0; kb < kKBlocks; ++kb) {
                uint32_t* d = v + kb * kWordsPerBlock;
                ld_shared_v4(src + L::kOffSfA + kb * kSfAtomBytes, d[0], d[1], d[2], d[3]);
                ld_shared_v4(src + L::kOffSfBLo + kb * kSfAtomBytes, d[4], d[5], d[6], d[7]);
                if constexpr (kAtoms == 3) ld_shared_v4(src + L::kOffSfBHi + kb * kSfAtomBytes, d[8], d[9], d[10], d[11]);
            }
            return true;
        };
        for (int unit = blockIdx.x; ok && unit < total; unit += gridDim.x) {
            const Work w = S::get(p, unit, cursor);
            for (int i = 0; ok && i < w.k_tile_count; ++i) {
                if ((kt % kSfSets) != sf_set) {
                    // the other set's k-tile: only keep the counters in step
                    units += kUnitsPerKTile;
                    buf += kUnitsPerKTile;
                    if (buf >= static_cast<uint32_t>(TM::kBuffers)) { buf -= TM::kBuffers; ++use; }
                    ++kt;
                    if (++s == kStages) { s = 0; ph ^= 1u; }
                    continue;
                }
                if (!loaded && !load_k_tile(s, ph)) {
                    ok = false;
                    break;
                }
                trace(1);   // k-tile in registers
#pragma unroll
                for (int gr = 0; gr < kKBlocks / TM::kGranule; ++gr, ++units) {
                    // The unit's previous contents were read by the MMAs of k-tile
                    // (units - kBuffers) / kUnitsPerKTile; the stage's `empty` barrier
                    // (one tcgen05.commit per k-tile) says when those have retired.
                    if (units >= static_cast<uint32_t>(TM::kBuffers)) {
                        const uint32_t need = (units - TM::kBuffers) / kUnitsPerKTile;
                        if (retired <= need) {
                            // k-tiles retire in issue order (one issuer): waiting for the newest one
                            // needed covers the older ones; with two issuers every one is waited for
                            while (kIssuers == 1 && retired < need) {
                                ++retired;
                                if (++rs == kStages) { rs = 0; rph ^= 1u; }
                            }
                            while (ok && retired <= need) {
                                ok = mbar_wait<true, kLimit>(smem_u32(&ctl->empty[rs]), rph, abort_flag, p.status, kStatusSfWait);
                                ++retired;
                                if (++rs == kStages) { rs = 0; rph ^= 1u; }
                            }
                            if (!ok) break;
                            tc_fence_after_sync();
                        }
                    }
                    trace(2);   // ring unit free
                    if (!skip || use == 0) {
                        // one unit = kGranule blocks = contiguous TMEM columns
                        const uint32_t dst = tmem_base + quad_lane + TM::sfa_col(buf * TM::kGranule);
                        const uint32_t* src = v + gr * TM::kGranule * kWordsPerBlock;
                        constexpr int kUnitWords = TM::kGranule * kWordsPerBlock;   // 24 (N=256 modes) or 32
                        if constexpr (kUnitWords == 24) {
                            tc_st_x16(dst, src);
                            tc_st_x8(dst + 16, src + 16);
                        } else {
                            tc_st_x16(dst, src);
                            tc_st_x16(dst + 16, src + 16);
                        }
                    }
                    if (++buf == TM::kBuffers) { buf = 0; ++use; }
                }
                if (!ok) break;
                if (!skip || use == 0) tc_wait_st();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&ctl->sf_ready[kt & 3u]));
                trace(3);   // k-tile handed to the MMA warp
                ++kt;
                if (++s == kStages) { s = 0; ph ^= 1u; }
                loaded = false;
            }
        }
    } else if (warp == 5) {
        // ------------------------------ TMA producer
        // The whole warp runs the loop in lock step on warp-uniform values; one elected lane issues.
        {
            uint32_t s = 0, ph = 0;
            int cursor = 0, last_group = -1;
            bool ok = true;
            Tracer trace(kTimingProbes && lane == 0 ? p.trace : nullptr, 2);
            for (int unit = blockIdx.x; ok && unit < total; unit += gridDim.x) {
                const Work w = S::get(p, unit, cursor);
                if (M != Mode::Dual && w.group != last_group) {
                    tensormap_acquire(w.map_a);
                    tensormap_acquire(w.map_blo);
                    last_group = w.group;
                }
                for (int i = 0; i < w.k_tile_count; ++i) {
                    if (!__all_sync(0xffffffffu, mbar_wait<true, kLimit>(smem_u32(&ctl->empty[s]), ph ^ 1u, abort_flag,
                                                                         p.status, kStatusProducerWait))) {
                        ok = false;
                        break;
                    }
                    trace(1);   // stage free, loads issued
                    if (kInjectLostLoad && i == 1) {   // self-test: this k-tile never arrives
                        if (++s == kStages) { s = 0; ph ^= 1u; }
                        continue;
                    }
                    issue_stage_loads<M, kTimingProbes, true>(w, w.k_tile_begin + i, smem_base + s * L::kBytes,
                                                              smem_u32(&ctl->full[s]), flags);
                    if (++s == kStages) { s = 0; ph ^= 1u; }
                }
            }
            if (!ok) {
                // error path only: give copies still in flight time to land
                for (int i = 0; i < 64; ++i) __nanosleep(2000);
            }
        }
        __syncwarp();
    } else if (warp == 4 || (kIssuers == 2 && kSfSets == 2 && warp == 6)) {
        // ------------------------------ MMA issuer(s)
        // kIssuers threads (on different SM sub-partitions) issue the MMAs, taking
        // turns k-tile by k-tile.  Each tcgen05.mma, tcgen05.commit and
        // mbarrier.try_wait costs its thread about 50 cycles; four MMAs occupy the
        // tensor pipe for 520 cycles, so the loop is kept to the bare minimum.
        // Per k-tile an issuer does one wait (on the scale factors; their writers
        // waited for the stage's `full` barrier before reading the stage, which
        // orders the operand bytes before these MMAs too), four MMAs and one commit.
        // Accumulation commutes, so with two issuers the streams need no mutual order
        // except at the start of a tile: the k-tile that clears the accumulator must have
        // retired before the other issuer adds to it.
        if (lane == 0) {
            using T = ModeTraits<M>;
            constexpr uint32_t kUnitCols = TM::kGranule * TM::kSlotCols;
            constexpr uint32_t kUnitsPerKTile = kKBlocks / TM::kGranule;
            const uint32_t me = (warp == 4) ? 0u : 1u;
            const uint32_t desc_lo_base = smem_desc_lo(smem_base + L::kOffA);
            const uint32_t sf_ready_bar = smem_u32(&ctl->sf_ready[0]);
            const uint32_t empty_bar = smem_u32(&ctl->empty[0]);
            const uint32_t sf_base = tmem_base + TM::kSfBase;
            uint32_t s = 0, s_use = 0, a_lo = desc_lo_base;   // stage, how often it has been used, its A descriptor
            uint32_t kt = 0;                                   // running k-tile count
            uint32_t buf = 0;                                  // scale-factor ring unit of the k-tile's first half
            int cursor = 0, it = 0;
            bool failed = false;
            const int mma_blocks = (kTimingProbes && (flags & kFlagSkipMma)) ? 1 : kKBlocks;
            const bool no_sf = kTimingProbes && (flags & kFlagNoSfWarps);
            const bool no_epi = kTimingProbes && (flags & kFlagNoEpilogue);
            Tracer trace(kTimingProbes && me == 0 ? p.trace : nullptr, 0);
            for (int unit = blockIdx.x; unit < total && !failed; unit += gridDim.x, ++it) {
                const Work w = S::get(p, unit, cursor);
                if (it > 0 && !no_epi) {
                    const int r = it - 1;   // wait for hand-back number r
                    if (!mbar_wait<false, kLimit>(smem_u32(&ctl->acc_release[r & 1]), (r >> 1) & 1, abort_flag, p.status,
                                   kStatusMmaWaitAcc)) {
                        failed = true;
                        break;
                    }
                    tc_fence_after_sync();
                }
                trace(9);   // accumulator buffer available
                const uint32_t acc_addr = tmem_base + (it & 1) * TM::kAccStride;
                const int k_tiles = w.k_tile_count;
                // the tile's first k-tile clears the accumulator; if the other issuer owns it,
                // wait until it has retired (its stage's `empty` barrier) before adding anything
                const bool first_is_mine = (kt % kIssuers) == me;
                const uint32_t first_empty = empty_bar + s * 8, first_parity = s_use & 1u;
                bool first_done = first_is_mine;
#pragma unroll 1
                for (int i = 0; i < k_tiles; ++i) {
                    if (kIssuers == 1 || (kt % kIssuers) == me) {
                        if (kIssuers > 1 && !first_done) {
                            if (!mbar_wait<false, kLimit>(first_empty, first_parity, abort_flag, p.status, kStatusMmaWaitAcc)) {
                                failed = true;
                                break;
                            }
                            first_done = true;
                        }
                        const uint32_t bar = no_sf ? smem_u32(&ctl->full[s]) : sf_ready_bar + (kt & 3u) * 8u;
                        const uint32_t parity = no_sf ? s_use & 1u : (kt >> 2) & 1u;
                        if (!mbar_wait<false, kLimit>(bar, parity, abort_flag, p.status, kStatusMmaWaitFull)) {
                            failed = true;
                            break;
                        }
                        tc_fence_after_sync();
                        trace(1);   // k-tile ready
                        uint32_t b = buf;
#pragma unroll
                        for (int kb = 0; kb < kKBlocks; ++kb) {
                            if (kb > 0 && kb % TM::kGranule == 0) b = (b + 1 == TM::kBuffers) ? 0u : b + 1;
                            if (kTimingProbes && kb >= mma_blocks) continue;
                            const uint32_t sfa = sf_base + b * kUnitCols + (kb % TM::kGranule) * TM::kSlotCols;
                            tc_mma_mxf4nvf4_lo(acc_addr, a_lo + 2 * kb, a_lo + (L::kOffBLo >> 4) + 2 * kb,
                                               idesc_mxf4nvf4(128, T::kMmaN), sfa, sfa + 4,
                                               (kb > 0 || i > 0) ? 1u : 0u);
                        }
                        // one commit per k-tile: frees the stage for the producer and tells the
                        // scale-factor warps that the ring units this k-tile read are reusable
                        tc_commit(empty_bar + s * 8);
                    }
                    ++kt;
                    buf += kUnitsPerKTile;
                    if (buf >= static_cast<uint32_t>(TM::kBuffers)) buf -= TM::kBuffers;
                    ++s;
                    a_lo += L::kBytes >> 4;
                    if (s == kStages) { s = 0; a_lo = desc_lo_base; ++s_use; }
                }
                if (failed) break;
                tc_commit(smem_u32(&ctl->acc_full[it & 1]));   // arrives once this issuer's MMAs of the tile retire
            }
            // drain: every MMA issued above must retire before TMEM is freed
            tc_commit(smem_u32(&ctl->aux[me]));
            mbar_wait<false, kLimit>(smem_u32(&ctl->aux[me]), 0, abort_flag, p.status, kStatusMmaWaitAcc);
        }
        __syncwarp();
    } else if (warp < 4) {
        // ------------------------------ epilogue warps 0-3
        int cursor = 0, it = 0;
        bool ok = true;
        Tracer trace(kTimingProbes && warp == 0 && lane == 0 ? p.trace : nullptr, 3);
        for (int unit = blockIdx.x; ok && unit < total; unit += gridDim.x, ++it) {
            const Work w = S::get(p, unit, cursor);
            const uint32_t release_bar = smem_u32(&ctl->acc_release[it & 1]);
            if constexpr (!TM::kOverlapped) {
                // disjoint buffers: hand-back number `it` says "tile it-1 is drained"
                __syncwarp();
                if (lane == 0) mbar_arrive(release_bar);
            }
            if (!mbar_wait<true, kLimit>(smem_u32(&ctl->acc_full[it & 1]), (it >> 1) & 1, abort_flag, p.status,
                                 kStatusEpilogueWait)) {
                ok = false;
                break;
            }
            tc_fence_after_sync();
            trace(1);   // accumulator complete
            const bool store = !(kTimingProbes && (flags & kFlagSkipStores));
            bool split = false;
            if constexpr (M == Mode::Dual) split = p.k_splits > 1;
            if (split) {
                if constexpr (M == Mode::Dual) {
                    ok = (it & 1) ? epilogue_tile_splitk<1>(p, w, tmem_base, warp, lane, release_bar, abort_flag)
                                  : epilogue_tile_splitk<0>(p, w, tmem_base, warp, lane, release_bar, abort_flag);
                }
            } else if (it & 1)
                epilogue_tile<M, 1>(w, tmem_base, warp, lane, release_bar, store);
            else
                epilogue_tile<M, 0>(w, tmem_base, warp, lane, release_bar, store);
            trace(2);   // tile stored
            tc_fence_before_sync();
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 4) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemColumns);
    }
    if (blockIdx.x == 0 && threadIdx.x == 0 && p.cycles) *p.cycles = static_cast<unsigned long long>(clock64() - launch_t0);
}

// ---------------------------------------------------------------------------
// Serial kernel: one CTA (128 threads) per work unit, one stage, every step
// waits for the previous one.  Slow by construction; exists to validate the
// descriptors and layouts independently of the pipelined kernel.
// ---------------------------------------------------------------------------
template <Mode M>
__global__ void __launch_bounds__(128, 1)
nvfp4_gemm_serial(const __grid_constant__ typename Scheduler<M>::Params p, int flags) {
    using L = StageLayout<M>;
    using S = Scheduler<M>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    ControlBlock* ctl = reinterpret_cast<ControlBlock*>(smem_raw + (smem_base - smem_u32(smem_raw)) + L::kBytes);
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&ctl->full[0]), 1);
        mbar_init(smem_u32(&ctl->empty[0]), 1);
        mbar_init(smem_u32(&ctl->acc_release[0]), 4);
        ctl->abort_flag = 0;
        fence_mbar_init();
        fence_proxy_async_smem();
    }
    if (warp == 0) {
        tmem_alloc(smem_u32(&ctl->tmem_base), kTmemColumns);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = ctl->tmem_base;
    volatile uint32_t* abort_flag = &ctl->abort_flag;
    int cursor = 0;
    const int unit = blockIdx.x;
    if (unit < S::total_units(p)) {
        const Work w = S::get(p, unit, cursor);
        if (threadIdx.x == 0) {
            if (M != Mode::Dual) {
                tensormap_acquire(w.map_a);
                tensormap_acquire(w.map_blo);
            }
            uint32_t ph = 0;
            for (int i = 0; i < w.k_tile_count; ++i, ph ^= 1u) {
                issue_stage_loads<M>(w, w.k_tile_begin + i, smem_base, smem_u32(&ctl->full[0]));
                if (!mbar_wait(smem_u32(&ctl->full[0]), ph, abort_flag, p.status, kStatusSerialWait)) break;
                tc_fence_after_sync();
#pragma unroll
                for (int kb = 0; kb < kKBlocks; ++kb) issue_sf_copy<M>(smem_base, tmem_base, kb, kb);
#pragma unroll
                for (int kb = 0; kb < kKBlocks; ++kb)
                    issue_mma<M>(smem_base, tmem_base, 0, kb, kb, (i > 0 || kb > 0) ? 1u : 0u,
                                 (flags & kFlagTwoMma) != 0);
                tc_commit(smem_u32(&ctl->empty[0]));
                if (!mbar_wait(smem_u32(&ctl->empty[0]), ph, abort_flag, p.status, kStatusSerialWait)) break;
            }
        }
        __syncwarp();
        tc_fence_before_sync();
        __syncthreads();
        tc_fence_after_sync();
        if (!*abort_flag) epilogue_tile<M, 0>(w, tmem_base, warp, lane, smem_u32(&ctl->acc_release[0]));
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemColumns);
    }
}

}  // namespace b200
