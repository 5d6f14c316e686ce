// The steps around the grouped GEMM in a mixture-of-experts layer, as the reference's MoE
// states them (moe/moe_fibench_ref.py:20-33, 106-176): DeepSeek-V3 "no-aux" routing, the
// permutation of token rows into per-expert row ranges, and the weighted combination of
// the experts' outputs.  The reference does all of this with torch ops on fp32 / FP8 data;
// here the expert GEMM is the NVFP4 grouped GEMM, so the gather also quantises.
//
//   moe_route             logits [T, E] -> top_k expert ids and weights per token
//   moe_count/scan/place  counting sort of the T * top_k (token, slot) entries by expert,
//                         stable in token order: per-expert counts, row ranges, row of
//                         every entry, source token of every row
//   moe_quantize_rows / moe_gather_rows   x[token] -> NVFP4 row of the expert's A operand + scale factors
//   moe_fill_group_table  the dynamic fields of the grouped GEMM's descriptor table
//   moe_combine           out[t] = sum over slots of weight * y[row(t, slot)]
// All are HBM-bound integer / byte kernels except the last two steps' arithmetic; nothing
// here reads back to the host.
#pragma once

#include <cfloat>

#include "nvfp4_gemm_kernels.cuh"
#include "nvfp4_quantize.cuh"

namespace b200 {

constexpr int kMoeMaxExperts = 256;
constexpr int kMoeChunk = 1024;          // (token, slot) entries per block of the counting sort
#ifndef B200_MOE_SCATTER_SPLIT
#define B200_MOE_SCATTER_SPLIT 4
#endif
constexpr int kMoeScatterSplit = B200_MOE_SCATTER_SPLIT;   // warps that share one token in moe_quantize_scatter

// Largest value in the warp and the smallest index that holds it.
__device__ __forceinline__ void warp_argmax(float& val, int& idx) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, val, off);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, off);
        if (ov > val || (ov == val && oi < idx)) {
            val = ov;
            idx = oi;
        }
    }
}

// One warp per token (moe/moe_fibench_ref.py:106-134):
//   s = sigmoid(logits), s_b = s + bias; experts form n_group groups; a group's score is the sum
//   of its two largest s_b; only the topk_group best groups stay; the top_k largest s_b among
//   them are the token's experts; weight = s / (sum of the chosen s + 1e-20) * scale.
// Ties go to the smaller index.  Slots are written in descending order of s_b.
__global__ void __launch_bounds__(256) moe_route(const float* __restrict__ logits, const float* __restrict__ bias,
                                                 int tokens, int experts, int n_group, int topk_group, int top_k,
                                                 float scale, int* __restrict__ topk_idx, float* __restrict__ topk_w) {
    __shared__ float s_sig[8][kMoeMaxExperts];
    __shared__ float s_wb[8][kMoeMaxExperts];
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    const int token = blockIdx.x * 8 + wib;
    if (token >= tokens) return;
    float* sig = s_sig[wib];
    float* wb = s_wb[wib];
    for (int e = lane; e < experts; e += 32) {
        const float s = 1.0f / (1.0f + expf(-logits[static_cast<long long>(token) * experts + e]));
        sig[e] = s;
        wb[e] = s + (bias ? bias[e] : 0.0f);
    }
    __syncwarp();
    const int group_size = experts / n_group;
    // group score: lane g scans group g
    float gscore = -FLT_MAX;
    if (lane < n_group) {
        float a = -FLT_MAX, b = -FLT_MAX;      // largest, second largest
        for (int i = 0; i < group_size; ++i) {
            const float v = wb[lane * group_size + i];
            if (v > a) {
                b = a;
                a = v;
            } else if (v > b) {
                b = v;
            }
        }
        gscore = group_size >= 2 ? a + b : a;
    }
    uint32_t group_mask = 0;
    for (int r = 0; r < topk_group; ++r) {
        float v = gscore;
        int g = lane;
        warp_argmax(v, g);
        group_mask |= 1u << g;
        if (lane == g) gscore = -FLT_MAX;
    }
    // experts outside the kept groups drop to the lowest value (the reference fills them with finfo.min)
    for (int e = lane; e < experts; e += 32)
        if (!((group_mask >> (e / group_size)) & 1u)) wb[e] = -FLT_MAX;
    __syncwarp();
    float wsum = 0.0f, my_w = 0.0f;
    int my_e = 0;
    for (int r = 0; r < top_k; ++r) {
        float v = -FLT_MAX;
        int best = 0x7fffffff;
        for (int e = lane; e < experts; e += 32) {
            const float c = wb[e];
            if (c > v || (c == v && e < best)) {
                v = c;
                best = e;
            }
        }
        warp_argmax(v, best);
        const float s = sig[best];
        wsum += s;
        if (lane == r) {
            my_e = best;
            my_w = s;
        }
        __syncwarp();
        if (lane == 0) wb[best] = -INFINITY;   // taken
        __syncwarp();
    }
    if (lane < top_k) {
        topk_idx[static_cast<long long>(token) * top_k + lane] = my_e;
        topk_w[static_cast<long long>(token) * top_k + lane] = my_w / (wsum + 1e-20f) * scale;
    }
}

// The same routing with the token's scores in registers: lane l of the token's warp holds the kPerLane
// consecutive experts [l * kPerLane, (l + 1) * kPerLane), so a group of experts is a run of
// `lanes_per_group` = group_size / kPerLane lanes (a power of two) and nothing is re-read from shared memory
// for the group scores or for any of the top_k picks.  For experts == 32 * kPerLane, group_size % kPerLane == 0
// and lanes_per_group a power of two; same picks, same order, same ties (smaller index) as moe_route.
template <int kPerLane>
__global__ void __launch_bounds__(256) moe_route_regs(const float* __restrict__ logits, const float* __restrict__ bias,
                                                      int tokens, int n_group, int topk_group, int top_k, float scale,
                                                      int* __restrict__ topk_idx, float* __restrict__ topk_w) {
    constexpr int kExperts = 32 * kPerLane;
    const int lane = threadIdx.x & 31;
    const int token = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (token >= tokens) return;
    float sig[kPerLane], wb[kPerLane];
    const float* row = logits + static_cast<long long>(token) * kExperts + lane * kPerLane;
#pragma unroll
    for (int j = 0; j < kPerLane; ++j) {
        const float s = 1.0f / (1.0f + expf(-row[j]));
        sig[j] = s;
        wb[j] = s + (bias ? bias[lane * kPerLane + j] : 0.0f);
    }
    // the two largest biased scores of this lane's experts, then of its group (duplicates count twice)
    float a = -FLT_MAX, b = -FLT_MAX;
#pragma unroll
    for (int j = 0; j < kPerLane; ++j) {
        const float v = wb[j];
        if (v > a) {
            b = a;
            a = v;
        } else if (v > b) {
            b = v;
        }
    }
    const int group_size = kExperts / n_group;
    const int lanes_per_group = group_size / kPerLane;
    for (int off = 1; off < lanes_per_group; off <<= 1) {
        const float oa = __shfl_xor_sync(0xffffffffu, a, off);
        const float ob = __shfl_xor_sync(0xffffffffu, b, off);
        if (a >= oa) {
            b = fmaxf(b, oa);
        } else {
            b = fmaxf(ob, a);
            a = oa;
        }
    }
    const float total = group_size >= 2 ? a + b : a;
    // lane g ranks group g, whose lanes start at g * lanes_per_group
    float gscore = __shfl_sync(0xffffffffu, total, (lane < n_group ? lane : 0) * lanes_per_group);
    if (lane >= n_group) gscore = -FLT_MAX;
    uint32_t group_mask = 0;
    for (int r = 0; r < topk_group; ++r) {
        float v = gscore;
        int g = lane;
        warp_argmax(v, g);
        group_mask |= 1u << g;
        if (lane == g) gscore = -FLT_MAX;
    }
    if (!((group_mask >> (lane / lanes_per_group)) & 1u)) {
#pragma unroll
        for (int j = 0; j < kPerLane; ++j) wb[j] = -FLT_MAX;    // like the reference's finfo.min fill
    }
    float wsum = 0.0f, my_w = 0.0f;
    int my_e = 0;
    for (int r = 0; r < top_k; ++r) {
        float v = wb[0];
        int best = lane * kPerLane;
#pragma unroll
        for (int j = 1; j < kPerLane; ++j)
            if (wb[j] > v) {
                v = wb[j];
                best = lane * kPerLane + j;
            }
        warp_argmax(v, best);
        const int owner = best / kPerLane, bj = best % kPerLane;
        float s = 0.0f;
#pragma unroll
        for (int j = 0; j < kPerLane; ++j)
            if (j == bj) {
                s = sig[j];
                if (lane == owner) wb[j] = -INFINITY;    // taken
            }
        s = __shfl_sync(0xffffffffu, s, owner);
        wsum += s;
        if (lane == r) {
            my_e = best;
            my_w = s;
        }
    }
    if (lane < top_k) {
        topk_idx[static_cast<long long>(token) * top_k + lane] = my_e;
        topk_w[static_cast<long long>(token) * top_k + lane] = my_w / (wsum + 1e-20f) * scale;
    }
}

// Counting sort, step 1: block b counts the experts of entries [b * kMoeChunk, (b + 1) * kMoeChunk).
__global__ void __launch_bounds__(kMoeChunk) moe_count(const int* __restrict__ topk_idx, int entries, int experts,
                                                       int* __restrict__ block_counts) {
    __shared__ int hist[kMoeMaxExperts];
    for (int e = threadIdx.x; e < experts; e += blockDim.x) hist[e] = 0;
    __syncthreads();
    const int i = blockIdx.x * kMoeChunk + threadIdx.x;
    if (i < entries) {
        const int e = topk_idx[i];
        if (static_cast<unsigned>(e) < static_cast<unsigned>(experts)) atomicAdd(&hist[e], 1);   // ids out of range are dropped
    }
    __syncthreads();
    for (int e = threadIdx.x; e < experts; e += blockDim.x) block_counts[blockIdx.x * experts + e] = hist[e];
}

// Step 2 (one block): per expert the exclusive prefix over the blocks, then over the experts the row
// ranges (rows of expert e are [row_offsets[e], row_offsets[e + 1])) and the 128-row scale-factor
// atoms before each expert (every expert's scale factors start on an atom boundary).
__global__ void __launch_bounds__(kMoeMaxExperts) moe_scan(int* __restrict__ block_counts, int blocks, int experts,
                                                           int* __restrict__ counts, int* __restrict__ row_offsets,
                                                           int* __restrict__ sfa_atom_offsets) {
    __shared__ int total[kMoeMaxExperts];
    const int e = threadIdx.x;
    if (e < experts) {
        int run = 0;
        // sixteen independent loads per trip: one dependent load per block made this kernel 20 us long
        for (int b0 = 0; b0 < blocks; b0 += 16) {
            int c[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) c[i] = (b0 + i < blocks) ? block_counts[(b0 + i) * experts + e] : 0;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                if (b0 + i < blocks) block_counts[(b0 + i) * experts + e] = run;   // the block's base inside the expert
                run += c[i];
            }
        }
        total[e] = run;
        counts[e] = run;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int rows = 0, atoms = 0;
        for (int i = 0; i < experts; ++i) {
            row_offsets[i] = rows;
            sfa_atom_offsets[i] = atoms;
            rows += total[i];
            atoms += (total[i] + 127) / 128;
        }
        row_offsets[experts] = rows;
        sfa_atom_offsets[experts] = atoms;
    }
}

// Step 3: every entry finds its row: expert's first row + entries of the same expert in earlier
// blocks + in earlier warps of this block + in earlier lanes of this warp (stable in entry order,
// so an expert's rows are in token order like the reference's nonzero(), moe_fibench_ref.py:144-149).
__global__ void __launch_bounds__(kMoeChunk) moe_place(const int* __restrict__ topk_idx, int entries, int experts,
                                                       int top_k, const int* __restrict__ block_base,
                                                       const int* __restrict__ row_offsets, int* __restrict__ row_of,
                                                       int* __restrict__ src_token) {
    __shared__ int warp_cnt[kMoeChunk / 32][kMoeMaxExperts];
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    for (int j = threadIdx.x; j < (kMoeChunk / 32) * kMoeMaxExperts; j += blockDim.x) (&warp_cnt[0][0])[j] = 0;
    __syncthreads();
    const int i = blockIdx.x * kMoeChunk + threadIdx.x;
    int e = i < entries ? topk_idx[i] : -1;
    const bool live = static_cast<unsigned>(e) < static_cast<unsigned>(experts);   // ids out of range get no row
    if (!live) e = -1 - lane;                                   // dead lanes match nobody
    const uint32_t same = __match_any_sync(0xffffffffu, e);
    const int rank_in_warp = __popc(same & ((1u << lane) - 1u));
    if (live && rank_in_warp == 0) warp_cnt[wib][e] = __popc(same);
    __syncthreads();
    if (live) {
        int before = 0;
        for (int w = 0; w < wib; ++w) before += warp_cnt[w][e];
        const int row = row_offsets[e] + block_base[blockIdx.x * experts + e] + before + rank_in_warp;
        row_of[i] = row;
        src_token[row] = i / top_k;
    }
}

// Dynamic fields of the grouped GEMM's descriptor table (the tensor maps, B-side pointers and
// shapes were uploaded by the host): one thread per expert, then one thread numbers the tiles.
__global__ void __launch_bounds__(kMoeMaxExperts) moe_fill_group_table(GroupEntry* __restrict__ table, int experts,
                                                                       const int* __restrict__ counts,
                                                                       const int* __restrict__ row_offsets,
                                                                       const int* __restrict__ sfa_atom_offsets,
                                                                       const uint8_t* sfa_all, __half* y_all, int n, int k,
                                                                       int rows_per_tile, int* __restrict__ total_tiles) {
    __shared__ int tiles[kMoeMaxExperts];
    const int e = threadIdx.x;
    if (e < experts) {
        GroupEntry& g = table[e];
        const int m = counts[e];
        g.m = m;
        g.m_tiles = (m + rows_per_tile - 1) / rows_per_tile;
        g.a_row0 = row_offsets[e];
        g.sfa = sfa_all + static_cast<long long>(sfa_atom_offsets[e]) * (k / 64) * 512;
        g.c = y_all + static_cast<long long>(row_offsets[e]) * n;
        tiles[e] = g.m_tiles * g.n_tiles;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int i = 0; i < experts; ++i) {
            table[i].tile_begin = run;
            run += tiles[i];
        }
        *total_tiles = run;
    }
}

// Step 1 of the gather: every token row is quantised once, like nvfp4_quantize does (same block
// arithmetic), into a scratch copy: packed e2m1 [tokens, k/2] and its scale factors ROW-MAJOR
// [tokens, k/16], so that a row's scale factors are contiguous for step 2.  One lane owns one
// 16-element block, a warp a 512-k stretch of one row.
template <int kDtype>
__global__ void __launch_bounds__(256) moe_quantize_rows(const uint16_t* __restrict__ x, long long ldx, int tokens, int k,
                                                         uint8_t* __restrict__ q, uint8_t* __restrict__ sf_rows) {
    const int lane = threadIdx.x & 31;
    const int blocks_per_row = k / 16;
    const int chunks_per_row = (blocks_per_row + 31) / 32;
    const long long warps = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
    const long long items = static_cast<long long>(tokens) * chunks_per_row;
    for (long long item = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); item < items;
         item += warps) {
        const int row = static_cast<int>(item / chunks_per_row);
        const int kb = static_cast<int>(item % chunks_per_row) * 32 + lane;       // 16-k block of this lane
        if (kb < blocks_per_row) {
            const uint16_t* src = x + static_cast<long long>(row) * ldx + kb * 16;
            const uint4 a = __ldg(reinterpret_cast<const uint4*>(src));
            const uint4 b = __ldg(reinterpret_cast<const uint4*>(src) + 1);
            uint2 packed;
            const uint32_t sbyte = quantize_block<kDtype>(a, b, packed);
            *reinterpret_cast<uint2*>(q + static_cast<long long>(row) * (k / 2) + kb * 8) = packed;
            sf_rows[static_cast<long long>(row) * blocks_per_row + kb] = static_cast<uint8_t>(sbyte);
        }
    }
}

// Step 2: row r of the permuted order = quantised row src_token[r] (quantisation is per row, so
// this equals quantising the gathered rows).  One warp per row copies its k/2 packed bytes in
// 16-byte pieces and scatters its k/16 scale bytes, four at a time, into its expert's atoms.  The
// quantised activations (tokens * k * 9/16 bytes) stay in the L2 while every row is read top_k times.
__global__ void __launch_bounds__(256) moe_gather_rows(const uint8_t* __restrict__ q, const uint8_t* __restrict__ sf_rows,
                                                       const int* __restrict__ src_token,
                                                       const int* __restrict__ row_offsets,
                                                       const int* __restrict__ sfa_atom_offsets, int experts, int k,
                                                       uint8_t* __restrict__ a_q, uint8_t* __restrict__ sfa_all) {
    const int lane = threadIdx.x & 31;
    const int total_rows = row_offsets[experts];
    const int row_bytes = k / 2, sf_words = k / 64, rest_k = k / 64;
    const long long warps = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
    for (long long row = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); row < total_rows;
         row += warps) {
        // expert of the row: last e with row_offsets[e] <= row
        int lo = 0, hi = experts;
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (row_offsets[mid] <= row) lo = mid;
            else hi = mid;
        }
        const int local = static_cast<int>(row) - row_offsets[lo];
        const long long token = src_token[row];
        const uint4* src = reinterpret_cast<const uint4*>(q + token * row_bytes);
        uint4* dst = reinterpret_cast<uint4*>(a_q + row * row_bytes);
        for (int i = lane; i < row_bytes / 16; i += 32) dst[i] = __ldg(src + i);
        const uint32_t* sf_src = reinterpret_cast<const uint32_t*>(sf_rows + token * (k / 16));
        uint8_t* sf_dst = sfa_all + (static_cast<long long>(sfa_atom_offsets[lo] + local / 128) * rest_k) * 512 +
                          (local % 32) * 16 + ((local % 128) / 32) * 4;
        for (int j = lane; j < sf_words; j += 32)     // word j = the four scale factors of 64-k block j
            *reinterpret_cast<uint32_t*>(sf_dst + static_cast<long long>(j) * 512) = __ldg(sf_src + j);
    }
}

// Both steps in one pass from the token's side: one warp per token reads the token's row once,
// quantises it 16 values per lane and writes every 16-k block straight to the token's top_k rows of the
// permuted order (and its scale factors to those rows' places in their experts' atoms).  The token's
// 2 * k bytes are read once and nothing goes through an intermediate buffer: tokens * k * (2 + top_k *
// 9/16) bytes in all.  Lane s < top_k looks up slot s once (row, expert by bisection of the row ranges,
// byte addresses); the loop over the row's blocks broadcasts them.
template <int kDtype>
__global__ void __launch_bounds__(256) moe_quantize_scatter(const uint16_t* __restrict__ x, long long ldx, int tokens, int k,
                                                            const int* __restrict__ row_of,
                                                            const int* __restrict__ row_offsets,
                                                            const int* __restrict__ sfa_atom_offsets, int experts, int top_k,
                                                            uint8_t* __restrict__ a_q, uint8_t* __restrict__ sfa_all) {
    const int lane = threadIdx.x & 31;
    const int blocks_per_row = k / 16, rest_k = k / 64;
    const long long warps = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
    // kMoeScatterSplit warps share a token (every kMoeScatterSplit-th run of 32 blocks each): more loads in flight
    const long long items = static_cast<long long>(tokens) * kMoeScatterSplit;
    for (long long item = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); item < items;
         item += warps) {
        const long long token = item / kMoeScatterSplit;
        const int part = static_cast<int>(item % kMoeScatterSplit);
        unsigned long long q_dst = 0, sf_dst = 0;      // of slot `lane`
        if (lane < top_k) {
            const int row = row_of[token * top_k + lane];
            int lo = 0, hi = experts;                   // expert of the row: last e with row_offsets[e] <= row
            while (hi - lo > 1) {
                const int mid = (lo + hi) >> 1;
                if (row_offsets[mid] <= row) lo = mid;
                else hi = mid;
            }
            const int local = row - row_offsets[lo];
            q_dst = reinterpret_cast<unsigned long long>(a_q + static_cast<long long>(row) * (k / 2));
            sf_dst = reinterpret_cast<unsigned long long>(
                sfa_all + (static_cast<long long>(sfa_atom_offsets[lo] + local / 128) * rest_k) * 512 + (local % 32) * 16 +
                ((local % 128) / 32) * 4);
        }
        const uint16_t* src_row = x + token * ldx;
        for (int kb = part * 32 + lane; kb - lane < blocks_per_row; kb += 32 * kMoeScatterSplit) {   // whole warps loop
            const bool real = kb < blocks_per_row;
            uint2 packed = make_uint2(0u, 0u);
            uint32_t sbyte = 0;
            if (real) {
                const uint4 a = __ldg(reinterpret_cast<const uint4*>(src_row + kb * 16));
                const uint4 b = __ldg(reinterpret_cast<const uint4*>(src_row + kb * 16) + 1);
                sbyte = quantize_block<kDtype>(a, b, packed);
            }
            // four consecutive 16-k blocks of a row are one 32-bit word of the scale-factor layout
            uint32_t word = sbyte;
            word |= __shfl_down_sync(0xffffffffu, sbyte, 1) << 8;
            word |= __shfl_down_sync(0xffffffffu, sbyte, 2) << 16;
            word |= __shfl_down_sync(0xffffffffu, sbyte, 3) << 24;
            for (int s = 0; s < top_k; ++s) {
                const unsigned long long qd = __shfl_sync(0xffffffffu, q_dst, s);
                const unsigned long long sd = __shfl_sync(0xffffffffu, sf_dst, s);
                if (real) {
                    *reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(qd) + kb * 8) = packed;
                    if ((lane & 3) == 0)
                        *reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(sd) + static_cast<long long>(kb >> 2) * 512) = word;
                }
            }
        }
    }
}

// out[t, :] = sum over the token's slots of weight * y[row, :] in fp32, stored as fp16 or bf16
// (moe/moe_fibench_ref.py:172-176 accumulates the same products with index_add_).  One block per
// token; a thread owns eight consecutive columns (one 16-byte load per slot).
template <int kOutDtype>
__global__ void __launch_bounds__(256) moe_combine(const __half* __restrict__ y, int n, const int* __restrict__ row_of,
                                                   const float* __restrict__ topk_w, int top_k, uint16_t* __restrict__ out,
                                                   long long ldo) {
    const int token = blockIdx.x;
    for (int col = threadIdx.x * 8; col < n; col += blockDim.x * 8) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int s = 0; s < top_k; ++s) {
            const int row = row_of[static_cast<long long>(token) * top_k + s];
            const float w = topk_w[static_cast<long long>(token) * top_k + s];
            const uint4 v = __ldg(reinterpret_cast<const uint4*>(y + static_cast<long long>(row) * n + col));
            const uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const __half2 h = *reinterpret_cast<const __half2*>(&words[i]);
                acc[2 * i] = fmaf(w, __low2float(h), acc[2 * i]);
                acc[2 * i + 1] = fmaf(w, __high2float(h), acc[2 * i + 1]);
            }
        }
        uint32_t packed[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (kOutDtype == kQuantDtypeF16) {
                const __half2 h = __floats2half2_rn(acc[2 * i], acc[2 * i + 1]);
                packed[i] = *reinterpret_cast<const uint32_t*>(&h);
            } else {
                const __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
                packed[i] = *reinterpret_cast<const uint32_t*>(&h);
            }
        }
        *reinterpret_cast<uint4*>(out + static_cast<long long>(token) * ldo + col) =
            make_uint4(packed[0], packed[1], packed[2], packed[3]);
    }
}

}  // namespace b200
