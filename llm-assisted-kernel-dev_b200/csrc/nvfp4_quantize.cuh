// Activation quantiser: fp16 / bf16 [rows, k] -> NVFP4 (packed e2m1, low nibble = even k)
// plus one e4m3 scale factor per 16 consecutive k, written straight into the
// (rest_mn, rest_k, 32, 4, 4) byte layout the GEMM kernels read.  The step before the
// GEMMs in a real FFN; the reference has no counterpart (it draws pre-quantised
// operands, dual_gemm/reference.py:114-190).
//
//   s = e4m3_rn_satfinite(max|x| / 6)                     per 16 k
//   q = e2m1_rn_even_satfinite(x * fp32(1 / float(s)))    (all zero when s == 0)
// (one correctly rounded reciprocal per block and a multiply per element: sixteen IEEE
// divisions per block made the kernel issue-bound at 43 % of the HBM rate)
//
// HBM-bound: 2 bytes read, 0.5625 bytes written per element.  One lane owns one
// 16-element block (two 16-byte loads, one 8-byte store), a warp a 512-k stretch of one
// row, so loads and stores of a warp are contiguous; the four scale bytes that share a
// 32-bit word of the layout are gathered with shuffles and stored by one lane.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdint>

namespace b200 {

constexpr int kQuantDtypeF16 = 0;
constexpr int kQuantDtypeBF16 = 1;

// two floats -> one byte of two e2m1 codes (`lo` in the low nibble)
__device__ __forceinline__ uint32_t cvt_e2m1x2(float lo, float hi) {
    uint32_t r;
    asm("{\n\t"
        ".reg .b8 t;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 t, %1, %2;\n\t"
        "cvt.u32.u8 %0, t;\n\t"
        "}\n"
        : "=r"(r)
        : "f"(hi), "f"(lo));
    return r;
}
// float -> e4m3fn byte (round to nearest even, saturating at 448)
__device__ __forceinline__ uint32_t cvt_e4m3(float v) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(0.0f), "f"(v));
    return static_cast<uint32_t>(r) & 0xffu;
}
// e4m3fn byte -> float
__device__ __forceinline__ float e4m3_to_float(uint32_t byte) {
    uint32_t h2;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(static_cast<uint16_t>(byte)));
    return __half2float(__ushort_as_half(static_cast<unsigned short>(h2 & 0xffffu)));
}

template <int kDtype> __device__ __forceinline__ void unpack16(const uint4& a, const uint4& b, float (&v)[16]) {
    const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        if (kDtype == kQuantDtypeF16) {
            const __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
            v[2 * i] = __low2float(h);
            v[2 * i + 1] = __high2float(h);
        } else {
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
}

// 32 bytes in one load (sixteen 16-bit inputs of one scale-factor block); the address
// must be 32-byte aligned
__device__ __forceinline__ void ld_global_nc_32B(const void* p, uint4& a, uint4& b) {
    asm volatile("ld.global.nc.L1::no_allocate.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w), "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w)
                 : "l"(p));
}

template <int kDtype>
__device__ __forceinline__ uint32_t quantize_block(const uint4& a, const uint4& b, uint2& packed) {
    float v[16];
    unpack16<kDtype>(a, b, v);
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
    const uint32_t sbyte = cvt_e4m3(__fdiv_rn(amax, 6.0f));
    const float s = e4m3_to_float(sbyte);
    uint32_t lo = 0, hi = 0;
    if (s > 0.0f) {
        const float r = __frcp_rn(s);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            lo |= cvt_e2m1x2(__fmul_rn(v[2 * i], r), __fmul_rn(v[2 * i + 1], r)) << (8 * i);
            hi |= cvt_e2m1x2(__fmul_rn(v[8 + 2 * i], r), __fmul_rn(v[9 + 2 * i], r)) << (8 * i);
        }
    }
    packed = make_uint2(lo, hi);
    return sbyte;
}

// x: [rows, k] with row pitch ldx (elements); q: [rows, k/2] bytes; sf: the permuted
// scale-factor buffer of ceil(rows/128) x (k/64) atoms of 512 bytes.  Rows of the last
// 128-row block that lie past `rows` get zero scale factors.  A warp takes kUnroll
// 512-k stretches per trip and issues all their loads before any arithmetic.  kWide:
// x and its row pitch are 32-byte aligned, so a block is fetched with one 32-byte load.
template <int kDtype, bool kWide>
__global__ void __launch_bounds__(256) nvfp4_quantize(const uint16_t* __restrict__ x, long long ldx,
                                                      uint8_t* __restrict__ q, uint8_t* __restrict__ sf, int rows,
                                                      int k) {
    constexpr int kUnroll = 2;
    const int lane = threadIdx.x & 31;
    const int blocks_per_row = k / 16;                       // scale factors per row
    const int chunks_per_row = (blocks_per_row + 31) / 32;   // 512-k stretches
    const int rows_padded = (rows + 127) / 128 * 128;
    const int rest_k = k / 64;
    // (row, stretch) of a warp's work items advance by a fixed step: one division at entry
    // instead of one per item
    const int warps = static_cast<int>(gridDim.x * (blockDim.x >> 5));
    const int first = static_cast<int>(blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5));
    const int step_row = warps / chunks_per_row, step_c = warps % chunks_per_row;
    int cur_row = first / chunks_per_row, cur_c = first % chunks_per_row;
    while (cur_row < rows_padded) {
        uint4 a[kUnroll], b[kUnroll];
        int row[kUnroll], kb[kUnroll];
        bool live[kUnroll], real[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            row[u] = cur_row;
            kb[u] = cur_c * 32 + lane;   // 16-k block of this lane
            cur_row += step_row;
            cur_c += step_c;
            if (cur_c >= chunks_per_row) {
                cur_c -= chunks_per_row;
                ++cur_row;
            }
            live[u] = row[u] < rows_padded && kb[u] < blocks_per_row;
            real[u] = live[u] && row[u] < rows;
            if (real[u]) {
                const uint16_t* src = x + static_cast<long long>(row[u]) * ldx + kb[u] * 16;
                if (kWide) {
                    ld_global_nc_32B(src, a[u], b[u]);
                } else {
                    a[u] = __ldg(reinterpret_cast<const uint4*>(src));
                    b[u] = __ldg(reinterpret_cast<const uint4*>(src) + 1);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            uint32_t sbyte = 0;
            if (real[u]) {
                uint2 packed;
                sbyte = quantize_block<kDtype>(a[u], b[u], packed);
                *reinterpret_cast<uint2*>(q + static_cast<long long>(row[u]) * (k / 2) + kb[u] * 8) = packed;
            }
            // four consecutive 16-k blocks of a row are one 32-bit word of the layout
            uint32_t word = sbyte;
            word |= __shfl_down_sync(0xffffffffu, sbyte, 1) << 8;
            word |= __shfl_down_sync(0xffffffffu, sbyte, 2) << 16;
            word |= __shfl_down_sync(0xffffffffu, sbyte, 3) << 24;
            if (live[u] && (lane & 3) == 0) {
                const long long off = (static_cast<long long>(row[u] / 128) * rest_k + kb[u] / 4) * 512 +
                                      (row[u] % 32) * 16 + ((row[u] % 128) / 32) * 4;
                *reinterpret_cast<uint32_t*>(sf + off) = word;
            }
        }
    }
}

}  // namespace b200
