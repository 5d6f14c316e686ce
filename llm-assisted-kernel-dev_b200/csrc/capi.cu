// Host side of libb200nvfp4.so: argument validation, tensor-map encoding,
// launch configuration and the extern "C" entry points declared in
// include/b200_nvfp4.h.  No torch types, no allocation of caller-visible memory.
#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/b200_nvfp4.h"
#include "nvfp4_gemm_kernels.cuh"
#include "nvfp4_pair_kernels.cuh"
#include "nvfp4_quantize.cuh"
#include "moe_kernels.cuh"
#include "feed_probe.cuh"

namespace b200 {
namespace {

thread_local std::string t_last_error;
std::mutex g_mutex;
uint64_t g_launches = 0;
uint64_t g_epoch = 0;                  // split-k launches so far (their flag value)
const char* g_last_kernel = "";       // name of the kernel the last launch used

__device__ uint32_t g_device_status;   // library-owned status word (one per device)
__device__ unsigned long long g_device_cycles;   // clock64 span of CTA 0 of the last GEMM launch (one per device)

int fail(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    t_last_error = buf;
    return code;
}

int cuda_fail(cudaError_t e, const char* what) {
    return fail(static_cast<int>(e), "%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
}

#define B200_CUDA(expr)                                              \
    do {                                                             \
        cudaError_t e_ = (expr);                                     \
        if (e_ != cudaSuccess) return cuda_fail(e_, #expr);          \
    } while (0)

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// --------------------------------------------------------------------------
// Driver entry point for tensor-map encoding (no link-time libcuda dependency).
// --------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                   CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

int load_driver() {
    if (g_encode) return 0;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || fn == nullptr) {
        cudaGetLastError();
        return fail(B200_E_DRIVER, "cuTensorMapEncodeTiled is unavailable (no CUDA driver?)");
    }
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    return 0;
}

// Packed e2m1 operand [batches][rows][k/2] bytes -> 3-D map, box 128 B x box_rows rows,
// 128-byte swizzle, out-of-range rows read as zero.
int encode_operand_map(CUtensorMap* map, const void* base, int rows, int k, int batches,
                       long long batch_stride_bytes, unsigned box_rows = 128) {
    if (rows <= 0) rows = 1;   // empty group: never dereferenced, keep the encoder happy
    cuuint64_t dims[3] = {static_cast<cuuint64_t>(k / 2), static_cast<cuuint64_t>(rows),
                          static_cast<cuuint64_t>(batches)};
    cuuint64_t strides[2] = {static_cast<cuuint64_t>(k / 2), static_cast<cuuint64_t>(batch_stride_bytes)};
    cuuint32_t box[3] = {128, box_rows, 1};
    cuuint32_t elem[3] = {1, 1, 1};
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(B200_E_DRIVER, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return 0;
}

// fp16 output [batches][rows][ldc] -> 3-D map for TMA stores, box 64 columns x 32 rows
// (128 bytes wide, the 128-byte-swizzle limit).
int encode_output_map(CUtensorMap* map, void* base, int rows, int cols, int batches, long long ldc,
                      long long batch_stride) {
    cuuint64_t dims[3] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows),
                          static_cast<cuuint64_t>(batches)};
    cuuint64_t strides[2] = {static_cast<cuuint64_t>(ldc) * 2, static_cast<cuuint64_t>(batch_stride) * 2};
    cuuint32_t box[3] = {64, 32, 1};
    cuuint32_t elem[3] = {1, 1, 1};
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, base, dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(B200_E_DRIVER, "cuTensorMapEncodeTiled (output) failed with CUresult %d", (int)r);
    return 0;
}

// --------------------------------------------------------------------------
// Per-device state
// --------------------------------------------------------------------------
struct DeviceState {
    bool ready = false;
    int sm_count = 0;
    uint32_t* status = nullptr;
    unsigned long long* cycles = nullptr;
};
std::map<int, DeviceState> g_devices;

template <typename K> int opt_in_smem(K kernel, uint32_t bytes) {
    B200_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)));
    return 0;
}

constexpr int B200_VARIANT_LAST = B200_VARIANT_SELFTEST_LOST_LOAD;   // 6, 7: pair variants
static_assert(pair_smem_bytes<PairDual>() <= 227u * 1024u && pair_smem_bytes<PairDualNarrow>() <= 227u * 1024u,
              "shared memory budget of the pair kernels");
constexpr int kDualStages = 4;
constexpr int kG128Stages = 6;
constexpr int kG256Stages = 4;

// Padded to more than half of the SM's shared memory so that only one serial CTA
// (each allocates all 512 TMEM columns) is resident per SM.
template <Mode M> constexpr uint32_t smem_bytes_serial() {
    constexpr uint32_t need = 1024u + StageLayout<M>::kBytes + sizeof(ControlBlock);
    return need > 120u * 1024u ? need : 120u * 1024u;
}

int device_state(int device, DeviceState** out) {
    DeviceState& st = g_devices[device];
    if (!st.ready) {
        int rc = load_driver();
        if (rc) return rc;
        B200_CUDA(cudaDeviceGetAttribute(&st.sm_count, cudaDevAttrMultiProcessorCount, device));
        B200_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&st.status), g_device_status));
        B200_CUDA(cudaMemset(st.status, 0, sizeof(uint32_t)));
        B200_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&st.cycles), g_device_cycles));
        B200_CUDA(cudaMemset(st.cycles, 0, sizeof(unsigned long long)));
        if ((rc = opt_in_smem(nvfp4_gemm_persistent<Mode::Dual, kDualStages>,
                              smem_bytes_persistent<Mode::Dual, kDualStages>()))) return rc;
#ifdef B200_TIMING_PROBES
        if ((rc = opt_in_smem(nvfp4_gemm_persistent<Mode::Dual, kDualStages, true>,
                              smem_bytes_persistent<Mode::Dual, kDualStages>()))) return rc;
        if ((rc = opt_in_smem(nvfp4_gemm_pair<PairDual, true>, pair_smem_bytes<PairDual>()))) return rc;
        if ((rc = opt_in_smem(nvfp4_gemm_pair<PairDualNarrow, true>, pair_smem_bytes<PairDualNarrow>()))) return rc;
#endif
        if ((rc = opt_in_smem(nvfp4_gemm_persistent<Mode::Dual, kDualStages, false, true>,
                              smem_bytes_persistent<Mode::Dual, kDualStages>()))) return rc;
        if ((rc = opt_in_smem(nvfp4_gemm_persistent<Mode::Group128, kG128Stages>,
                              smem_bytes_persistent<Mode::Group128, kG128Stages>()))) return rc;
        if ((rc = opt_in_smem(nvfp4_gemm_persistent<Mode::Group256, kG256Stages>,
                              smem_bytes_persistent<Mode::Group256, kG256Stages>()))) return rc;
        if ((rc = opt_in_smem(nvfp4_gemm_pair<PairDual>, pair_smem_bytes<PairDual>()))) return rc;
        if ((rc = opt_in_smem(nvfp4_gemm_pair<PairDualStreamK>, pair_smem_bytes<PairDualStreamK>()))) return rc;
        if ((rc = opt_in_smem(nvfp4_gemm_pair<PairDualGather>, pair_smem_bytes<PairDualGather>()))) return rc;
        if ((rc = opt_in_smem(nvfp4_gemm_pair<PairDualNarrow>, pair_smem_bytes<PairDualNarrow>()))) return rc;
        if ((rc = opt_in_smem(nvfp4_gemm_pair<PairGrouped>, pair_smem_bytes<PairGrouped>()))) return rc;
        if ((rc = opt_in_smem(nvfp4_gemm_pair<PairGroupedShared>, pair_smem_bytes<PairGroupedShared>()))) return rc;
        if ((rc = opt_in_smem(nvfp4_gemm_pair<PairDualQuant>, pair_smem_bytes<PairDualQuant>()))) return rc;
        if ((rc = opt_in_smem(nvfp4_gemm_serial<Mode::Dual>, smem_bytes_serial<Mode::Dual>()))) return rc;
        if ((rc = opt_in_smem(nvfp4_gemm_serial<Mode::Group128>, smem_bytes_serial<Mode::Group128>()))) return rc;
        if ((rc = opt_in_smem(nvfp4_gemm_serial<Mode::Group256>, smem_bytes_serial<Mode::Group256>()))) return rc;
        st.ready = true;
    }
    *out = &st;
    return 0;
}

struct DeviceGuard {
    int prev = -1;
    bool switched = false;
    int enter(int device) {
        B200_CUDA(cudaGetDevice(&prev));
        if (prev != device) {
            B200_CUDA(cudaSetDevice(device));
            switched = true;
        }
        return 0;
    }
    ~DeviceGuard() {
        if (switched) cudaSetDevice(prev);
    }
};

// --------------------------------------------------------------------------
// Dual GEMM
// --------------------------------------------------------------------------
struct DualKey {
    const void *a, *b1, *b2, *c;
    int m, n, k, l, device;
    long long b_batch, ldc, c_batch;
    bool quant;   // quantised-output call: `c` is the packed output and the entry holds no fp16 store map
    bool operator==(const DualKey& o) const {
        return a == o.a && b1 == o.b1 && b2 == o.b2 && c == o.c && m == o.m && n == o.n && k == o.k && l == o.l &&
               device == o.device && b_batch == o.b_batch && ldc == o.ldc && c_batch == o.c_batch &&
               quant == o.quant;
    }
};
struct DualMaps {
    DualKey key;
    CUtensorMap a, b1, b2, c;
    CUtensorMap b1n, b2n;     // 64-row boxes, encoded on first use by the narrow pair kernel
    bool has_narrow;
};
std::vector<DualMaps> g_dual_cache;   // small most-recently-used list

int validate_dual(const void* a, const void* b1, const void* b2, const void* sfa, const void* sfb1,
                  const void* sfb2, const void* c, int m, int n, int k, int l, long long ldc, long long c_batch,
                  long long b_batch, long long sfb_batch) {
    if (!a || !b1 || !b2 || !sfa || !sfb1 || !sfb2 || !c) return fail(B200_E_NULL, "dual gemm: NULL tensor pointer");
    if (m <= 0 || n <= 0 || k <= 0 || l <= 0)
        return fail(B200_E_SHAPE, "dual gemm: m, n, k, l must be positive (got %d %d %d %d)", m, n, k, l);
    if (m % 128) return fail(B200_E_SHAPE, "dual gemm: m=%d is not a multiple of 128", m);
    if (n % 128) return fail(B200_E_SHAPE, "dual gemm: n=%d is not a multiple of 128", n);
    if (k % 256) return fail(B200_E_SHAPE, "dual gemm: k=%d is not a multiple of 256", k);
    if (ldc < n || ldc % 8) return fail(B200_E_ALIGN, "dual gemm: ldc=%lld must be >= n and a multiple of 8", ldc);
    if (c_batch % 8 || b_batch % 16 || sfb_batch % 16)
        return fail(B200_E_ALIGN, "dual gemm: batch strides must keep 16-byte alignment");
    if (!aligned16(a) || !aligned16(b1) || !aligned16(b2) || !aligned16(sfa) || !aligned16(sfb1) ||
        !aligned16(sfb2) || !aligned16(c))
        return fail(B200_E_ALIGN, "dual gemm: every tensor pointer must be 16-byte aligned");
    return 0;
}

// Split-k factor for a dual GEMM with `tiles` output tiles of `k_tiles` k-tiles on
// `sms` SMs: as many units as fit in one wave, at least four k-tiles per unit.
int split_count(int tiles, int k_tiles, int sms) {
    if (tiles * 2 > sms) return 1;
    int s = sms / tiles;
    if (s > k_tiles / 4) s = k_tiles / 4;
    if (s > 8) s = 8;
    // every unit must own at least one k-tile when the range is cut into ceil(k_tiles / s) pieces
    while (s > 1 && (s - 1) * ((k_tiles + s - 1) / s) >= k_tiles) --s;
    return s < 1 ? 1 : s;
}
// Pair tiles that go into the stream-k tail of a dual GEMM with `pair_tiles` 256 x 128 tiles of
// `k_tiles` k-tiles on `pairs` CTA pairs: one round plus the remainder, when dealing whole tiles
// would leave the last round under-filled (0 = whole tiles only).  `force` skips the 3 % threshold.
int streamk_tiles(int pair_tiles, int k_tiles, int pairs, bool force) {
    if (pairs <= 0 || pair_tiles <= pairs || k_tiles < 2) return 0;
    const int rem = pair_tiles % pairs;
    if (rem == 0) return 0;
    const int full = pair_tiles / pairs;
    const double exact = static_cast<double>(pair_tiles) / pairs;
    if (!force && (full + 1 - exact) / exact < 0.03) return 0;
    return pairs + rem;
}
size_t streamk_flag_bytes(int pairs) { return (static_cast<size_t>(pairs) * kStreamKFlagWords * 4 + 255) & ~static_cast<size_t>(255); }
size_t streamk_bytes(int pairs) { return streamk_flag_bytes(pairs) + static_cast<size_t>(pairs) * kStreamKSlotFloats * 4; }
size_t splitk_bytes(size_t tiles, int splits);
size_t splitk_flag_bytes(size_t tiles) { return (tiles * 8 * sizeof(uint32_t) + 255) & ~static_cast<size_t>(255); }
// epoch words (eight per tile) followed by the fp32 partial sums
size_t splitk_bytes(size_t tiles, int splits) {
    return splits <= 1 ? 0 : splitk_flag_bytes(tiles) + tiles * splits * 128 * 256 * sizeof(float);
}

// Both GEMM kernels are launched with the programmatic-stream-serialization attribute: they signal
// `launch_dependents` on entry and wait for their predecessors (griddepcontrol.wait) before they touch
// global memory, so back-to-back launches overlap one kernel's set-up with the tail of the one before.
// `pdl` = false for a launch that directly follows a host-to-device copy it depends on.
template <Mode M, int kStages, typename P, bool kTimingProbes = false, bool kInjectLostLoad = false>
int launch_persistent(const P& prob, int units, int sm_count, int flags, cudaStream_t stream, bool pdl = true) {
    const int grid = units < sm_count ? units : sm_count;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(kPersistentThreads, 1, 1);
    cfg.dynamicSmemBytes = smem_bytes_persistent<M, kStages>();
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    B200_CUDA(cudaLaunchKernelEx(&cfg, nvfp4_gemm_persistent<M, kStages, kTimingProbes, kInjectLostLoad>, prob, flags));
    ++g_launches;
    g_last_kernel = M == Mode::Dual ? "nvfp4_gemm_persistent<Dual>"
                    : M == Mode::Group128 ? "nvfp4_gemm_persistent<Group128>" : "nvfp4_gemm_persistent<Group256>";
    return 0;
}

// CTA pairs: clusters of two CTAs, one pair per TPC, each pair walks pair tiles.
template <typename S, bool kTimingProbes = false>
int launch_pair(const typename S::Params& prob, int pair_tiles, int sm_count, int flags, cudaStream_t stream,
                bool pdl = true) {
    int pairs = sm_count / 2;
    if (pairs > pair_tiles) pairs = pair_tiles;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.gridDim = dim3(2 * pairs, 1, 1);
    cfg.blockDim = dim3(kPairThreads, 1, 1);
    cfg.dynamicSmemBytes = pair_smem_bytes<S>();
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 2 : 1;
    B200_CUDA(cudaLaunchKernelEx(&cfg, nvfp4_gemm_pair<S, kTimingProbes>, prob, flags));
    ++g_launches;
    g_last_kernel = S::kName;
    return 0;
}
int dual_pair_tiles(const DenseProblem& p) { return (p.m_tiles / 2) * p.n_tiles * p.batches; }

template <Mode M, typename P> int launch_serial(const P& prob, int units, int two_mma, cudaStream_t stream) {
    nvfp4_gemm_serial<M><<<units, 128, smem_bytes_serial<M>(), stream>>>(prob, two_mma);
    B200_CUDA(cudaGetLastError());
    ++g_launches;
    g_last_kernel = "nvfp4_gemm_serial";
    return 0;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

const char* b200_version(void) { return "b200nvfp4 0.1 (sm_100a)"; }

const char* b200_last_error(void) { return t_last_error.c_str(); }

uint64_t b200_launch_count(void) { return g_launches; }

const char* b200_last_kernel(void) { return g_last_kernel; }

size_t b200_dual_streamk_workspace_bytes(int m, int n, int k, int l) {
    if (m <= 0 || n <= 0 || k <= 0 || l <= 0 || m % 256 || n % 128 || k % 256) return 0;
    const long long pair_tiles = static_cast<long long>(m / 256) * (n / 128) * l;
    if (pair_tiles > 100000000) return 0;
    const int pairs = 148 / 2;
    return streamk_tiles(static_cast<int>(pair_tiles), k / 256, pairs, true) > 0 ? streamk_bytes(pairs) : 0;
}

size_t b200_dual_splitk_workspace_bytes(int m, int n, int k, int l) {
    if (m <= 0 || n <= 0 || k <= 0 || l <= 0 || m % 128 || n % 128 || k % 256) return 0;
    const size_t tiles = static_cast<size_t>(m / 128) * (n / 128) * l;
    const int splits = split_count(static_cast<int>(tiles > 1000000 ? 1000000 : tiles), k / 256, 148);
    return splitk_bytes(tiles, splits);
}

// Shared body of the dual-GEMM entry points.  q_out / sf_out non-NULL: the CTA-pair kernel
// writes the re-quantised result there instead of fp16 to c (c is then unused).
static int dual_gemm_impl(const void* a, const void* b1, const void* b2, const void* sfa, const void* sfb1,
                          const void* sfb2, void* c, int m, int n, int k, int l, int64_t ldc, int64_t c_batch,
                          int64_t b_batch_bytes, int64_t sfb_batch_bytes, int variant, void* workspace,
                          size_t workspace_bytes, void* stream, int device, uint32_t* status, void* q_out,
                          void* sf_out) {
    const bool quant = q_out != nullptr;
    if (c_batch == 0) c_batch = static_cast<int64_t>(m) * ldc;
    if (b_batch_bytes == 0) b_batch_bytes = static_cast<int64_t>(n) * (k / 2);
    if (sfb_batch_bytes == 0) sfb_batch_bytes = static_cast<int64_t>(n / 128) * (k / 64) * 512;
    int rc = validate_dual(a, b1, b2, sfa, sfb1, sfb2, c, m, n, k, l, ldc, c_batch, b_batch_bytes, sfb_batch_bytes);
    if (rc) return rc;
#ifdef B200_TIMING_PROBES
    // Instrumented build only: variant = kProbeBase + bits runs the one-CTA kernel, kProbeBase + 300 + bits
    // the CTA-pair kernel, with parts of the data path switched off (kFlag* bits; the output is then wrong by
    // design) and, given a 64 KiB workspace, a clock64 event log of CTA 0.
    constexpr int kProbeBase = 100;
    const bool probe = variant >= kProbeBase && variant < kProbeBase + 256;
    const bool pair_probe = variant >= kProbeBase + 300 && variant < kProbeBase + 556;
    const bool narrow_probe = variant >= kProbeBase + 600 && variant < kProbeBase + 856;
#else
    constexpr int kProbeBase = 0;
    constexpr bool probe = false, pair_probe = false, narrow_probe = false;
#endif
    if (!probe && !pair_probe && !narrow_probe && (variant < B200_VARIANT_AUTO || variant > B200_VARIANT_LAST))
        return fail(B200_E_VARIANT, "dual gemm: unknown variant %d", variant);

    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceGuard guard;
    if ((rc = guard.enter(device))) return rc;
    DeviceState* st = nullptr;
    if ((rc = device_state(device, &st))) return rc;

    DenseProblem p;
    memset(&p, 0, sizeof p);
    DualKey key{a, b1, b2, c, m, n, k, l, device, b_batch_bytes, ldc, c_batch, quant};
    DualMaps* maps = nullptr;
    for (DualMaps& e : g_dual_cache)
        if (e.key == key) { maps = &e; break; }
    if (!maps) {
        DualMaps fresh;
        memset(&fresh, 0, sizeof fresh);
        fresh.key = key;
        fresh.has_narrow = false;
        if ((rc = encode_operand_map(&fresh.a, a, m, k, l, static_cast<long long>(m) * (k / 2)))) return rc;
        if ((rc = encode_operand_map(&fresh.b1, b1, n, k, l, b_batch_bytes))) return rc;
        if ((rc = encode_operand_map(&fresh.b2, b2, n, k, l, b_batch_bytes))) return rc;
        if (!quant && (rc = encode_output_map(&fresh.c, c, m, n, l, ldc, c_batch))) return rc;
        if (g_dual_cache.size() >= 16) g_dual_cache.erase(g_dual_cache.begin());
        g_dual_cache.push_back(fresh);
        maps = &g_dual_cache.back();
    }
    p.map_a = maps->a;
    p.map_b1 = maps->b1;
    p.map_b2 = maps->b2;
    p.map_c = maps->c;
    p.sfa = static_cast<const uint8_t*>(sfa);
    p.sfb1 = static_cast<const uint8_t*>(sfb1);
    p.sfb2 = static_cast<const uint8_t*>(sfb2);
    p.c = static_cast<__half*>(c);
    p.q_out = static_cast<uint8_t*>(q_out);
    p.sf_out = static_cast<uint8_t*>(sf_out);
    p.ldc = ldc;
    p.c_batch = c_batch;
    p.sfa_batch = static_cast<long long>(m / 128) * (k / 64) * 512;
    p.sfb_batch = sfb_batch_bytes;
    p.m_tiles = m / 128;
    p.n_tiles = n / 128;
    p.k_tiles = k / 256;
    p.batches = l;
    p.total_tiles = p.m_tiles * p.n_tiles * l;
    p.sf_k_atoms = k / 64;
    p.k_splits = 1;
    p.status = status ? status : st->status;
    p.cycles = st->cycles;
    // timing probes: an optional 8 x 1024 x 8-byte event log for CTA 0
    p.trace = ((probe || pair_probe || narrow_probe) && workspace && workspace_bytes >= 8 * 1024 * sizeof(unsigned long long))
                  ? static_cast<unsigned long long*>(workspace) : nullptr;

    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (quant) return launch_pair<PairDualQuant>(p, dual_pair_tiles(p), st->sm_count, 0, s);
#ifdef B200_TIMING_PROBES
    if (probe)
        return launch_persistent<Mode::Dual, kDualStages, DenseProblem, true>(p, p.total_tiles, st->sm_count,
                                                                              variant - kProbeBase, s);
    if (pair_probe && p.m_tiles % 2 == 0)
        return launch_pair<PairDual, true>(p, dual_pair_tiles(p), st->sm_count, variant - kProbeBase - 300, s);
    if (narrow_probe && p.m_tiles % 2 == 0) {
        if ((rc = encode_operand_map(&p.map_b1n, b1, n, k, l, b_batch_bytes, 64))) return rc;
        if ((rc = encode_operand_map(&p.map_b2n, b2, n, k, l, b_batch_bytes, 64))) return rc;
        return launch_pair<PairDualNarrow, true>(p, p.total_tiles, st->sm_count, variant - kProbeBase - 600, s);
    }
#endif
    (void)kProbeBase;
    // Split-k only on request (B200_VARIANT_SPLITK): its partial-sum exchange through
    // global memory currently costs more than the idle SMs it puts to work.
    if (variant == B200_VARIANT_SPLITK) {
        const int splits = split_count(p.total_tiles, p.k_tiles, st->sm_count);
        const size_t need = splitk_bytes(static_cast<size_t>(p.total_tiles), splits);
        if (splits > 1 && workspace && workspace_bytes >= need && !(reinterpret_cast<uintptr_t>(workspace) & 255u)) {
            p.k_splits = splits;
            // any value no earlier launch has used; the workspace starts zero-filled
            p.splitk_epoch = static_cast<uint32_t>(++g_epoch);
            if (p.splitk_epoch == 0) p.splitk_epoch = static_cast<uint32_t>(++g_epoch);
            p.splitk_flags = static_cast<uint32_t*>(workspace);
            p.splitk_ws = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + splitk_flag_bytes(p.total_tiles));
        } else if (variant == B200_VARIANT_SPLITK && splits > 1) {
            return fail(B200_E_WORKSPACE, "dual gemm: split-k needs a 256-byte aligned workspace of %zu bytes", need);
        }
    }
    if (p.k_splits > 1)
        return launch_persistent<Mode::Dual, kDualStages>(p, p.total_tiles * p.k_splits, st->sm_count, 0, s);
    const bool wants_pair = variant == B200_VARIANT_PAIR || variant == B200_VARIANT_PAIR_NARROW ||
                            variant == B200_VARIANT_PAIR_STREAMK;
    if (wants_pair && p.m_tiles % 2)
        return fail(B200_E_SHAPE, "dual gemm: CTA pairs need m to be a multiple of 256 (m=%d)", m);
    // AUTO with row tiles that pair up: 256 x 64 tiles when that puts all of them into one round of the
    // GPU's CTA pairs (shapes with few tiles: twice as many SMs stream the operands), else 256 x 128 tiles.
    // Without pairing rows (m an odd multiple of 128) the one-CTA kernel runs.
    const int pairs_avail = st->sm_count / 2;
    const bool narrow = variant == B200_VARIANT_PAIR_NARROW ||
                        (variant == B200_VARIANT_AUTO && p.m_tiles % 2 == 0 && p.total_tiles <= pairs_avail);
    if (narrow) {
        if (!maps->has_narrow) {
            if ((rc = encode_operand_map(&maps->b1n, b1, n, k, l, b_batch_bytes, 64))) return rc;
            if ((rc = encode_operand_map(&maps->b2n, b2, n, k, l, b_batch_bytes, 64))) return rc;
            maps->has_narrow = true;
        }
        p.map_b1n = maps->b1n;
        p.map_b2n = maps->b2n;
        return launch_pair<PairDualNarrow>(p, p.total_tiles, st->sm_count, 0, s);
    }
    if (wants_pair || (variant == B200_VARIANT_AUTO && p.m_tiles % 2 == 0)) {
        // Stream-k tail: when whole tiles would leave the last round under-filled, the last round and the
        // remainder are cut along k so that every pair gets the same number of k-tiles.  Needs scratch.
        const int pair_tiles = dual_pair_tiles(p);
        const int pairs = pairs_avail < pair_tiles ? pairs_avail : pair_tiles;
        // Only on request: on a one-eighth column shard of the 8192 x 14336 x 4096 problem (448 tiles on 74
        // pairs) the cut version measured 62.7 us against 53.2 us for whole tiles; the extra tile
        // boundaries and the partial-sum reads at the very end cost more than the 0.95 round they save.
        const int sk = variant != B200_VARIANT_PAIR_STREAMK ? 0 : streamk_tiles(pair_tiles, p.k_tiles, pairs, true);
        if (sk > 0) {
            const size_t need = streamk_bytes(pairs);
            const bool usable = workspace && workspace_bytes >= need && !(reinterpret_cast<uintptr_t>(workspace) & 255u);
            if (usable) {
                p.sk_tiles = sk;
                p.splitk_epoch = static_cast<uint32_t>(++g_epoch);     // a value no earlier launch has used;
                if (p.splitk_epoch == 0) p.splitk_epoch = static_cast<uint32_t>(++g_epoch);   // the flags start at zero
                p.splitk_flags = static_cast<uint32_t*>(workspace);
                p.splitk_ws = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + streamk_flag_bytes(pairs));
            } else if (variant == B200_VARIANT_PAIR_STREAMK) {
                return fail(B200_E_WORKSPACE, "dual gemm: the stream-k tail needs a 256-byte aligned workspace of %zu bytes",
                            need);
            }
        }
        if (p.sk_tiles > 0) return launch_pair<PairDualStreamK>(p, pair_tiles, st->sm_count, 0, s);
        return launch_pair<PairDual>(p, pair_tiles, st->sm_count, 0, s);
    }
    switch (variant) {
        case B200_VARIANT_SERIAL:
            return launch_serial<Mode::Dual>(p, p.total_tiles, 0, s);
        case B200_VARIANT_SERIAL_2MMA:
            return launch_serial<Mode::Dual>(p, p.total_tiles, 1, s);
        case B200_VARIANT_SELFTEST_LOST_LOAD:
            // failure-detection self-test: the producer drops one k-tile's loads, the waits give up
            // after about a millisecond, the status word becomes non-zero and C stays unwritten
            return launch_persistent<Mode::Dual, kDualStages, DenseProblem, false, true>(p, p.total_tiles,
                                                                                         st->sm_count, 0, s);
        default:
            return launch_persistent<Mode::Dual, kDualStages>(p, p.total_tiles, st->sm_count, 0, s);
    }
}

int b200_dual_gemm_nvfp4_ex(const void* a, const void* b1, const void* b2, const void* sfa, const void* sfb1,
                            const void* sfb2, void* c, int m, int n, int k, int l, int64_t ldc, int64_t c_batch,
                            int64_t b_batch_bytes, int64_t sfb_batch_bytes, int variant, void* workspace,
                            size_t workspace_bytes, void* stream, int device, uint32_t* status) {
    return dual_gemm_impl(a, b1, b2, sfa, sfb1, sfb2, c, m, n, k, l, ldc, c_batch, b_batch_bytes, sfb_batch_bytes,
                          variant, workspace, workspace_bytes, stream, device, status, nullptr, nullptr);
}

int b200_dual_gemm_nvfp4_quant(const void* a, const void* b1, const void* b2, const void* sfa, const void* sfb1,
                               const void* sfb2, void* q, void* sf, int m, int n, int k, void* stream, int device,
                               uint32_t* status) {
    if (!q || !sf) return fail(B200_E_NULL, "dual gemm (quantised output): NULL output pointer");
    if (!aligned16(q) || !aligned16(sf))
        return fail(B200_E_ALIGN, "dual gemm (quantised output): output pointers must be 16-byte aligned");
    if (m > 0 && m % 256)
        return fail(B200_E_SHAPE, "dual gemm (quantised output): m=%d is not a multiple of 256 (CTA-pair kernel)", m);
    // `q` stands in for c in the shared argument checks (same alignment rule); it is never written as fp16
    return dual_gemm_impl(a, b1, b2, sfa, sfb1, sfb2, q, m, n, k, 1, n, 0, 0, 0, B200_VARIANT_AUTO, nullptr, 0, stream,
                          device, status, q, sf);
}

int b200_dual_gemm_nvfp4_gather(const void* a, const void* b1, const void* b2, const void* sfa, const void* sfb1,
                                const void* sfb2, void* const* c_ranks, int world, int rank, int m, int n_local, int n_total,
                                int col_offset, int k, void* stream, int device, uint32_t* status) {
    if (!c_ranks) return fail(B200_E_NULL, "dual gemm (gather): c_ranks is NULL");
    if (world < 1 || world > 8) return fail(B200_E_LIMIT, "dual gemm (gather): world=%d must be in 1..8", world);
    if (rank < 0 || rank >= world) return fail(B200_E_SHAPE, "dual gemm (gather): rank=%d is not in [0, %d)", rank, world);
    for (int r = 0; r < world; ++r) {
        if (!c_ranks[r]) return fail(B200_E_NULL, "dual gemm (gather): the C pointer of rank %d is NULL", r);
        if (!aligned16(c_ranks[r])) return fail(B200_E_ALIGN, "dual gemm (gather): the C pointer of rank %d is not 16-byte aligned", r);
    }
    if (m > 0 && m % 256) return fail(B200_E_SHAPE, "dual gemm (gather): m=%d is not a multiple of 256 (CTA-pair kernel)", m);
    if (n_total <= 0 || n_total % 128 || col_offset < 0 || col_offset % 128 || col_offset + n_local > n_total)
        return fail(B200_E_SHAPE, "dual gemm (gather): columns [%d, %d) do not fit a C of %d columns in 128-column steps",
                    col_offset, col_offset + n_local, n_total);
    int rc = validate_dual(a, b1, b2, sfa, sfb1, sfb2, c_ranks[rank], m, n_local, k, 1, n_total,
                           static_cast<long long>(m) * n_total, static_cast<long long>(n_local) * (k / 2),
                           static_cast<long long>(n_local / 128) * (k / 64) * 512);
    if (rc) return rc;
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceGuard guard;
    if ((rc = guard.enter(device))) return rc;
    DeviceState* st = nullptr;
    if ((rc = device_state(device, &st))) return rc;
    DenseProblem p;
    memset(&p, 0, sizeof p);
    // no cache: three operand maps and `world` output maps are encoded per call (a few microseconds)
    if ((rc = encode_operand_map(&p.map_a, a, m, k, 1, static_cast<long long>(m) * (k / 2)))) return rc;
    if ((rc = encode_operand_map(&p.map_b1, b1, n_local, k, 1, static_cast<long long>(n_local) * (k / 2)))) return rc;
    if ((rc = encode_operand_map(&p.map_b2, b2, n_local, k, 1, static_cast<long long>(n_local) * (k / 2)))) return rc;
    for (int r = 0; r < world; ++r)
        if ((rc = encode_output_map(&p.map_c_rank[r], c_ranks[r], m, n_total, 1, n_total, static_cast<long long>(m) * n_total)))
            return rc;
    p.map_c = p.map_c_rank[rank];
    p.gather_world = world;
    p.gather_col0 = col_offset;
    p.sfa = static_cast<const uint8_t*>(sfa);
    p.sfb1 = static_cast<const uint8_t*>(sfb1);
    p.sfb2 = static_cast<const uint8_t*>(sfb2);
    p.c = static_cast<__half*>(c_ranks[rank]);
    p.ldc = n_total;
    p.c_batch = static_cast<long long>(m) * n_total;
    p.sfa_batch = static_cast<long long>(m / 128) * (k / 64) * 512;
    p.sfb_batch = static_cast<long long>(n_local / 128) * (k / 64) * 512;
    p.m_tiles = m / 128;
    p.n_tiles = n_local / 128;
    p.k_tiles = k / 256;
    p.batches = 1;
    p.total_tiles = p.m_tiles * p.n_tiles;
    p.sf_k_atoms = k / 64;
    p.k_splits = 1;
    p.status = status ? status : st->status;
    p.cycles = st->cycles;
    return launch_pair<PairDualGather>(p, dual_pair_tiles(p), st->sm_count, 0, static_cast<cudaStream_t>(stream));
}

int b200_dual_gemm_nvfp4(const void* a, const void* b1, const void* b2, const void* sfa, const void* sfb1,
                         const void* sfb2, void* c, int m, int n, int k, int l, int64_t ldc, void* stream,
                         int device, uint32_t* status) {
    return b200_dual_gemm_nvfp4_ex(a, b1, b2, sfa, sfb1, sfb2, c, m, n, k, l, ldc, 0, 0, 0, B200_VARIANT_AUTO,
                                   nullptr, 0, stream, device, status);
}

size_t b200_grouped_workspace_bytes(int groups) {
    if (groups <= 0) return 0;
    return static_cast<size_t>(groups) * sizeof(GroupEntry);
}

}  // extern "C"

namespace b200 {
namespace {
constexpr int kTilingPair = -256;   // `tiling` value that selects 256 x 256 CTA-pair tiles

// Fills `table[0 .. groups)` for the given tiling (128 or 256 output columns per one-CTA
// tile, or kTilingPair) and returns the number of tiles through *total_tiles.
int build_group_table(GroupEntry* table, int groups, const void* const* a, const void* const* b,
                      const void* const* sfa, const void* const* sfb, void* const* c, const int* mnk, int tiling,
                      int* total_tiles) {
    memset(table, 0, static_cast<size_t>(groups) * sizeof(GroupEntry));
    const bool pair = tiling == kTilingPair;
    int tile_begin = 0, rc;
    for (int g = 0; g < groups; ++g) {
        const int m = mnk[3 * g], n = mnk[3 * g + 1], k = mnk[3 * g + 2];
        GroupEntry& e = table[g];
        e.m = m;
        e.n = n;
        e.k_tiles = k / 256;
        e.m_tiles = pair ? (m + 255) / 256 : (m + 127) / 128;
        e.n_tiles = pair ? n / 256 : (n + tiling - 1) / tiling;
        e.tile_begin = tile_begin;
        e.sf_k_atoms = k / 64;
        e.sfb_row_atoms = n / 128;
        e.ldc = n;
        tile_begin += e.m_tiles * e.n_tiles;
        if (m == 0) continue;
        e.sfa = static_cast<const uint8_t*>(sfa[g]);
        e.sfb = static_cast<const uint8_t*>(sfb[g]);
        e.c = static_cast<__half*>(c[g]);
        if ((rc = encode_operand_map(&e.map_a, a[g], m, k, 1, static_cast<long long>(m) * (k / 2)))) return rc;
        if ((rc = encode_operand_map(&e.map_b, b[g], n, k, 1, static_cast<long long>(n) * (k / 2)))) return rc;
        // the CTA-pair kernel stores through this map: its m rows are the extent, so rows of a tile past them are clipped
        if (pair && (rc = encode_output_map(&e.map_c, c[g], m, n, 1, n, static_cast<long long>(m) * n))) return rc;
    }
    *total_tiles = tile_begin;
    return 0;
}

// What the library last wrote to a given workspace address, so identical
// descriptor tables are not rebuilt or re-uploaded on every call.  An entry is
// only as good as the caller's promise not to touch the workspace in between:
// b200_grouped_workspace_forget() withdraws it (the Python wrapper calls that
// whenever a workspace changes hands).
struct WorkspaceImage {
    std::vector<uint8_t> key;       // raw call arguments
    int total_tiles = 0;
    int tile_n = 0;
    cudaEvent_t uploaded = nullptr;         // recorded behind the copy of the table
    std::vector<cudaStream_t> ordered;      // streams whose later work is ordered behind that copy
};
std::map<std::pair<int, const void*>, WorkspaceImage> g_workspaces;

void drop_workspace_images() {
    for (auto& kv : g_workspaces)
        if (kv.second.uploaded) cudaEventDestroy(kv.second.uploaded);
    g_workspaces.clear();
}

// The table copy of a grouped call has a host stack / heap source that dies when the
// call returns: under stream capture it would become a graph node that re-reads dead
// memory on every replay.  Such calls are refused.
int reject_capture(cudaStream_t s, const char* what) {
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    cudaError_t e = cudaStreamIsCapturing(s, &cs);
    if (e != cudaSuccess) return cuda_fail(e, "cudaStreamIsCapturing");
    if (cs != cudaStreamCaptureStatusNone)
        return fail(B200_E_CAPTURE,
                    "%s: the stream is being captured and this call has to upload its descriptor table or wait "
                    "for that upload; make the call once on this stream outside the capture first", what);
    return 0;
}
}  // namespace
}  // namespace b200

extern "C" {

int b200_grouped_gemm_nvfp4_ex(int groups, const void* const* a, const void* const* b, const void* const* sfa,
                               const void* const* sfb, void* const* c, const int* mnk, void* workspace,
                               size_t workspace_bytes, int variant, int tile_n, void* stream, int device,
                               uint32_t* status) {
    if (groups <= 0) return fail(B200_E_SHAPE, "grouped gemm: groups=%d must be positive", groups);
    if (!a || !b || !sfa || !sfb || !c || !mnk) return fail(B200_E_NULL, "grouped gemm: NULL argument array");
    if (variant != B200_VARIANT_AUTO && variant != B200_VARIANT_PERSISTENT && variant != B200_VARIANT_SERIAL &&
        variant != B200_VARIANT_PAIR)
        return fail(B200_E_VARIANT, "grouped gemm: unknown variant %d", variant);
    if (tile_n != 0 && tile_n != 128 && tile_n != 256)
        return fail(B200_E_VARIANT, "grouped gemm: tile_n=%d must be 0, 128 or 256", tile_n);
    bool all_n256 = true;
    long long tiles128 = 0, tiles256 = 0, pair_tiles = 0;
    for (int g = 0; g < groups; ++g) {
        const int m = mnk[3 * g], n = mnk[3 * g + 1], k = mnk[3 * g + 2];
        if (m < 0 || n <= 0 || k <= 0)
            return fail(B200_E_SHAPE, "grouped gemm: group %d has invalid shape (%d, %d, %d)", g, m, n, k);
        if (n % 128) return fail(B200_E_SHAPE, "grouped gemm: group %d n=%d is not a multiple of 128", g, n);
        if (k % 256) return fail(B200_E_SHAPE, "grouped gemm: group %d k=%d is not a multiple of 256", g, k);
        if (m == 0) continue;
        if (!a[g] || !b[g] || !sfa[g] || !sfb[g] || !c[g])
            return fail(B200_E_NULL, "grouped gemm: group %d has a NULL tensor pointer", g);
        if (!aligned16(a[g]) || !aligned16(b[g]) || !aligned16(sfa[g]) || !aligned16(sfb[g]) || !aligned16(c[g]))
            return fail(B200_E_ALIGN, "grouped gemm: group %d has a pointer that is not 16-byte aligned", g);
        if (n % 256) all_n256 = false;
        tiles128 += static_cast<long long>((m + 127) / 128) * (n / 128);
        tiles256 += static_cast<long long>((m + 127) / 128) * ((n + 255) / 256);
        pair_tiles += static_cast<long long>((m + 255) / 256) * (n / 256);
    }
    if (variant == B200_VARIANT_PAIR && !all_n256)
        return fail(B200_E_SHAPE, "grouped gemm: CTA pairs need every n to be a multiple of 256");
    if (!workspace) return fail(B200_E_WORKSPACE, "grouped gemm: workspace is NULL");
    if (reinterpret_cast<uintptr_t>(workspace) & 255u)
        return fail(B200_E_WORKSPACE, "grouped gemm: workspace must be 256-byte aligned");
    if (workspace_bytes < b200_grouped_workspace_bytes(groups))
        return fail(B200_E_WORKSPACE, "grouped gemm: workspace has %zu bytes, %zu needed", workspace_bytes,
                    b200_grouped_workspace_bytes(groups));
    if (tiles128 == 0) return 0;   // every group is empty: nothing to do

    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceGuard guard;
    int rc;
    if ((rc = guard.enter(device))) return rc;
    DeviceState* st = nullptr;
    if ((rc = device_state(device, &st))) return rc;

    // The library's choice: the tiling with the fewest rounds x cycles per k-tile.  Measured k-tile
    // cadences on a B200: 128 x 128 tiles ~750 cycles, 128 x 256 tiles ~1000, 256 x 256 pair tiles ~700
    // (all k-tiles of a list are equally long in the shapes this path serves, so rounds stand for time).
    const bool tile_n_chosen_here = tile_n == 0;
    bool use_pair = variant == B200_VARIANT_PAIR;
    if (tile_n == 0) {
        const long long sms = st->sm_count, pairs = st->sm_count / 2;
        const long long cost128 = (tiles128 + sms - 1) / sms * 750;
        const long long cost256 = all_n256 ? (tiles256 + sms - 1) / sms * 1000 : (1LL << 60);
        const long long cost_pair = all_n256 && variant == B200_VARIANT_AUTO ? (pair_tiles + pairs - 1) / pairs * 700 : (1LL << 60);
        tile_n = cost256 < cost128 ? 256 : 128;
        if (cost_pair <= cost128 && cost_pair <= cost256) use_pair = true;
    }
    (void)tile_n_chosen_here;
    if (use_pair) tile_n = kTilingPair;   // marks the pair tiling in the cache key and the table

    std::vector<uint8_t> key(sizeof(int) * 2 + groups * (5 * sizeof(void*) + 3 * sizeof(int)));
    {
        uint8_t* w = key.data();
        auto put = [&w](const void* src, size_t nbytes) { memcpy(w, src, nbytes); w += nbytes; };
        put(&groups, sizeof(int));
        put(&tile_n, sizeof(int));
        put(a, groups * sizeof(void*));
        put(b, groups * sizeof(void*));
        put(sfa, groups * sizeof(void*));
        put(sfb, groups * sizeof(void*));
        put(c, groups * sizeof(void*));
        put(mnk, groups * 3 * sizeof(int));
    }
    if (g_workspaces.size() > 256 && !g_workspaces.count({device, workspace})) drop_workspace_images();
    WorkspaceImage& img = g_workspaces[{device, workspace}];
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool uploads = img.key != key;
    if (img.key != key) {
        if ((rc = reject_capture(s, "grouped gemm"))) return rc;
        std::vector<GroupEntry> table(groups);
        int total = 0;
        if ((rc = build_group_table(table.data(), groups, a, b, sfa, sfb, c, mnk, tile_n, &total)))
            return rc;
        // Pageable source: the runtime stages the bytes before returning, so
        // `table` may go out of scope while the copy is still queued.
        img.key.clear();   // if anything below fails the entry must not look valid
        B200_CUDA(cudaMemcpyAsync(workspace, table.data(), groups * sizeof(GroupEntry), cudaMemcpyHostToDevice, s));
        if (!img.uploaded) B200_CUDA(cudaEventCreateWithFlags(&img.uploaded, cudaEventDisableTiming));
        B200_CUDA(cudaEventRecord(img.uploaded, s));
        img.ordered.assign(1, s);
        img.key = key;
        img.total_tiles = total;
        img.tile_n = tile_n;
    } else if (std::find(img.ordered.begin(), img.ordered.end(), s) == img.ordered.end()) {
        // Same table, first use on this stream: order the stream behind the copy that wrote the table.
        // A stream under capture cannot wait for work outside its graph, so there the call is refused.
        if ((rc = reject_capture(s, "grouped gemm (first use of this workspace on the stream)"))) return rc;
        B200_CUDA(cudaStreamWaitEvent(s, img.uploaded, 0));
        if (img.ordered.size() >= 16) img.ordered.erase(img.ordered.begin() + 1);
        img.ordered.push_back(s);
    }
    const WorkspaceImage& cur = g_workspaces[{device, workspace}];
    GroupedProblem p;
    p.groups = static_cast<const GroupEntry*>(workspace);
    p.total_tiles_dev = nullptr;
    p.num_groups = groups;
    p.total_tiles = cur.total_tiles;
    p.status = status ? status : st->status;
    p.cycles = st->cycles;
    p.trace = nullptr;
    const bool pdl = !uploads;    // the launch behind the table's copy keeps its full stream dependency
    if (cur.tile_n == kTilingPair) return launch_pair<PairGrouped>(p, p.total_tiles, st->sm_count, 0, s, pdl);
    if (variant == B200_VARIANT_SERIAL) {
        return cur.tile_n == 256 ? launch_serial<Mode::Group256>(p, p.total_tiles, 0, s)
                                 : launch_serial<Mode::Group128>(p, p.total_tiles, 0, s);
    }
    return cur.tile_n == 256
               ? launch_persistent<Mode::Group256, kG256Stages>(p, p.total_tiles, st->sm_count, 0, s, pdl)
               : launch_persistent<Mode::Group128, kG128Stages>(p, p.total_tiles, st->sm_count, 0, s, pdl);
}

int b200_grouped_gemm_nvfp4(int groups, const void* const* a, const void* const* b, const void* const* sfa,
                            const void* const* sfb, void* const* c, const int* mnk, void* workspace,
                            size_t workspace_bytes, void* stream, int device, uint32_t* status) {
    return b200_grouped_gemm_nvfp4_ex(groups, a, b, sfa, sfb, c, mnk, workspace, workspace_bytes, B200_VARIANT_AUTO,
                                      0, stream, device, status);
}

int b200_grouped_workspace_forget(int device, const void* workspace) {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (workspace == nullptr) {           // every workspace of the device
        for (auto it = g_workspaces.begin(); it != g_workspaces.end();) {
            if (it->first.first == device) {
                if (it->second.uploaded) cudaEventDestroy(it->second.uploaded);
                it = g_workspaces.erase(it);
            } else {
                ++it;
            }
        }
        return 0;
    }
    auto it = g_workspaces.find({device, workspace});
    if (it != g_workspaces.end()) {
        if (it->second.uploaded) cudaEventDestroy(it->second.uploaded);
        g_workspaces.erase(it);
    }
    return 0;
}

}  // extern "C"

namespace b200 {
namespace {
// Descriptor table of the entry point that may not allocate: part of the
// library's device image, so it exists on every GPU the library is loaded on.
// In host code this name is only a handle for cudaGetSymbolAddress; the kernels
// get the device address looked up below.
static __device__ __align__(256) GroupEntry g_static_group_table[B200_STATIC_MAX_GROUPS];

constexpr int kMaxDevices = 64;
GroupEntry* g_static_table_addr[kMaxDevices] = {};   // per device, filled on first use

// Device address of the table on the current device (`device` must be current).
int static_table_address(int device, GroupEntry** out) {
    if (device < 0 || device >= kMaxDevices) return fail(B200_E_LIMIT, "device index %d out of range", device);
    if (!g_static_table_addr[device]) {
        void* ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_group_table);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(g_static_group_table)");
        g_static_table_addr[device] = static_cast<GroupEntry*>(ptr);
    }
    *out = g_static_table_addr[device];
    return 0;
}
}  // namespace
}  // namespace b200

extern "C" {

int b200_grouped_gemm_nvfp4_static(int groups, const void* const* a, const void* const* b, const void* const* sfa,
                                   const void* const* sfb, void* const* c, const int* mnk, void* stream, int device,
                                   uint32_t* status) {
    if (groups <= 0) return fail(B200_E_SHAPE, "grouped gemm (static table): groups=%d must be positive", groups);
    if (groups > B200_STATIC_MAX_GROUPS)
        return fail(B200_E_LIMIT,
                    "grouped gemm (static table): %d groups exceed the built-in table of %d entries; use "
                    "b200_grouped_gemm_nvfp4 with a workspace, or split the call",
                    groups, B200_STATIC_MAX_GROUPS);
    if (!a || !b || !sfa || !sfb || !c || !mnk)
        return fail(B200_E_NULL, "grouped gemm (static table): NULL argument array");
    bool all_n256 = true;
    long long tiles128 = 0;
    for (int g = 0; g < groups; ++g) {
        const int m = mnk[3 * g], n = mnk[3 * g + 1], k = mnk[3 * g + 2];
        if (m < 0 || n <= 0 || k <= 0)
            return fail(B200_E_SHAPE, "grouped gemm (static table): group %d has invalid shape (%d, %d, %d)", g, m, n,
                        k);
        if (n % 128) return fail(B200_E_SHAPE, "grouped gemm (static table): group %d n=%d is not a multiple of 128", g, n);
        if (k % 256) return fail(B200_E_SHAPE, "grouped gemm (static table): group %d k=%d is not a multiple of 256", g, k);
        if (m == 0) continue;
        if (!a[g] || !b[g] || !sfa[g] || !sfb[g] || !c[g])
            return fail(B200_E_NULL, "grouped gemm (static table): group %d has a NULL tensor pointer", g);
        if (!aligned16(a[g]) || !aligned16(b[g]) || !aligned16(sfa[g]) || !aligned16(sfb[g]) || !aligned16(c[g]))
            return fail(B200_E_ALIGN, "grouped gemm (static table): group %d has a pointer that is not 16-byte aligned",
                        g);
        if (n % 256) all_n256 = false;
        tiles128 += static_cast<long long>((m + 127) / 128) * (n / 128);
    }
    if (tiles128 == 0) return 0;

    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceGuard guard;
    int rc;
    if ((rc = guard.enter(device))) return rc;
    DeviceState* st = nullptr;
    if ((rc = device_state(device, &st))) return rc;        // one-time per-device set-up, no allocation
    GroupEntry* table_dev = nullptr;
    if ((rc = static_table_address(device, &table_dev))) return rc;

    const int tile_n = (all_n256 && tiles128 / 2 >= 2LL * st->sm_count) ? 256 : 128;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if ((rc = reject_capture(s, "grouped gemm (static table)"))) return rc;
    // Host copy of the table on the stack (32 KiB at most): nothing is allocated.
    GroupEntry table[B200_STATIC_MAX_GROUPS];
    int tile_begin = 0;
    if ((rc = build_group_table(table, groups, a, b, sfa, sfb, c, mnk, tile_n, &tile_begin))) return rc;
    // Every entry this launch reads is rewritten here, so nothing left by an earlier
    // call is ever consumed; entries beyond `groups` keep stale bytes and are not read.
    // The source is pageable stack memory: the runtime has copied it out by the time
    // this returns, so `table` may die while the transfer is still queued on `s`.
    B200_CUDA(cudaMemcpyAsync(table_dev, table, static_cast<size_t>(groups) * sizeof(GroupEntry),
                              cudaMemcpyHostToDevice, s));
    GroupedProblem p;
    p.groups = table_dev;
    p.total_tiles_dev = nullptr;
    p.num_groups = groups;
    p.total_tiles = tile_begin;
    p.status = status ? status : st->status;
    p.cycles = st->cycles;
    p.trace = nullptr;
    return tile_n == 256 ? launch_persistent<Mode::Group256, kG256Stages>(p, p.total_tiles, st->sm_count, 0, s, false)
                         : launch_persistent<Mode::Group128, kG128Stages>(p, p.total_tiles, st->sm_count, 0, s, false);
}

// --------------------------------------------------------------------------
// Mixture-of-experts steps around the grouped GEMM
// --------------------------------------------------------------------------
static int moe_check_shape(const char* what, int tokens, int experts, int top_k) {
    if (tokens <= 0 || experts <= 0 || top_k <= 0)
        return fail(B200_E_SHAPE, "%s: tokens, experts and top_k must be positive (got %d %d %d)", what, tokens, experts,
                    top_k);
    if (experts > kMoeMaxExperts) return fail(B200_E_LIMIT, "%s: at most %d experts (got %d)", what, kMoeMaxExperts, experts);
    if (top_k > 32 || top_k > experts) return fail(B200_E_SHAPE, "%s: top_k=%d must be <= 32 and <= experts", what, top_k);
    if (static_cast<long long>(tokens) * top_k > 0x7fffffffLL / 2)
        return fail(B200_E_LIMIT, "%s: tokens * top_k does not fit the 32-bit row index", what);
    return 0;
}

int b200_moe_route(const float* logits, const float* bias, int tokens, int experts, int n_group, int topk_group,
                   int top_k, float routed_scaling, int32_t* topk_idx, float* topk_w, void* stream, int device) {
    int rc = moe_check_shape("moe route", tokens, experts, top_k);
    if (rc) return rc;
    if (!logits || !topk_idx || !topk_w) return fail(B200_E_NULL, "moe route: NULL tensor pointer");
    if (n_group <= 0 || n_group > 32 || experts % n_group || topk_group <= 0 || topk_group > n_group)
        return fail(B200_E_SHAPE, "moe route: n_group=%d must divide experts=%d, be <= 32 and >= topk_group=%d > 0", n_group,
                    experts, topk_group);
    if (top_k > topk_group * (experts / n_group))
        return fail(B200_E_SHAPE, "moe route: top_k=%d exceeds the %d experts of the kept groups", top_k,
                    topk_group * (experts / n_group));
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceGuard guard;
    if ((rc = guard.enter(device))) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // scores in registers when a lane's run of experts and a group's run of lanes are both whole
    const int per_lane = experts % 32 == 0 ? experts / 32 : 0;
    const int group_size = experts / n_group;
    const int lanes_per_group = per_lane > 0 && group_size % per_lane == 0 ? group_size / per_lane : 0;
    const bool in_registers = (per_lane == 2 || per_lane == 4 || per_lane == 8) && lanes_per_group > 0 &&
                              (lanes_per_group & (lanes_per_group - 1)) == 0;
    const dim3 grid((tokens + 7) / 8);
    if (in_registers && per_lane == 2)
        moe_route_regs<2><<<grid, 256, 0, s>>>(logits, bias, tokens, n_group, topk_group, top_k, routed_scaling, topk_idx, topk_w);
    else if (in_registers && per_lane == 4)
        moe_route_regs<4><<<grid, 256, 0, s>>>(logits, bias, tokens, n_group, topk_group, top_k, routed_scaling, topk_idx, topk_w);
    else if (in_registers)
        moe_route_regs<8><<<grid, 256, 0, s>>>(logits, bias, tokens, n_group, topk_group, top_k, routed_scaling, topk_idx, topk_w);
    else
        moe_route<<<grid, 256, 0, s>>>(logits, bias, tokens, experts, n_group, topk_group, top_k, routed_scaling, topk_idx,
                                       topk_w);
    B200_CUDA(cudaGetLastError());
    ++g_launches;
    g_last_kernel = in_registers ? "moe_route_regs" : "moe_route";
    return 0;
}

size_t b200_moe_plan_scratch_bytes(int tokens, int experts, int top_k) {
    if (tokens <= 0 || experts <= 0 || top_k <= 0) return 0;
    const long long entries = static_cast<long long>(tokens) * top_k;
    const long long blocks = (entries + kMoeChunk - 1) / kMoeChunk;
    return static_cast<size_t>(blocks) * experts * sizeof(int);
}

int b200_moe_plan(const int32_t* topk_idx, int tokens, int experts, int top_k, int32_t* counts, int32_t* row_offsets,
                  int32_t* sfa_atom_offsets, int32_t* row_of, int32_t* src_token, void* scratch, size_t scratch_bytes,
                  void* stream, int device) {
    int rc = moe_check_shape("moe plan", tokens, experts, top_k);
    if (rc) return rc;
    if (!topk_idx || !counts || !row_offsets || !sfa_atom_offsets || !row_of || !src_token || !scratch)
        return fail(B200_E_NULL, "moe plan: NULL tensor pointer");
    if (scratch_bytes < b200_moe_plan_scratch_bytes(tokens, experts, top_k))
        return fail(B200_E_WORKSPACE, "moe plan: scratch has %zu bytes, %zu needed", scratch_bytes,
                    b200_moe_plan_scratch_bytes(tokens, experts, top_k));
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceGuard guard;
    if ((rc = guard.enter(device))) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int entries = tokens * top_k;
    const int blocks = (entries + kMoeChunk - 1) / kMoeChunk;
    int* block_counts = static_cast<int*>(scratch);
    moe_count<<<blocks, kMoeChunk, 0, s>>>(topk_idx, entries, experts, block_counts);
    moe_scan<<<1, kMoeMaxExperts, 0, s>>>(block_counts, blocks, experts, counts, row_offsets, sfa_atom_offsets);
    moe_place<<<blocks, kMoeChunk, 0, s>>>(topk_idx, entries, experts, top_k, block_counts, row_offsets, row_of, src_token);
    B200_CUDA(cudaGetLastError());
    g_launches += 3;
    g_last_kernel = "moe_place";
    return 0;
}

size_t b200_moe_sfa_bytes(int tokens, int experts, int top_k, int k) {
    if (tokens <= 0 || experts <= 0 || top_k <= 0 || k <= 0 || k % 64) return 0;
    // every expert's rows are padded to whole 128-row atoms: at most one partly filled atom each
    const long long atoms = (static_cast<long long>(tokens) * top_k + 127) / 128 + experts;
    return static_cast<size_t>(atoms) * (k / 64) * 512;
}

size_t b200_moe_gather_scratch_bytes(int tokens, int k) {
    if (tokens <= 0 || k <= 0 || k % 64) return 0;
    // packed rows, then row-major scale factors (both multiples of 16 bytes per row)
    return static_cast<size_t>(tokens) * (k / 2) + static_cast<size_t>(tokens) * (k / 16);
}

int b200_moe_gather_quantize(const void* x, int dtype, int tokens, int k, int64_t ldx, const int32_t* src_token,
                             const int32_t* row_offsets, const int32_t* sfa_atom_offsets, int experts, int top_k,
                             void* a_q, void* sfa, void* scratch, size_t scratch_bytes, void* stream, int device) {
    int rc = moe_check_shape("moe gather", tokens, experts, top_k);
    if (rc) return rc;
    if (!x || !src_token || !row_offsets || !sfa_atom_offsets || !a_q || !sfa || !scratch)
        return fail(B200_E_NULL, "moe gather: NULL tensor pointer");
    if (dtype != B200_DTYPE_F16 && dtype != B200_DTYPE_BF16)
        return fail(B200_E_VARIANT, "moe gather: dtype %d is neither B200_DTYPE_F16 nor B200_DTYPE_BF16", dtype);
    if (k <= 0 || k % 64) return fail(B200_E_SHAPE, "moe gather: k=%d is not a positive multiple of 64", k);
    if (ldx < k || ldx % 8) return fail(B200_E_ALIGN, "moe gather: ldx=%lld must be >= k and a multiple of 8", (long long)ldx);
    if (!aligned16(x) || !aligned16(a_q) || !aligned16(sfa) || !aligned16(scratch))
        return fail(B200_E_ALIGN, "moe gather: every tensor pointer must be 16-byte aligned");
    if (scratch_bytes < b200_moe_gather_scratch_bytes(tokens, k))
        return fail(B200_E_WORKSPACE, "moe gather: scratch has %zu bytes, %zu needed", scratch_bytes,
                    b200_moe_gather_scratch_bytes(tokens, k));
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceGuard guard;
    if ((rc = guard.enter(device))) return rc;
    DeviceState* st = nullptr;
    if ((rc = device_state(device, &st))) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    uint8_t* q_rows = static_cast<uint8_t*>(scratch);
    uint8_t* sf_rows = q_rows + static_cast<size_t>(tokens) * (k / 2);
    const long long cap = static_cast<long long>(st->sm_count) * 16;
    long long blocks = (static_cast<long long>(tokens) * ((k / 16 + 31) / 32) + 7) / 8;
    if (blocks > cap) blocks = cap;
    const uint16_t* src = static_cast<const uint16_t*>(x);
    if (dtype == B200_DTYPE_F16)
        moe_quantize_rows<kQuantDtypeF16><<<static_cast<unsigned>(blocks), 256, 0, s>>>(src, ldx, tokens, k, q_rows, sf_rows);
    else
        moe_quantize_rows<kQuantDtypeBF16><<<static_cast<unsigned>(blocks), 256, 0, s>>>(src, ldx, tokens, k, q_rows, sf_rows);
    blocks = (static_cast<long long>(tokens) * top_k + 7) / 8;
    if (blocks > cap) blocks = cap;
    moe_gather_rows<<<static_cast<unsigned>(blocks), 256, 0, s>>>(q_rows, sf_rows, src_token, row_offsets, sfa_atom_offsets,
                                                                  experts, k, static_cast<uint8_t*>(a_q),
                                                                  static_cast<uint8_t*>(sfa));
    B200_CUDA(cudaGetLastError());
    g_launches += 2;
    g_last_kernel = "moe_gather_rows";
    return 0;
}

int b200_moe_quantize_scatter(const void* x, int dtype, int tokens, int k, int64_t ldx, const int32_t* row_of,
                              const int32_t* row_offsets, const int32_t* sfa_atom_offsets, int experts, int top_k,
                              void* a_q, void* sfa, void* stream, int device) {
    int rc = moe_check_shape("moe quantize+scatter", tokens, experts, top_k);
    if (rc) return rc;
    if (!x || !row_of || !row_offsets || !sfa_atom_offsets || !a_q || !sfa)
        return fail(B200_E_NULL, "moe quantize+scatter: NULL tensor pointer");
    if (dtype != B200_DTYPE_F16 && dtype != B200_DTYPE_BF16)
        return fail(B200_E_VARIANT, "moe quantize+scatter: dtype %d is neither B200_DTYPE_F16 nor B200_DTYPE_BF16", dtype);
    if (k <= 0 || k % 64) return fail(B200_E_SHAPE, "moe quantize+scatter: k=%d is not a positive multiple of 64", k);
    if (ldx < k || ldx % 8)
        return fail(B200_E_ALIGN, "moe quantize+scatter: ldx=%lld must be >= k and a multiple of 8", (long long)ldx);
    if (!aligned16(x) || !aligned16(a_q) || !aligned16(sfa))
        return fail(B200_E_ALIGN, "moe quantize+scatter: every tensor pointer must be 16-byte aligned");
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceGuard guard;
    if ((rc = guard.enter(device))) return rc;
    DeviceState* st = nullptr;
    if ((rc = device_state(device, &st))) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    long long blocks = (static_cast<long long>(tokens) * kMoeScatterSplit + 7) / 8;   // kMoeScatterSplit warps per token
    const long long cap = static_cast<long long>(st->sm_count) * 32;
    if (blocks > cap) blocks = cap;
    const uint16_t* src = static_cast<const uint16_t*>(x);
    if (dtype == B200_DTYPE_F16)
        moe_quantize_scatter<kQuantDtypeF16><<<static_cast<unsigned>(blocks), 256, 0, s>>>(
            src, ldx, tokens, k, row_of, row_offsets, sfa_atom_offsets, experts, top_k, static_cast<uint8_t*>(a_q),
            static_cast<uint8_t*>(sfa));
    else
        moe_quantize_scatter<kQuantDtypeBF16><<<static_cast<unsigned>(blocks), 256, 0, s>>>(
            src, ldx, tokens, k, row_of, row_offsets, sfa_atom_offsets, experts, top_k, static_cast<uint8_t*>(a_q),
            static_cast<uint8_t*>(sfa));
    B200_CUDA(cudaGetLastError());
    ++g_launches;
    g_last_kernel = "moe_quantize_scatter";
    return 0;
}

size_t b200_moe_gemm_workspace_bytes(int experts) {
    if (experts <= 0) return 0;
    return static_cast<size_t>(experts) * sizeof(GroupEntry) + 256;      // table + the tile count
}

int b200_moe_grouped_gemm_nvfp4(int experts, const void* a_q, const void* sfa, int total_rows, const void* const* b,
                                const void* const* sfb, int n, int k, const int32_t* counts, const int32_t* row_offsets,
                                const int32_t* sfa_atom_offsets, void* y, void* workspace, size_t workspace_bytes,
                                void* stream, int device, uint32_t* status) {
    if (experts <= 0 || experts > kMoeMaxExperts)
        return fail(B200_E_LIMIT, "moe gemm: experts=%d must be in 1..%d", experts, kMoeMaxExperts);
    if (!a_q || !sfa || !b || !sfb || !counts || !row_offsets || !sfa_atom_offsets || !y)
        return fail(B200_E_NULL, "moe gemm: NULL argument");
    if (total_rows <= 0) return fail(B200_E_SHAPE, "moe gemm: total_rows=%d must be positive", total_rows);
    if (n <= 0 || n % 128) return fail(B200_E_SHAPE, "moe gemm: n=%d is not a positive multiple of 128", n);
    if (k <= 0 || k % 256) return fail(B200_E_SHAPE, "moe gemm: k=%d is not a positive multiple of 256", k);
    if (!aligned16(a_q) || !aligned16(sfa) || !aligned16(y))
        return fail(B200_E_ALIGN, "moe gemm: every tensor pointer must be 16-byte aligned");
    for (int e = 0; e < experts; ++e) {
        if (!b[e] || !sfb[e]) return fail(B200_E_NULL, "moe gemm: expert %d has a NULL weight pointer", e);
        if (!aligned16(b[e]) || !aligned16(sfb[e]))
            return fail(B200_E_ALIGN, "moe gemm: expert %d has a weight pointer that is not 16-byte aligned", e);
    }
    if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255u))
        return fail(B200_E_WORKSPACE, "moe gemm: workspace must be non-NULL and 256-byte aligned");
    if (workspace_bytes < b200_moe_gemm_workspace_bytes(experts))
        return fail(B200_E_WORKSPACE, "moe gemm: workspace has %zu bytes, %zu needed", workspace_bytes,
                    b200_moe_gemm_workspace_bytes(experts));

    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceGuard guard;
    int rc;
    if ((rc = guard.enter(device))) return rc;
    DeviceState* st = nullptr;
    if ((rc = device_state(device, &st))) return rc;
    // The row counts live on the device, so the tiling is chosen from what the host knows: CTA pairs
    // (256 x 256 tiles) when n allows it and the rows would give every pair a tile, else 128 x 128 tiles.
    const bool use_pair = n % 256 == 0 && static_cast<long long>(total_rows / 256) * (n / 256) >= st->sm_count / 2;
    const int tiling = use_pair ? kTilingPair : 128;

    std::vector<uint8_t> key(4 * sizeof(int) + 3 * sizeof(void*) + static_cast<size_t>(experts) * 2 * sizeof(void*) + 8);
    {
        uint8_t* w = key.data();
        auto put = [&w](const void* src, size_t nbytes) { memcpy(w, src, nbytes); w += nbytes; };
        const char tag[8] = {'m', 'o', 'e', 0, 0, 0, 0, 0};
        put(tag, 8);
        put(&experts, sizeof(int));
        put(&total_rows, sizeof(int));
        put(&n, sizeof(int));
        put(&k, sizeof(int));
        put(&a_q, sizeof(void*));
        put(&sfa, sizeof(void*));
        put(&y, sizeof(void*));
        put(b, experts * sizeof(void*));
        put(sfb, experts * sizeof(void*));
    }
    if (g_workspaces.size() > 256 && !g_workspaces.count({device, workspace})) drop_workspace_images();
    WorkspaceImage& img = g_workspaces[{device, workspace}];
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    GroupEntry* table_dev = static_cast<GroupEntry*>(workspace);
    int* total_dev = reinterpret_cast<int*>(static_cast<uint8_t*>(workspace) + static_cast<size_t>(experts) * sizeof(GroupEntry));
    if (img.key != key) {
        // static part of the table: one tensor map over the whole A buffer shared by all experts, one
        // per expert's weights, shapes and B-side pointers.  The device fills in the rest every call.
        if ((rc = reject_capture(s, "moe gemm"))) return rc;
        std::vector<GroupEntry> table(experts);
        memset(table.data(), 0, static_cast<size_t>(experts) * sizeof(GroupEntry));
        CUtensorMap map_a;
        if ((rc = encode_operand_map(&map_a, a_q, total_rows, k, 1, static_cast<long long>(total_rows) * (k / 2)))) return rc;
        for (int e = 0; e < experts; ++e) {
            GroupEntry& g = table[e];
            g.map_a = map_a;
            if ((rc = encode_operand_map(&g.map_b, b[e], n, k, 1, static_cast<long long>(n) * (k / 2)))) return rc;
            g.sfb = static_cast<const uint8_t*>(sfb[e]);
            g.ldc = n;
            g.n = n;
            g.k_tiles = k / 256;
            g.n_tiles = use_pair ? n / 256 : n / 128;
            g.sf_k_atoms = k / 64;
            g.sfb_row_atoms = n / 128;
        }
        img.key.clear();
        B200_CUDA(cudaMemcpyAsync(workspace, table.data(), static_cast<size_t>(experts) * sizeof(GroupEntry),
                                  cudaMemcpyHostToDevice, s));
        if (!img.uploaded) B200_CUDA(cudaEventCreateWithFlags(&img.uploaded, cudaEventDisableTiming));
        B200_CUDA(cudaEventRecord(img.uploaded, s));
        img.ordered.assign(1, s);
        img.key = key;
        img.tile_n = tiling;
    } else if (std::find(img.ordered.begin(), img.ordered.end(), s) == img.ordered.end()) {
        if ((rc = reject_capture(s, "moe gemm (first use of this workspace on the stream)"))) return rc;
        B200_CUDA(cudaStreamWaitEvent(s, img.uploaded, 0));
        if (img.ordered.size() >= 16) img.ordered.erase(img.ordered.begin() + 1);
        img.ordered.push_back(s);
    }
    moe_fill_group_table<<<1, kMoeMaxExperts, 0, s>>>(table_dev, experts, counts, row_offsets, sfa_atom_offsets,
                                                      static_cast<const uint8_t*>(sfa), static_cast<__half*>(y), n, k,
                                                      use_pair ? 256 : 128, total_dev);
    B200_CUDA(cudaGetLastError());
    ++g_launches;
    GroupedProblem p;
    p.groups = table_dev;
    p.total_tiles_dev = total_dev;
    p.num_groups = experts;
    p.total_tiles = 0;
    p.status = status ? status : st->status;
    p.cycles = st->cycles;
    p.trace = nullptr;
    // full grid: how many tiles there are is only known on the device
    // rows past an expert's count are the next expert's: row-predicated stores, not the per-group store maps
    if (use_pair) return launch_pair<PairGroupedShared>(p, 1 << 30, st->sm_count, 0, s);
    return launch_persistent<Mode::Group128, kG128Stages>(p, 1 << 30, st->sm_count, 0, s);
}

int b200_moe_combine(const void* y, int n, const int32_t* row_of, const float* topk_w, int tokens, int top_k,
                     int out_dtype, void* out, int64_t ldo, void* stream, int device) {
    if (!y || !row_of || !topk_w || !out) return fail(B200_E_NULL, "moe combine: NULL tensor pointer");
    if (tokens <= 0 || top_k <= 0) return fail(B200_E_SHAPE, "moe combine: tokens and top_k must be positive");
    if (n <= 0 || n % 8) return fail(B200_E_SHAPE, "moe combine: n=%d is not a positive multiple of 8", n);
    if (ldo < n || ldo % 8) return fail(B200_E_ALIGN, "moe combine: ldo=%lld must be >= n and a multiple of 8", (long long)ldo);
    if (out_dtype != B200_DTYPE_F16 && out_dtype != B200_DTYPE_BF16)
        return fail(B200_E_VARIANT, "moe combine: out_dtype %d is neither B200_DTYPE_F16 nor B200_DTYPE_BF16", out_dtype);
    if (!aligned16(y) || !aligned16(out)) return fail(B200_E_ALIGN, "moe combine: y and out must be 16-byte aligned");
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceGuard guard;
    int rc;
    if ((rc = guard.enter(device))) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (out_dtype == B200_DTYPE_F16)
        moe_combine<kQuantDtypeF16><<<tokens, 256, 0, s>>>(static_cast<const __half*>(y), n, row_of, topk_w, top_k,
                                                           static_cast<uint16_t*>(out), ldo);
    else
        moe_combine<kQuantDtypeBF16><<<tokens, 256, 0, s>>>(static_cast<const __half*>(y), n, row_of, topk_w, top_k,
                                                            static_cast<uint16_t*>(out), ldo);
    B200_CUDA(cudaGetLastError());
    ++g_launches;
    g_last_kernel = "moe_combine";
    return 0;
}

size_t b200_quantize_sf_bytes(int rows, int k) {
    if (rows <= 0 || k <= 0 || k % 64) return 0;
    return static_cast<size_t>((rows + 127) / 128) * (k / 64) * 512;
}

int b200_quantize_nvfp4(const void* x, int dtype, int rows, int k, int64_t ldx, void* q, void* sf, void* stream,
                        int device) {
    if (!x || !q || !sf) return fail(B200_E_NULL, "quantize: NULL tensor pointer");
    if (dtype != B200_DTYPE_F16 && dtype != B200_DTYPE_BF16)
        return fail(B200_E_VARIANT, "quantize: dtype %d is neither B200_DTYPE_F16 nor B200_DTYPE_BF16", dtype);
    if (rows <= 0 || k <= 0) return fail(B200_E_SHAPE, "quantize: rows and k must be positive (got %d %d)", rows, k);
    if (k % 64) return fail(B200_E_SHAPE, "quantize: k=%d is not a multiple of 64", k);
    if (ldx < k || ldx % 8) return fail(B200_E_ALIGN, "quantize: ldx=%lld must be >= k and a multiple of 8", (long long)ldx);
    if (!aligned16(x) || !aligned16(q) || !aligned16(sf))
        return fail(B200_E_ALIGN, "quantize: every tensor pointer must be 16-byte aligned");
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceGuard guard;
    int rc;
    if ((rc = guard.enter(device))) return rc;
    DeviceState* st = nullptr;
    if ((rc = device_state(device, &st))) return rc;
    const long long chunks = static_cast<long long>((rows + 127) / 128 * 128) * ((k / 16 + 31) / 32);
    long long blocks = (chunks + 7) / 8;                       // eight warps per block
    const long long cap = static_cast<long long>(st->sm_count) * 16;
    if (blocks > cap) blocks = cap;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const uint16_t* src = static_cast<const uint16_t*>(x);
    const bool wide = (reinterpret_cast<uintptr_t>(x) % 32 == 0) && (ldx % 16 == 0);
    const unsigned grid = static_cast<unsigned>(blocks);
    uint8_t* qp = static_cast<uint8_t*>(q);
    uint8_t* sfp = static_cast<uint8_t*>(sf);
    if (dtype == B200_DTYPE_F16) {
        if (wide) nvfp4_quantize<kQuantDtypeF16, true><<<grid, 256, 0, s>>>(src, ldx, qp, sfp, rows, k);
        else nvfp4_quantize<kQuantDtypeF16, false><<<grid, 256, 0, s>>>(src, ldx, qp, sfp, rows, k);
    } else {
        if (wide) nvfp4_quantize<kQuantDtypeBF16, true><<<grid, 256, 0, s>>>(src, ldx, qp, sfp, rows, k);
        else nvfp4_quantize<kQuantDtypeBF16, false><<<grid, 256, 0, s>>>(src, ldx, qp, sfp, rows, k);
    }
    B200_CUDA(cudaGetLastError());
    ++g_launches;
    g_last_kernel = "nvfp4_quantize";
    return 0;
}

int b200_probe_l2_feed(int device, int ctas, int share, int tiled, int copies_per_cta, double* tb_per_s,
                       double* bytes_per_clk_per_sm, double* sm_mhz) {
    if (!tb_per_s || !bytes_per_clk_per_sm) return fail(B200_E_NULL, "probe_l2_feed: an output pointer is NULL");
    if (ctas < 1 || ctas > 1024 || share < 1 || copies_per_cta < kFeedSlots)
        return fail(B200_E_SHAPE, "probe_l2_feed: ctas=%d share=%d copies_per_cta=%d", ctas, share, copies_per_cta);
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceGuard guard;
    int rc;
    if ((rc = guard.enter(device))) return rc;
    DeviceState* st = nullptr;
    if ((rc = device_state(device, &st))) return rc;
    constexpr int kRows = 16384, kRowBytes = 2048;            // 32 MiB: stays in L2
    uint8_t* window = nullptr;
    unsigned long long* cycles = nullptr;
    B200_CUDA(cudaMalloc(&window, static_cast<size_t>(kRows) * kRowBytes));
    if (cudaMalloc(&cycles, static_cast<size_t>(ctas) * sizeof(unsigned long long)) != cudaSuccess) {
        cudaFree(window);
        return fail(static_cast<int>(cudaErrorMemoryAllocation), "probe_l2_feed: out of device memory");
    }
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    auto cleanup = [&]() {
        if (e0) cudaEventDestroy(e0);
        if (e1) cudaEventDestroy(e1);
        cudaFree(cycles);
        cudaFree(window);
    };
    FeedProbe p;
    memset(&p, 0, sizeof p);
    rc = encode_operand_map(&p.map, window, kRows, kRowBytes * 2, 1, static_cast<long long>(kRows) * kRowBytes);
    if (rc) { cleanup(); return rc; }
    p.window = window;
    p.rows = kRows;
    p.row_bytes = kRowBytes;
    constexpr int kMine = kFeedSlots / kFeedIssuers;
    p.copies_per_issuer = (copies_per_cta / kFeedIssuers + kMine - 1) / kMine * kMine;
    p.share = share;
    p.tiled = tiled ? 1 : 0;
    p.cycles = cycles;
    p.status = st->status;
    const size_t smem = static_cast<size_t>(kFeedSlots) * kFeedSlotBytes + 1024;
    float ms = 0.f;
    std::vector<unsigned long long> host(ctas);
    cudaError_t err = cudaMemset(window, 0x11, static_cast<size_t>(kRows) * kRowBytes);
    if (err == cudaSuccess) err = cudaFuncSetAttribute(l2_feed_probe, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (err == cudaSuccess) err = cudaEventCreate(&e0);
    if (err == cudaSuccess) err = cudaEventCreate(&e1);
    for (int rep = 0; rep < 2 && err == cudaSuccess; ++rep) {   // the first pass brings the window into L2
        cudaEventRecord(e0, nullptr);
        l2_feed_probe<<<ctas, kFeedThreads, smem, nullptr>>>(p);
        cudaEventRecord(e1, nullptr);
        err = cudaEventSynchronize(e1);
        if (err == cudaSuccess) err = cudaGetLastError();
    }
    if (err == cudaSuccess) err = cudaEventElapsedTime(&ms, e0, e1);
    if (err == cudaSuccess) err = cudaMemcpy(host.data(), cycles, host.size() * sizeof(unsigned long long), cudaMemcpyDeviceToHost);
    cleanup();
    if (err != cudaSuccess) return fail(static_cast<int>(err), "probe_l2_feed: %s", cudaGetErrorString(err));
    ++g_launches;
    unsigned long long slowest = 1;
    for (unsigned long long v : host) slowest = v > slowest ? v : slowest;
    const double bytes_per_cta = static_cast<double>(p.copies_per_issuer) * kFeedIssuers * kFeedSlotBytes;
    *tb_per_s = bytes_per_cta * ctas / (static_cast<double>(ms) * 1e-3) / 1e12;
    *bytes_per_clk_per_sm = bytes_per_cta / static_cast<double>(slowest);
    if (sm_mhz) *sm_mhz = static_cast<double>(slowest) / (static_cast<double>(ms) * 1e3);
    return 0;
}

int b200_read_last_cycles(int device, void* stream, uint64_t* out) {
    if (!out) return fail(B200_E_NULL, "read_last_cycles: out is NULL");
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceGuard guard;
    int rc;
    if ((rc = guard.enter(device))) return rc;
    DeviceState* st = nullptr;
    if ((rc = device_state(device, &st))) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    B200_CUDA(cudaStreamSynchronize(s));
    unsigned long long v = 0;
    B200_CUDA(cudaMemcpy(&v, st->cycles, sizeof v, cudaMemcpyDeviceToHost));
    *out = v;
    return 0;
}

int b200_read_status(int device, void* stream, uint32_t* out) {
    if (!out) return fail(B200_E_NULL, "read_status: out is NULL");
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceGuard guard;
    int rc;
    if ((rc = guard.enter(device))) return rc;
    DeviceState* st = nullptr;
    if ((rc = device_state(device, &st))) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    B200_CUDA(cudaStreamSynchronize(s));
    B200_CUDA(cudaMemcpy(out, st->status, sizeof(uint32_t), cudaMemcpyDeviceToHost));
    if (*out) B200_CUDA(cudaMemset(st->status, 0, sizeof(uint32_t)));
    return 0;
}

}  // extern "C"
