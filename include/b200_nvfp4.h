/*
 * C ABI of libb200nvfp4.so: NVFP4 block-scaled dual GEMM and grouped GEMM for
 * NVIDIA B200 (sm_100a).
 *
 * All pointers marked "device" are device addresses on `device`; the library
 * never allocates or frees them.  Calls enqueue work on `stream` (a
 * cudaStream_t passed as void*, NULL = default stream) and return without
 * synchronising, like the reference's custom_kernel() entry points.
 *
 * Return value of every int function: 0 = success, < 0 = argument rejected on
 * the host before any CUDA work (B200_E_*), > 0 = a CUDA runtime/driver error
 * code (cudaError_t).  b200_last_error() describes the last non-zero return of
 * the calling thread.
 */
#ifndef B200_NVFP4_H_
#define B200_NVFP4_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_E_NULL (-1)      /* a required pointer is NULL                      */
#define B200_E_SHAPE (-2)     /* m/n/k/l violate the divisibility rules          */
#define B200_E_ALIGN (-3)     /* a pointer or pitch is not 16-byte aligned       */
#define B200_E_WORKSPACE (-4) /* workspace too small or misaligned               */
#define B200_E_VARIANT (-5)   /* unknown kernel variant                          */
#define B200_E_DRIVER (-6)    /* CUDA driver entry point unavailable             */
#define B200_E_LIMIT (-7)     /* size beyond a documented maximum                */
#define B200_E_CAPTURE (-8)   /* the stream is being captured and the call must copy
                                 from host memory that dies when it returns      */

/* Kernel variants (the `variant` argument of the *_ex entry points). */
#define B200_VARIANT_AUTO 0       /* library picks by shape.  Dual GEMM with m % 256 == 0:
                                     PAIR_NARROW when all 256 x 64 tiles fit one round of
                                     the GPU's CTA pairs, else PAIR; other m: PERSISTENT  */
#define B200_VARIANT_PERSISTENT 1 /* warp-specialised persistent kernel               */
#define B200_VARIANT_SERIAL 2     /* one CTA per tile, single stage (bring-up / debug) */
#define B200_VARIANT_SERIAL_2MMA 3/* as SERIAL but two N=128 MMAs per k-block          */
#define B200_VARIANT_SPLITK 4     /* persistent kernel, k-range split over CTAs with an
                                     fp32 partial-sum exchange before the epilogue     */
#define B200_VARIANT_PAIR 5       /* CTA pairs (2-SM MMA, 256-row tiles).  Dual GEMM:
                                     needs m % 256 == 0.  Grouped GEMM: 256 x 256 tiles,
                                     needs every n % 256 == 0, any m.  AUTO picks, for a
                                     grouped list, the tiling (128 x 128, 128 x 256 or
                                     pairs) with the fewest rounds x measured cycles per
                                     k-tile                                             */

#define B200_VARIANT_PAIR_NARROW 6 /* dual GEMM: CTA pairs on 256 x 64 output tiles (2-SM MMA
                                     256 x 128 x 64); for shapes with few tiles            */
#define B200_VARIANT_PAIR_STREAMK 7 /* dual GEMM: PAIR whose last round and remainder are cut
                                     along k so that every CTA pair gets the same number of
                                     k-tiles; the two pairs that share a tile exchange fp32
                                     partial sums through the workspace
                                     (b200_dual_streamk_workspace_bytes)                   */
#define B200_VARIANT_SELFTEST_LOST_LOAD 8 /* dual GEMM only, failure-detection self-test: the
                                     one-CTA kernel with its producer dropping the loads of
                                     every tile's second k-tile and every on-device wait
                                     limited to about a millisecond.  The waits give up, the
                                     launch ends by itself, C is not written and the status
                                     word becomes non-zero (needs k >= 512)               */

/* Library version string, e.g. "b200nvfp4 0.1 (sm_100a)". */
const char* b200_version(void);

/* Message for the calling thread's last failing call ("" if none). */
const char* b200_last_error(void);

/*
 * C[m, n, l] = silu(A . B1^T) * (A . B2^T), fp32 accumulation, fp16 output.
 * Replaces custom_kernel(data) of the reference's dual GEMM
 * (dual_gemm/submission.py:894-957, dual_gemm/dual_gemm_opt_cute.py:2706-2832).
 *
 *   a            device, [m, k/2, l] packed e2m1 (2 per byte, low nibble = even k),
 *                K-major, batch stride m*k/2 bytes                    (data[0])
 *   b1, b2       device, [n, k/2, l] packed e2m1, batch stride
 *                b_batch_bytes (n*k/2 when 0)                          (data[1], data[2])
 *   sfa          device, e4m3 scale factors of A in the permuted layout
 *                (32,4,ceil(m/128),4,k/64,l)                           (data[6])
 *   sfb1, sfb2   device, same layout for B1/B2 rows; batch stride
 *                sfb_batch_bytes (ceil(n/128)*(k/64)*512 when 0)       (data[7], data[8])
 *   c            device, fp16, element (i, j, b) at c[b*c_batch + i*ldc + j]
 *                (c_batch = m*ldc when 0), written in place            (data[9])
 *   m % 128 == 0, n % 128 == 0, k % 256 == 0, l >= 1; ldc % 8 == 0;
 *   every pointer 16-byte aligned.
 *
 * `n` may be a column shard of a wider problem: pass the shard's rows of
 * B1/B2, its scale-factor atoms and a `c` pointer offset to the shard's first
 * column with `ldc` the full row pitch.
 *
 * status: device pointer to one uint32 the kernel ORs a non-zero code into if
 * a bounded on-device wait gives up (0 stays 0 on success), or NULL to use a
 * library-owned word readable with b200_read_status().
 */
int b200_dual_gemm_nvfp4(const void* a, const void* b1, const void* b2, const void* sfa,
                         const void* sfb1, const void* sfb2, void* c, int m, int n, int k, int l,
                         int64_t ldc, void* stream, int device, uint32_t* status);

/* Same, with explicit batch strides, kernel variant and an optional split-k
 * workspace (256-byte aligned, b200_dual_splitk_workspace_bytes() bytes).  Shapes
 * with fewer than half as many 128x128 output tiles as the GPU has SMs are cut
 * along k so that every SM gets a piece; the pieces exchange fp32 partial sums
 * through the workspace before the silu*mul epilogue.  Only B200_VARIANT_SPLITK
 * splits (and fails without a large enough workspace); the other variants ignore
 * the workspace.  The first bytes of the workspace hold
 * per-unit flag words that each launch stamps with a fresh number: zero-fill the
 * workspace once before its first use.  One workspace per stream.  The units of
 * a tile wait for one another inside the launch, so the library never starts
 * more units than the GPU has SMs. */
int b200_dual_gemm_nvfp4_ex(const void* a, const void* b1, const void* b2, const void* sfa,
                            const void* sfb1, const void* sfb2, void* c, int m, int n, int k, int l,
                            int64_t ldc, int64_t c_batch, int64_t b_batch_bytes,
                            int64_t sfb_batch_bytes, int variant, void* workspace,
                            size_t workspace_bytes, void* stream, int device, uint32_t* status);

/*
 * Column shard of the dual GEMM fused with the all-gather of the shards: rank `rank`
 * of `world` GPUs of one node computes columns [col_offset, col_offset + n_local) of
 * C [m, n_total] and its epilogue stores every tile into the full C of EVERY rank:
 * c_ranks[r] is rank r's [m, n_total] fp16 buffer as seen from this GPU (its own
 * buffer for r == rank, peer-mapped addresses for the others: CUDA peer access or
 * symmetric memory), written with plain TMA stores over NVLink, no multicast.  When
 * all ranks' launches have completed (synchronise, then a barrier), every rank holds
 * the whole C.  The reference is single-GPU and has no counterpart; it stands in
 * for "shard, then all-gather" (b200_dual_gemm_nvfp4 on a shard + a collective).
 *   a, sfa replicated; b1, b2, sfb1, sfb2 this rank's n_local rows; m % 256 == 0,
 *   n_local, n_total, col_offset % 128 == 0, k % 256 == 0, world <= 8.
 */
int b200_dual_gemm_nvfp4_gather(const void* a, const void* b1, const void* b2, const void* sfa,
                                const void* sfb1, const void* sfb2, void* const* c_ranks, int world,
                                int rank, int m, int n_local, int n_total, int col_offset, int k,
                                void* stream, int device, uint32_t* status);

/* Bytes of scratch for the stream-k tail of the CTA-pair dual GEMM on a 148-SM B200
 * (74 pairs x 256 KiB of fp32 partial sums plus flag words), or 0 when the shape's
 * tiles fill whole rounds and nothing would be cut.  Pass it as `workspace` of
 * b200_dual_gemm_nvfp4_ex with B200_VARIANT_PAIR_STREAMK: 256-byte aligned,
 * zero-filled once before its first use, one workspace per stream.  No other
 * variant cuts tiles. */
size_t b200_dual_streamk_workspace_bytes(int m, int n, int k, int l);

/* Bytes of split-k workspace for an (m, n, k, l) problem on a 148-SM B200;
 * 0 when the shape has enough tiles and is not split. */
size_t b200_dual_splitk_workspace_bytes(int m, int n, int k, int l);

/*
 * Grouped GEMM: for every group g, C_g[m_g, n_g] = A_g . B_g^T (fp16 output, no
 * activation), all groups in one launch.  Replaces custom_kernel(data) of the
 * reference's grouped GEMM (group_gemm/group_gemm_cute5_v2.py:4245-4424,
 * group_gemm/group_gemm_cute4.py:1252-1399).
 *
 *   a[g], b[g], c[g]   host arrays of device pointers: A_g [m_g, k_g/2],
 *                      B_g [n_g, k_g/2] packed e2m1, C_g [m_g, n_g] fp16 row-major
 *                      (abc_tensors[g])
 *   sfa[g], sfb[g]     device pointers to the permuted scale factors
 *                      (sfasfb_reordered_tensors[g]); rows of SFA beyond m_g may
 *                      hold anything
 *   mnk                host array of 3*groups ints (m_g, n_g, k_g);
 *                      m_g >= 0 (0 = group skipped), n_g % 128 == 0, k_g % 256 == 0
 *                      (problem_sizes[g][0:3], l == 1)
 *   workspace          device scratch of at least b200_grouped_workspace_bytes(groups)
 *                      bytes, 256-byte aligned; holds the per-group descriptors the
 *                      kernel indexes.  The library rewrites it only when the
 *                      descriptors differ from what it last put there.
 */
int b200_grouped_gemm_nvfp4(int groups, const void* const* a, const void* const* b,
                            const void* const* sfa, const void* const* sfb, void* const* c,
                            const int* mnk, void* workspace, size_t workspace_bytes, void* stream,
                            int device, uint32_t* status);

/* Same with an explicit kernel variant (AUTO, PERSISTENT, SERIAL or PAIR) and
 * N-tile width (0 = auto, 128 or 256).
 *
 * Both grouped entry points copy the descriptor table from host memory that
 * dies when the call returns, so a call that has to upload (first use of a
 * workspace, or changed arguments) is refused with B200_E_CAPTURE while `stream`
 * is being captured; a repeated call whose table is already in the workspace
 * only launches.  The first repeated call on another stream than the one that
 * uploaded makes that stream wait for the upload (an event), which a stream
 * under capture cannot do: it is refused the same way.  So before capturing,
 * make the call once, on the stream that will be captured. */
int b200_grouped_gemm_nvfp4_ex(int groups, const void* const* a, const void* const* b,
                               const void* const* sfa, const void* const* sfb, void* const* c,
                               const int* mnk, void* workspace, size_t workspace_bytes, int variant,
                               int tile_n, void* stream, int device, uint32_t* status);

size_t b200_grouped_workspace_bytes(int groups);

/* Tell the library that `workspace` on `device` no longer holds the descriptor
 * table it last uploaded there (the memory was freed, reused or overwritten), so
 * the next call uploads again.  workspace == NULL forgets every workspace of the
 * device.  Call it before releasing a workspace.  The reference rewrites its
 * pointer tables on every call instead (group_gemm/group_gemm_cute5_v2.py:4319-4345). */
int b200_grouped_workspace_forget(int device, const void* workspace);

/*
 * Grouped GEMM for callers that have no device memory to give and may not
 * allocate any.  No counterpart in the reference: there, PyTorch's allocator is
 * always at hand.  A serving engine that has handed every byte of the GPU to its
 * own pools, a plugin running inside someone else's memory budget, or code on a
 * path where cudaMalloc's implicit device synchronisation is unacceptable has
 * nowhere to put the per-group descriptor table that b200_grouped_gemm_nvfp4
 * keeps in the caller's workspace.  Here the table lives in a fixed array inside
 * the library's device image instead: B200_STATIC_MAX_GROUPS entries of 512
 * bytes (32 KiB), present on every GPU that loads the library until the process
 * exits.  Arguments and results are those of b200_grouped_gemm_nvfp4 without the
 * workspace.  It always runs the one-CTA-per-tile kernels (128 x 128 or 128 x 256
 * tiles); the workspace entry point additionally picks the CTA-pair kernel for
 * large lists.  Both give the same bits.
 *
 *  - groups > B200_STATIC_MAX_GROUPS is rejected with B200_E_LIMIT.
 *  - The call allocates and frees nothing, on the device or through any library.
 *  - The first call on a device looks up the array's device address and does the
 *    library's one-time per-device set-up; make that call before any stream
 *    capture begins.
 *  - Every call copies the table from the host stack into the array, so a call on
 *    a stream that is being captured is refused with B200_E_CAPTURE.
 *  - Every call rewrites the entries it uses and all calls share the one array:
 *    two calls whose GPU work can overlap (different streams, or the same stream
 *    from different threads without ordering) race on it.  Calls on one stream
 *    are safe back to back.
 */
#define B200_STATIC_MAX_GROUPS 64
int b200_grouped_gemm_nvfp4_static(int groups, const void* const* a, const void* const* b,
                                   const void* const* sfa, const void* const* sfb, void* const* c,
                                   const int* mnk, void* stream, int device, uint32_t* status);

/*
 * Dual GEMM with NVFP4 output: computes the same fp16 values as
 * b200_dual_gemm_nvfp4 and re-quantises them in the epilogue like
 * b200_quantize_nvfp4 would (byte for byte), so the result can be the `a` / `sfa`
 * of the next block-scaled GEMM (the down projection of a SwiGLU FFN) without a
 * round trip of fp16 C through memory.
 *   q   [m, n/2] packed e2m1;  sf  reordered e4m3 scale factors of an [m, n]
 *       operand, b200_quantize_sf_bytes(m, n) bytes
 *   m % 256 == 0 (runs on the CTA-pair kernel), n % 128 == 0, k % 256 == 0, l = 1.
 * No counterpart in the reference (its kernels store fp16, dual_gemm/submission.py:596-611).
 */
int b200_dual_gemm_nvfp4_quant(const void* a, const void* b1, const void* b2, const void* sfa,
                               const void* sfb1, const void* sfb2, void* q, void* sf, int m, int n,
                               int k, void* stream, int device, uint32_t* status);

/*
 * Activation quantiser: x [rows, k] fp16 or bf16 (row pitch ldx elements) ->
 * NVFP4 operand in the layout the GEMM entry points above take as `a`:
 *   q   [rows, k/2] packed e2m1, low nibble = even k
 *   sf  e4m3 scale factors, one per 16 consecutive k, in the reordered layout
 *       (ceil(rows/128), k/64, 32, 4, 4); b200_quantize_sf_bytes(rows, k) bytes;
 *       rows of the last 128-row block past `rows` get zero scale factors
 *   s = e4m3_rn_satfinite(max|x| / 6), q = e2m1_rn_satfinite(x * fp32(1 / s)) (0 when s == 0)
 * The step before the GEMMs in an FFN.  No counterpart in the reference, which
 * draws already-quantised operands (dual_gemm/reference.py:114-190).
 *   k % 64 == 0 (the GEMMs need k % 256 == 0); ldx % 8 == 0; pointers 16-byte aligned.
 */
#define B200_DTYPE_F16 0
#define B200_DTYPE_BF16 1
size_t b200_quantize_sf_bytes(int rows, int k);
int b200_quantize_nvfp4(const void* x, int dtype, int rows, int k, int64_t ldx, void* q, void* sf,
                        void* stream, int device);

/*
 * Mixture-of-experts steps around the grouped GEMM: routing, permutation of the token
 * rows into per-expert row ranges (quantising them to NVFP4 on the way), the expert
 * GEMMs with a descriptor table finished on the device, and the weighted combination.
 * They restate, for an NVFP4 expert GEMM, what the reference's MoE does with torch ops
 * on FP8 data (moe/moe_fibench_ref.py:20-33): routing :106-134, token gather :144-153,
 * expert GEMM :155-170, weighted accumulation :172-176.  Every array below is device
 * memory unless it says "host"; nothing is read back to the host, so the five calls of a
 * layer queue up on one stream without a synchronisation.
 *
 * b200_moe_route: DeepSeek-V3 "no-aux" routing of `tokens` rows of fp32 logits
 *   [tokens, experts] (bias [experts] or NULL): s = sigmoid(logits), s_b = s + bias; the
 *   experts form n_group equal groups scored by the sum of their two largest s_b; the
 *   topk_group best groups stay; the top_k largest s_b among their experts are chosen
 *   (ties: smaller index); weight = s / (sum of the chosen s + 1e-20) * routed_scaling.
 *   topk_idx / topk_w [tokens, top_k], slots in descending order of s_b.
 *   experts <= 256, n_group <= 32 and a divisor of experts, top_k <= 32.
 *   n_group = topk_group = 1 is plain top-k.
 */
int b200_moe_route(const float* logits, const float* bias, int tokens, int experts, int n_group,
                   int topk_group, int top_k, float routed_scaling, int32_t* topk_idx,
                   float* topk_w, void* stream, int device);

/* b200_moe_plan: stable counting sort of the tokens * top_k (token, slot) entries by
 *   expert.  counts [experts]; row_offsets [experts + 1]: expert e owns rows
 *   [row_offsets[e], row_offsets[e + 1]) of the permuted order, in token order;
 *   sfa_atom_offsets [experts + 1]: 128-row scale-factor atoms before each expert (every
 *   expert's scale factors start on an atom boundary); row_of [tokens * top_k]: row of
 *   each entry; src_token [tokens * top_k]: token of each row.  scratch:
 *   b200_moe_plan_scratch_bytes() bytes of device scratch. */
size_t b200_moe_plan_scratch_bytes(int tokens, int experts, int top_k);
int b200_moe_plan(const int32_t* topk_idx, int tokens, int experts, int top_k, int32_t* counts,
                  int32_t* row_offsets, int32_t* sfa_atom_offsets, int32_t* row_of,
                  int32_t* src_token, void* scratch, size_t scratch_bytes, void* stream,
                  int device);

/* b200_moe_gather_quantize: row r of the permuted order = x[src_token[r], :] (fp16 or
 *   bf16, row pitch ldx) quantised exactly like b200_quantize_nvfp4: a_q [tokens * top_k,
 *   k/2] packed e2m1 shared by all experts, sfa = b200_moe_sfa_bytes() bytes holding
 *   every expert's reordered scale factors from its atom offset on (rows of an expert's
 *   last atom past its count keep whatever the buffer held).  Two kernels: every token
 *   row is quantised once into `scratch` (b200_moe_gather_scratch_bytes() bytes), then
 *   the quantised rows are copied to their top_k places.  k % 64 == 0. */
size_t b200_moe_sfa_bytes(int tokens, int experts, int top_k, int k);
size_t b200_moe_gather_scratch_bytes(int tokens, int k);
int b200_moe_gather_quantize(const void* x, int dtype, int tokens, int k, int64_t ldx,
                             const int32_t* src_token, const int32_t* row_offsets,
                             const int32_t* sfa_atom_offsets, int experts, int top_k, void* a_q,
                             void* sfa, void* scratch, size_t scratch_bytes, void* stream,
                             int device);

/* b200_moe_quantize_scatter: the same a_q and sfa as b200_moe_gather_quantize in one
 *   kernel and without scratch memory, from the token's side: every token's row is read
 *   and quantised once and each 16-k block is written straight to the token's top_k rows
 *   row_of[token, slot] of the permuted order (tokens * k * (2 + top_k * 9/16) bytes of
 *   traffic instead of an intermediate buffer and a second pass).  The reference permutes
 *   with torch indexing (moe/moe_fibench_ref.py:142-151); it has no quantising step. */
int b200_moe_quantize_scatter(const void* x, int dtype, int tokens, int k, int64_t ldx,
                              const int32_t* row_of, const int32_t* row_offsets,
                              const int32_t* sfa_atom_offsets, int experts, int top_k, void* a_q,
                              void* sfa, void* stream, int device);

/* b200_moe_grouped_gemm_nvfp4: y[rows of expert e, :] = a_q[rows of e, :] . B_e^T for all
 *   experts in one launch (fp16 y [total_rows, n]).  b / sfb: host arrays of device
 *   pointers to each expert's [n, k/2] packed e2m1 weights and reordered scale factors.
 *   The per-expert row counts stay on the device: the host uploads the constant part of
 *   the descriptor table (tensor maps, weight pointers; only when its arguments change,
 *   and never under stream capture) and a one-block kernel fills in counts, row ranges
 *   and tile numbers before the GEMM kernel, which reads its tile count from device
 *   memory.  workspace: b200_moe_gemm_workspace_bytes(experts) bytes, 256-byte aligned.
 *   n % 128 == 0, k % 256 == 0, total_rows = tokens * top_k. */
size_t b200_moe_gemm_workspace_bytes(int experts);
int b200_moe_grouped_gemm_nvfp4(int experts, const void* a_q, const void* sfa, int total_rows,
                                const void* const* b, const void* const* sfb, int n, int k,
                                const int32_t* counts, const int32_t* row_offsets,
                                const int32_t* sfa_atom_offsets, void* y, void* workspace,
                                size_t workspace_bytes, void* stream, int device,
                                uint32_t* status);

/* b200_moe_combine: out[t, :] = sum over the token's top_k slots of topk_w * y[row_of, :],
 *   accumulated in fp32 in slot order, stored as fp16 or bf16 (B200_DTYPE_*) with row
 *   pitch ldo.  n % 8 == 0. */
int b200_moe_combine(const void* y, int n, const int32_t* row_of, const float* topk_w, int tokens,
                     int top_k, int out_dtype, void* out, int64_t ldo, void* stream, int device);

/* Synchronise `stream`, copy the library-owned status word of `device` into
 * *out and clear it. */
int b200_read_status(int device, void* stream, uint32_t* out);

/* Synchronise `stream` and return the SM-clock cycles (clock64) that the first
 * CTA of the last GEMM launch on `device` spent from entry to exit.  Divided by
 * the launch's CUDA-event time this gives the SM clock the launch really ran at,
 * which nvidia-smi cannot sample inside a millisecond-long region.  The
 * reference gathers the same kind of figure with in-kernel clock64 probes
 * (group_gemm/group_gemm_cute4.py:67-79, 622-637). */
int b200_read_last_cycles(int device, void* stream, uint64_t* out);

/* Measurement aid for the roofline of the GEMMs above: a kernel that does nothing
 * but TMA loads into shared memory (twelve 16 KiB slots in flight per CTA, four
 * issuing warps) from a 32 MiB window that stays in L2, on `ctas` CTAs of which
 * `share` consecutive ones read the same tiles at about the same time.  tiled != 0
 * loads 128-row x 128-byte boxes with the 128-byte swizzle, as the GEMMs' operand
 * loads do; 0 loads contiguous 16 KiB.  Allocates and frees its own device memory,
 * runs on the default stream and synchronises.  Returns the aggregate rate in
 * TB/s, the bytes per SM clock of the slowest CTA and (optionally, may be NULL)
 * the SM clock in MHz during the run.  The reference has no counterpart; its
 * authors reason about the same feed with in-kernel clock64 probes
 * (group_gemm/group_gemm_cute4.py:67-79). */
int b200_probe_l2_feed(int device, int ctas, int share, int tiled, int copies_per_cta, double* tb_per_s,
                       double* bytes_per_clk_per_sm, double* sm_mhz);

/* Name of the kernel the most recent launch of this process used (which one the
 * library's shape heuristic picked), e.g. "nvfp4_gemm_pair<PairDual>". */
const char* b200_last_kernel(void);

/* Number of kernels this library has launched in the calling process. */
uint64_t b200_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* B200_NVFP4_H_ */
