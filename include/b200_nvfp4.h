/*
 * C ABI of the B200 (sm_100a) NVFP4 hot-path library.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream handle
 * (a cudaStream_t passed as void*; NULL selects the legacy default stream), is
 * asynchronous on that stream, allocates no output memory and returns an int
 * status (B2_OK on success).  No exception crosses this boundary; a human
 * readable reason for the last failure of the calling thread is returned by
 * b2_last_error().
 *
 * Each declaration names the reference interface it stands in for, by the
 * path of the file inside the mlc-ai/TIRx-kernels project.
 */
#ifndef B200_NVFP4_H_
#define B200_NVFP4_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------ */
#define B2_OK 0
#define B2_ERR_INVALID_ARGUMENT 1 /* shape / alignment / null pointer; nothing was launched   */
#define B2_ERR_CUDA 2             /* a CUDA runtime or driver call failed                      */
#define B2_ERR_DEVICE_TIMEOUT 3   /* a bounded device-side wait expired (read by *_status())   */
#define B2_ERR_UNSUPPORTED 4      /* valid in the reference, not built here yet                */

/* ---- enums (ints on the wire) ------------------------------------------- */
#define B2_DTYPE_F16 0
#define B2_DTYPE_BF16 1

#define B2_SF_LINEAR 0 /* uint8[m, k/16] row-major                                   */
#define B2_SF_128x4 1  /* 128-row x 4-column tiles of 512 B, the tcgen05 / cuBLASLt layout */
#define B2_SF_8x4 2    /* 8-row x 4-column tiles of 32 B                            */

#define B2_SCALE_E4M3 0
#define B2_SCALE_UE8M0 1

/* op codes of b2_mufu_probe */
#define B2_MUFU_RCP_FTZ 0   /* rcp.approx.ftz.f32   */
#define B2_MUFU_RSQRT_FTZ 1 /* rsqrt.approx.ftz.f32 */
#define B2_MUFU_LG2 2       /* lg2.approx.f32       */
#define B2_MUFU_EX2 3       /* ex2.approx.f32       */
#define B2_MUFU_EX2_FTZ 4   /* ex2.approx.ftz.f32   */
/* The quantizer's SiLU on one fp32 value: as the kernel computes it (packed-FMA division with a
 * div.rn.f32 fallback) and with div.rn.f32 throughout; the two must agree bit for bit. */
#define B2_PROBE_SILU 5
#define B2_PROBE_SILU_DIV_RN 6

/* Reason for the most recent non-zero status returned to this thread. */
const char* b2_last_error(void);

/* Library ABI version (bumped when a signature changes). */
int b2_abi_version(void);

/*
 * NVFP4 block quantizer.
 *
 * Replaces the executables returned by get_kernel() in
 * tirx_kernels/flashinfer/quantization/nvfp4_quantize.py:191-377
 * (nvfp4_quantize_linear :214-221, nvfp4_quantize_swizzled :259-266), launched
 * by _run_launch :441-445.
 *
 *   in       [m, k] (or [m, 2k] = [gate | up] when fuse_silu) fp16/bf16, row-major
 *   out      uint8 [m, k/2]: element 2j in the low nibble, 2j+1 in the high nibble
 *   sf       uint8 scale factors, one E4M3 byte per 16 elements, in sf_layout;
 *            swizzled layouts are zero-filled in their padding rows and columns
 *   gs_dev   device pointer to the fp32 global (encode) scale
 * Requirements: k > 0, k % 16 == 0, m >= 1, `in` 32-byte aligned, `out` 8-byte aligned.
 */
int b2_nvfp4_quantize(const void* in, void* out, void* sf, const float* gs_dev, int m, int k,
                      int in_dtype, int sf_layout, int fuse_silu, int enable_pdl, void* stream);

/*
 * Per-token NVFP4 quantizer: the executable of
 * tirx_kernels/flashinfer/quantization/nvfp4_quantize_per_token.py:142-232, called as
 * ex(a_flat, out_flat, sf, pts, m, gs_inv) in run_test :321.  Every row gets its own scale:
 * token_scale[r] = amax(row r) * gs_inv[0] (0 for an all-zero row), and the blocks of the row are
 * quantized with 1 / token_scale in place of the global scale.
 *   in [m, k] fp16/bf16; out [m, k/2]; sf in `sf_layout` (b2_nvfp4_sf_bytes); token_scale [m] fp32
 * Padding columns AND padding rows of the swizzled layouts are zero-filled by the call (the
 * reference leaves the rows to a zero-initialised buffer from its host wrapper, :262-264).
 */
int b2_nvfp4_quantize_per_token(const void* in, void* out, void* sf, float* token_scale,
                                const float* gs_inv_dev, int m, int k, int in_dtype, int sf_layout,
                                int enable_pdl, void* stream);

/* Number of bytes of the scale-factor buffer for (m, k, sf_layout); mirrors
 * _sf_numel, tirx_kernels/flashinfer/quantization/nvfp4_quantize.py:126-129. */
int64_t b2_nvfp4_sf_bytes(int m, int k, int sf_layout);

/*
 * RMSNorm fused with FP4 block quantization.
 *
 * Replaces the executable returned by get_kernel() in
 * tirx_kernels/flashinfer/norm/rmsnorm_fp4quant.py:707-1033 (entry signature
 * :983-991, launched by _launch_tirx :1156-1165).
 *
 *   x        [M, H] fp16/bf16 row-major;  w  [H] same dtype
 *   y        uint8 [M, H/2] packed E2M1
 *   sf       block_size 16: E4M3 bytes; block_size 32: E4M3 or UE8M0 bytes; linear
 *            [M, H/block_size] or 128x4-swizzled (padding positions are left untouched)
 *   gs_dev   fp32 global scale (read only when the scale format in effect is E4M3)
 * Requirements: H >= 64, H % block_size == 0, M >= 1.
 */
int b2_rmsnorm_fp4quant(const void* x, const void* w, void* y, void* sf, const float* gs_dev,
                        int M, int H, float eps, int in_dtype, int block_size, int scale_format,
                        int swizzled, int enable_pdl, void* stream);

/*
 * Per-CTA timeline of b2_rmsnorm_fp4quant (observability, no counterpart in the reference).  While
 * `device_buf` is non-null, launches that take the register-resident kernel (rows of up to 16 chunks
 * per thread, the case of every benchmarked shape) record four 64-bit words per CTA at
 * device_buf[4 * cta]: start, row sums reduced, end (nanoseconds of the GPU's global timer) and the
 * SM id.  The buffer needs 4 * ceil(M / rows per CTA) words; 4 * M always suffices.  Null stops it.
 */
int b2_rmsnorm_fp4quant_timeline(unsigned long long* device_buf);

/*
 * Residual add + RMSNorm + FP4 block quantization: the executable of
 * tirx_kernels/flashinfer/norm/add_rmsnorm_fp4quant.py:1210-1221 (ABI x, residual, weight, y, scale,
 * scale_unswizzled, y_norm, global_scale, M, eps), called by _launch_tirx :1457-1470; the compile-time
 * knobs of get_kernel :788-799 are arguments here.
 *   residual  in: residual [M, H]; out: x + residual rounded to the input dtype (in place)
 *   sf        scale bytes, 128x4-swizzled when `swizzled` or `output_both_sf_layouts`, else [M, H/block]
 *   sf_unswizzled  second, linear copy of the scale bytes when `output_both_sf_layouts` (else unused, may be NULL)
 *   y_norm    the normalized, weighted row in the input dtype when `output_norm` (else unused, may be NULL)
 * Other arguments as b2_rmsnorm_fp4quant.  Rows with H >= 32768 are spread over a thread-block
 * cluster exactly where the reference does (_source_config :354-363), which fixes the summation order.
 */
int b2_add_rmsnorm_fp4quant(const void* x, void* residual, const void* w, void* y, void* sf,
                            void* sf_unswizzled, void* y_norm, const float* gs_dev, int M, int H,
                            float eps, int in_dtype, int block_size, int scale_format, int swizzled,
                            int output_both_sf_layouts, int output_norm, int enable_pdl, void* stream);

/*
 * Dense block-scaled NVFP4 GEMM:  D[M,N] (bf16) = alpha * A[M,K] * B[N,K]^T.
 *
 * Replaces _Runner.__call__ in tirx_kernels/basic/nvfp4_gemm.py:985-997 (kernel
 * :374-857, tensor maps :941-982).
 *
 *   A, B       packed E2M1, K-major: uint8 [M, K/2] and uint8 [N, K/2]
 *   SFA, SFB   E4M3 block scales (one per 16 along K) in the 128x4-swizzled layout,
 *              ceil(M/128)*128 x K/16 and ceil(N/128)*128 x K/16 bytes
 *   alpha_dev  device fp32 scalar (1 / (encode scale of A * encode scale of B))
 * Requirements: K % 256 == 0, N % 128 == 0, M >= 1, all pointers 16-byte aligned.
 * Tensor maps are cached per (pointers, shape) inside the library (host memory).
 *
 * Device memory the library allocates on the caller's behalf, and when (the reference's executable
 * allocates nothing; a caller that must not allocate uses b2_nvfp4_gemm_small_m_noalloc):
 *  - 256 bytes of status words per device, on the first GEMM call on that device;
 *  - for M <= 128 (the problem is cut into K ranges whose fp32 partial sums a second kernel adds):
 *    one scratch buffer per device, 32 MiB on the first such call, replaced by a larger one only
 *    when a later problem needs more (K ranges x M x N x 4 bytes).  An outgrown buffer is kept
 *    until the process exits, never freed, so launches in flight and captured graphs that name it
 *    stay valid and no call takes the device-wide synchronisation of cudaFree.
 * Consequences for M <= 128: make the first call of a shape class before any stream capture (a call
 * that allocates inside a capture invalidates it); calls on one device share the scratch, so keep
 * them in stream order - two such calls that overlap on the GPU (different streams, graphs
 * replayed concurrently) race on it.
 *
 * Launch order: the kernel is launched with the programmatic-stream-serialization attribute.  It may
 * therefore become resident while the kernel before it on `stream` is still running, but it executes
 * griddepcontrol.wait before its first access to global memory, so it observes everything earlier
 * work on the stream wrote, as an ordinary launch does; it then executes
 * griddepcontrol.launch_dependents, which matters only to a following kernel that was itself
 * launched with that attribute (such a kernel must wait the same way before it reads D).
 * B2_GEMM_PDL=0 in the environment launches without the attribute.
 */
int b2_nvfp4_gemm(const void* A, const void* B, const void* SFA, const void* SFB,
                  const float* alpha_dev, void* D, int M, int N, int K, void* stream);

/* Selects the kernel variant used by the following b2_nvfp4_gemm calls of this process
 * (-1 restores automatic selection): 0 single CTA / N tile 128, 1 single CTA / N tile 256,
 * 2 CTA pair / N tile 256, 3 CTA pair / N tile 128, 4 and 5 = 0 and 1 for M <= 32 (32 rows of A
 * per stage, deeper ring), 6 = M <= 32 with N tile 64 and all of K per CTA, 7 = 6 with two MMA-issuing
 * warps (two accumulators, added in the epilogue), 8 = 7 with 128 rows of A per stage (M <= 128), 9 = 0 with two
 * MMA-issuing warps (chosen for M > 128 when the 128 x 128 tiles fit the SMs in one wave).  The reference fixes its tiling per
 * shape in TIRX_CONFIGS, tirx_kernels/basic/nvfp4_gemm.py:860-903; this is the matching knob. */
int b2_nvfp4_gemm_set_variant(int variant);

/* Reads (and clears) the device status word written by bounded waits inside
 * b2_nvfp4_gemm on the current device; synchronises `stream` first.
 * Returns B2_OK, or B2_ERR_DEVICE_TIMEOUT with the detail in b2_last_error(). */
int b2_nvfp4_gemm_status(void* stream);

/*
 * Decode-sized GEMM (1 <= M <= 128) for callers that must not allocate device memory.  It has no
 * counterpart in the reference.  Same operands, kernel variant, K ranges and therefore the same bits
 * of the result as b2_nvfp4_gemm, but neither this call
 * nor its first-use set-up calls cudaMalloc, cudaFree or any allocating library routine: the
 * partial sums of its split-K path and its status words live in a 4 MiB + 256 B array built
 * into the library (resident on every GPU that loads it until the process exits).
 * Meant for hosts where a plugin may not allocate: a serving loop that owns all of HBM through its
 * own pool, a latency-critical section that cannot afford the device-wide synchronisation of
 * cudaMalloc / cudaFree, a sandbox that forbids the call.
 *  - The first call on a device resolves the array's device address; make it before any stream
 *    capture.
 *  - Problems whose partial sums (K ranges x M x N x 4 bytes) exceed 4 MiB are rejected with
 *    B2_ERR_INVALID_ARGUMENT; b2_last_error() states the requirement and the limit.
 *  - All calls on a device share the array: keep them in stream order, calls that overlap on the
 *    GPU race on it.  Nothing has to be cleared between calls.
 *  - Expired bounded waits end the kernel cleanly and are reported by
 *    b2_nvfp4_gemm_small_m_noalloc_status (not by b2_nvfp4_gemm_status, which reads the words of
 *    the allocating entry point).
 */
int b2_nvfp4_gemm_small_m_noalloc(const void* A, const void* B, const void* SFA, const void* SFB,
                                  const float* alpha_dev, void* D, int M, int N, int K, void* stream);

/* Reads (and clears) the status words b2_nvfp4_gemm_small_m_noalloc's kernels write on the current
 * device; synchronises `stream` first.  Returns B2_OK, or B2_ERR_DEVICE_TIMEOUT with the detail in
 * b2_last_error().  Allocates nothing (an 8-byte copy out of the built-in array).  No counterpart in
 * the reference. */
int b2_nvfp4_gemm_small_m_noalloc_status(void* stream);

/*
 * Test hooks of the device-side bounded waits (the reference has no analogue: its kernels wait
 * without a limit).  b2_nvfp4_gemm_set_wait_budget_ms shortens the budget of every wait in later
 * GEMM launches of this process to `milliseconds` (0 restores the default of one second; waits
 * downstream of a stalled role get twice the budget so that the status names the role that stalled
 * first).  b2_nvfp4_gemm_inject_test_fault(1) makes the NEXT launch announce, for the first K slab
 * of CTA 0, 16 bytes more than its copies deliver: every copy still lands and nothing stays in
 * flight, but the slab's barrier never completes, the MMA role's wait runs out, the kernel ends
 * through its abort path and b2_nvfp4_gemm_status reports B2_ERR_DEVICE_TIMEOUT.  Off by default.
 */
int b2_nvfp4_gemm_set_wait_budget_ms(int milliseconds);
int b2_nvfp4_gemm_inject_test_fault(int fault);

/*
 * Column-sharded projection with its output all-gather fused into the GEMM epilogue, for the
 * tensor-parallel FFN.  The reference's nearest analogues are tirx_kernels/basic/allgather_gemm.py
 * (peer puts of the INPUT rows in front of an fp16 GEMM) and tirx_kernels/basic/gemm_reduce_scatter.py
 * (GEMM with a fused collective on its output); it has no NVFP4 form of either.
 *
 * One process per GPU.  Every GPU owns one bf16 buffer [M, world * N] obtained from b2_peer_alloc;
 * b2_peer_export turns it into a 64-byte handle that the ranks exchange over their own control
 * channel, and b2_peer_open maps a peer's handle into this process (b2_peer_close unmaps it,
 * b2_peer_free releases the owner's buffer).  `D_all[g]` is this process's address of GPU g's buffer
 * (its own allocation for g == rank).
 *
 * b2_nvfp4_gemm_allgather multiplies A [M, K] by this rank's weight slab B [N, K] and stores every
 * finished tile into columns [rank * N, (rank + 1) * N) of all `world` buffers: the local one with
 * ordinary stores, the others with stores over NVLink.  No remote load, no multicast.  The call
 * is asynchronous; a peer's rows are complete only after that peer's stream has passed the call, so
 * the caller runs a cross-rank barrier (any host or NCCL barrier ordered after the stream) before
 * reading.  Needs M > 128, N % 128 == 0, K % 256 == 0, 1 <= world <= 8.
 */
int b2_peer_alloc(void** ptr, int64_t bytes);
int b2_peer_free(void* ptr);
int b2_peer_export(void* ptr, unsigned char* handle64);
int b2_peer_open(const unsigned char* handle64, void** ptr);
int b2_peer_close(void* ptr);
int b2_nvfp4_gemm_allgather(const void* A, const void* B, const void* SFA, const void* SFB,
                            const float* alpha_dev, void* const* D_all, int world, int rank,
                            int M, int N, int K, void* stream);

/*
 * In-kernel role timers of b2_nvfp4_gemm (observability; the reference's nearest analogue is the
 * u64 event buffer of tirx_kernels/basic/allgather_gemm.py:48-53).  `enable` != 0 makes later
 * launches record, for CTA 0, SM-cycle counters per warp role; `out12` (host, may be NULL)
 * receives the counters of the last recorded launch: [0] operand producer waiting for a free
 * stage, [1] producer total, [2] MMA waiting for data, [3] MMA waiting for a drained accumulator,
 * [4] MMA total, [5] MMA issue, [6] epilogue waiting, [7] epilogue body, [8] tiles,
 * [9] scale warp waiting, [10] scale warp body, [11] MMA total in nanoseconds.
 */
int b2_nvfp4_gemm_role_timers(int enable, unsigned long long* out12, void* stream);

/*
 * cuBLASLt NVFP4 matmul, the library peer the reference times beside its own
 * kernel: nvfp4_cublaslt in tirx_kernels/basic/nvfp4_gemm.py:196-239.
 * Lives in a separate shared object (libb200nvfp4_cublaslt.so) so the product
 * library carries no cuBLAS dependency.  `alpha` is a host scalar, as in the reference.
 */
int b2_nvfp4_gemm_cublaslt(const void* A, const void* B, const void* SFA, const void* SFB,
                           float alpha, void* D, int M, int N, int K, void* stream);

/*
 * Evaluates one hardware-approximate (MUFU) instruction elementwise:
 * out[i] = op(in[i]).  Test infrastructure for the CPU oracle: these
 * instructions (used by fp_quant.py rcp_approx_ftz :277-281 and
 * rmsnorm_fp4quant.py _rsqrt_approx_ftz :78-79, _cvt_f32_to_ue8m0 :155-171,
 * _ue8m0_to_output_scale :174-185) are not specified bit-for-bit, so the oracle
 * takes their values from the hardware and computes everything else itself.
 */
int b2_mufu_probe(int op, const float* in_dev, float* out_dev, int n, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200_NVFP4_H_ */
