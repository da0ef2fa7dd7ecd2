/* C ABI of libfeather_ops_b200.so: the sm_100a kernels behind the feather_ops quantized-matmul family.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream, enqueues its kernel(s) on that
 * stream and returns without synchronizing. The caller owns every buffer. Nothing here allocates device
 * memory. Pointers that the reference requires to be 16-byte aligned must be 16-byte aligned here too.
 * The names, argument order and argument meaning are those of the reference's own `extern "C"` launchers
 * (the ones its torch-free C++ benchmarks bind), with `cudaStream_t` in place of `hipStream_t`.
 *
 * Tile integers keep the reference's vocabulary (`feather_ops/tiles.py` there): they must name a row of
 * the tile table, and select the UMMA tile whose width matches the tuple's `16 * warps_n * repeat_n`.
 */
#ifndef FEATHER_OPS_B200_H_
#define FEATHER_OPS_B200_H_

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* feather_stream_t; /* a cudaStream_t */

/* C[M,N] = cast(cast((A[M,K] @ upcast(B)) * scale) + bias), fp32 accumulation.
 * a: fp16/bf16 bits [M,K] row-major. b_prepacked: fp8 bytes [ceil(K/128)*8][N][16]. scale: one float or NULL.
 * bias: N values in the output dtype or NULL. c: fp16/bf16 bits [M,N]. N % 16 == 0, K % 16 == 0, M >= 0.
 * Replaces `launch_scaled_mm`, reference csrc/hip_kernel.cu:687-713. Returns false for an unknown tile
 * tuple or an unsupported shape. */
bool launch_scaled_mm(const uint16_t* a, const uint8_t* b_prepacked, const float* scale, const uint16_t* bias, uint16_t* c, int64_t M,
                      int64_t N, int64_t K, int has_scale, int has_bias, bool use_fp8_e5m2, bool a_bf16, bool output_bf16,
                      int block_warps_m, int block_warps_n, int unroll_k, int repeat_m, int repeat_n, bool prefetch,
                      feather_stream_t stream);

/* Split-K variant of scaled_mm for skinny problems (M <= 128): one CTA per (64-column tile, K split) streams the
 * weight, fp32 partial tiles go to `partials`, the CTA that finishes a tile last sums them in split order and writes c.
 * partials: scratch of feather_scaled_mm_splitk_partial_floats(M, N, K, splits) floats (may be NULL when that is 0).
 * counters: ceil(N / 64) uint32, zero before the first launch; every launch leaves them zero. Launches sharing the
 * scratch must not overlap on the device. No counterpart in the reference's C ABI (its kernels have no split-K). */
bool launch_scaled_mm_splitk(const uint16_t* a, const uint8_t* b_prepacked, const float* scale, const uint16_t* bias, uint16_t* c, int64_t M,
                             int64_t N, int64_t K, int has_scale, int has_bias, bool use_fp8_e5m2, bool a_bf16, bool output_bf16, int splits,
                             float* partials, uint32_t* counters, feather_stream_t stream);

/* launch_scaled_mm_splitk for taller problems: the persistent one-CTA kernel with 128 x block_n tiles (block_n = 128 or
 * 256) walks (tile, K split) work items, so a product with fewer tiles than SMs (a few hundred rows) still uses all of
 * them; with more items than SMs the CTA that draws a tile's last ticket adds the partials in split order, with at most
 * one item per SM every CTA of a tile adds its share of the columns after a bounded wait for the others. Any M. With block_n = 256, more than
 * 128 rows and at most as many (256 x 256 tile, split) items as CTA pairs fit the device at once, the CTA-pair kernel runs
 * instead, one item per pair, and every CTA of a tile adds its share of the columns (at most 8 splits).
 * partials: scratch of feather_scaled_mm_splitk_wide_partial_floats(M, N, K, block_n, splits) floats.
 * counters: feather_scaled_mm_splitk_wide_counters(M, N, block_n) uint32, zero before the first launch, left zero by every
 * launch. The result does not depend on the order in which the CTAs finish. No counterpart in the reference's C ABI. */
bool launch_scaled_mm_splitk_wide(const uint16_t* a, const uint8_t* b_prepacked, const float* scale, const uint16_t* bias, uint16_t* c,
                                  int64_t M, int64_t N, int64_t K, int has_scale, int has_bias, bool use_fp8_e5m2, bool a_bf16,
                                  bool output_bf16, int block_n, int splits, float* partials, uint32_t* counters, feather_stream_t stream);

/* Number of floats of `partials` scratch launch_scaled_mm_splitk_wide needs: whole tiles per split (0 when the request
 * collapses to one split). No counterpart in the reference. */
int64_t feather_scaled_mm_splitk_wide_partial_floats(int64_t M, int64_t N, int64_t K, int block_n, int splits);

/* Number of uint32 tickets launch_scaled_mm_splitk_wide needs in `counters`. No counterpart in the reference. */
int64_t feather_scaled_mm_splitk_wide_counters(int64_t M, int64_t N, int block_n);

/* Number of floats of `partials` scratch launch_scaled_mm_splitk needs (0 when the request collapses to one split).
 * No counterpart in the reference. */
int64_t feather_scaled_mm_splitk_partial_floats(int64_t M, int64_t N, int64_t K, int splits);

/* launch_scaled_mm_splitk for hosts that cannot allocate device memory (a serving loop that gave all free memory to its
 * own arena, an FFI plugin without a device allocator, a callback in which allocation calls are forbidden): the partials
 * and tickets live in a 4 MiB + 1 KiB __device__ array inside the library, so no scratch is passed and nothing is
 * allocated. Limits: M <= 16, N <= 16384, at most 4 effective splits. Returns 0 = enqueued, 1 = invalid arguments,
 * 2 = larger than the built-in scratch, 3 = a CUDA call failed; error_message (may be NULL) receives the reason.
 * The first call on a device looks the array's address up (make it before any stream capture). All calls share
 * the array, so calls that overlap on the device race. This entry point has no counterpart in the reference. */
int launch_scaled_mm_splitk_static(const uint16_t* a, const uint8_t* b_prepacked, const float* scale, const uint16_t* bias, uint16_t* c,
                                   int64_t M, int64_t N, int64_t K, int has_scale, int has_bias, bool use_fp8_e5m2, bool a_bf16,
                                   bool output_bf16, int splits, feather_stream_t stream, char* error_message, size_t error_capacity);

/* Leaves `sms` SMs free in every later launch of the persistent scaled_mm kernels (0 restores full grids): for a caller
 * that overlaps the product with kernels that need SMs of their own, such as an NCCL collective on another stream (a
 * persistent CTA holds its SM until the kernel ends). Process-wide, takes effect at the next launch. Returns the previous
 * value. No counterpart in the reference (it has no multi-GPU path). */
int feather_scaled_mm_set_sm_margin(int sms);

/* out[r][g][:] = slabs[g][r][:] for g < world, r < rows, rows of width_bytes bytes (a multiple of 16; both pointers
 * 16-byte aligned): turns the [world][rows][width] result of an all-gather of column slabs into the row-major
 * [rows][world * width] matrix. Returns false for bad arguments. No counterpart in the reference. */
bool launch_interleave_slabs(const void* slabs, void* out, int64_t world, int64_t rows, int64_t width_bytes, feather_stream_t stream);

/* Output columns per tile (a multiple of 32 from 128 to 256) that launch_scaled_mm's CTA-pair kernel uses for M rows and N columns when `pairs`
 * CTA pairs are resident (74 on a B200): the width that minimises rounds of the persistent grid x (width + 304), i.e. a narrower tile only
 * where it fills the last round. The tile tuple of the call only says "256 wide" (csrc/hip_kernel.cu:825-846 takes the tuple as it is).
 * No counterpart in the reference. */
int feather_scaled_mm_pair_tile_width(int64_t M, int64_t N, int pairs);

/* Diagnostic: reads and clears the record that the scaled_mm kernel's bounded device waits report into.
 * out[0] = 0 when every wait completed, else the wait site; out[1] = block index. Synchronizes the device.
 * Returns 0 on success. No counterpart in the reference (its kernels have no device-side waits). */
int feather_scaled_mm_status(uint32_t* out);

/* ConvRot activation quantizer: per row, group-256 regular Hadamard rotation (fp32 radix-4, one rounding to the
 * input dtype), row absmax, int8 codes in [-127, 127] and one fp32 scale per row (absmax / 127, divided by 16
 * when rotating). x: [M, K] fp16 (input_fp16 != 0) or bf16, K % 256 == 0. col_scale: [K] multiplier applied
 * (and rounded to the input dtype) only when rotate is false, or NULL. q: [M, K] int8. row_scale: [M].
 * Replaces `launch_convrot_quantize`, reference csrc/hip_kernel_int8.cu:869-878. */
bool launch_convrot_quantize(const void* x, const float* col_scale, int8_t* q, float* row_scale, int64_t M, int64_t K, int input_fp16,
                             bool rotate, feather_stream_t stream);

/* int8 GEMM over the 4x4 micro-tile prepacked weight, int32 accumulation.
 * forward (transposed_b false): c[M, N_out] = cast(float(a[M, K] . W[N_out, K]^T) * a_scale[m] * b_scale[n] + bias[n]);
 * backward (transposed_b true): c[M, N_out] = cast(float(a[M, K] . W[K, N_out]) * a_scale[m]), b_scale and bias unused.
 * b_stride_kc / b_stride_out: micro-tile strides of one 4-wide step along the contraction / the output axis.
 * K_contract % 16 == 0, N_out % 4 == 0. output_dtype: 0 = fp16, 1 = bf16.
 * Replaces `launch_int8_scaled_mm`, reference csrc/hip_kernel_int8.cu:413-432. */
bool launch_int8_scaled_mm(const int8_t* a, const uint8_t* b, const float* a_scale, const float* b_scale, const uint16_t* bias,
                           uint16_t* c, int64_t M, int64_t N_out, int64_t K_contract, int64_t b_stride_kc, int64_t b_stride_out,
                           bool transposed_b, int block_warps_m, int block_warps_n, int unroll_k, int repeat_m, int repeat_n,
                           int output_dtype, feather_stream_t stream);

/* The same product over the released row-major weight w = [N, K] int8, without a prepack: the 128 x 128 byte boxes that the copy
 * engine fetches from w are tensor-core operands as they land (K-major forward, MN-major backward), so the kernel has no re-layout stage.
 * forward (transposed_b false): c[M, N] = cast(float(a[M, K] . w^T) * a_scale[m] * b_scale[n] + bias[n]);
 * backward (transposed_b true): c[M, K] = cast(float(a[M, N] . w) * a_scale[m]), b_scale and bias must be NULL.
 * a, w and c 16-byte aligned; K % 16 == 0, N % 4 == 0 (backward: N % 16 == 0). output_dtype: 0 = fp16, 1 = bf16.
 * No counterpart in the reference, whose kernels read the micro-tile prepack only (csrc/hip_kernel_int8.cu:413-432); it serves the
 * `weight_packed=False` calls of feather_ops/int8_convrot.py:344-397, for which the reference permutes the weight on every call. */
bool launch_int8_scaled_mm_plain(const int8_t* a, const int8_t* w, const float* a_scale, const float* b_scale, const uint16_t* bias,
                                 uint16_t* c, int64_t M, int64_t N, int64_t K, bool transposed_b, int output_dtype, feather_stream_t stream);

/* Output columns per tile (forward: a multiple of 16 in 128..256; backward: 128, 192 or 256) that launch_int8_scaled_mm_plain picks for a
 * product of M rows and N output columns when `pairs` CTA pairs are resident (74 on a B200): the width that minimises rounds of the
 * persistent grid x (width + a fixed part per tile). No counterpart in the reference (its tile tuples are picked in Python,
 * feather_ops/int8_convrot.py:28-82). */
int feather_int8_plain_tile_width(int64_t M, int64_t N, int pairs, bool transposed_b);

/* Diagnostic for the int8 GEMM's bounded waits, as feather_scaled_mm_status. No counterpart in the reference. */
int feather_int8_mm_status(uint32_t* out);

/* 3x3, stride 1, padding 1, NCHW conv2d with fp32 accumulation, bias added in fp32, one rounding.
 * x: [B, C_in, H, W]; wp: prepacked weight [ceil(C_in / 16) * 18, C_out, 8]; bias: [C_out] or NULL; y: [B, C_out, H, W];
 * one 16-bit dtype for all (is_bf16), C_in % 8 == 0. Tile = (warps_m, warps_n, repeat_m, repeat_n, rows).
 * Returns 0 on success, 1 for an unknown tile or an unsupported problem.
 * Replaces `feather_conv3x3_launch`, reference csrc/hip_conv2d_3x3.cu:561-575. */
int feather_conv3x3_launch(const void* x, const void* wp, const void* bias, void* y, int B, int C_in, int C_out, int H, int W, int has_bias,
                           int warps_m, int warps_n, int repeat_m, int repeat_n, int rows, int is_bf16, int prefetch, void* stream);

/* Diagnostic for the conv kernel's bounded waits, as feather_scaled_mm_status. No counterpart in the reference. */
int feather_conv3x3_status(uint32_t* out);

/* Self-test of the bounded device waits every tcgen05 kernel here is built on: one warp waits, for at most limit_cycles
 * SM clocks (clamped to [1e5, 4e9]), on a barrier that nothing arrives on, gives up, records it and the kernel ends
 * normally; a second waiter with a 64 times longer limit must leave through the abort flag. Synchronizes `stream`.
 * scratch: device memory for three uint32 (caller-owned). out (host, five uint32): [0] recorded wait site | tag << 8
 * (expected 2 | 5 << 8), [1] recorded block (0), [2] 1 if the first wait "completed" (expected 0), [3] the abort flag
 * (expected 1), [4] 1 if the second wait "completed" (expected 0). Returns 0 on success. Neither traps nor faults.
 * No counterpart in the reference (its kernels have no device-side waits). */
int feather_selftest_wait_runs_out(long long limit_cycles, uint32_t* scratch, uint32_t* out, feather_stream_t stream);

#ifdef __cplusplus
}
#endif

#endif /* FEATHER_OPS_B200_H_ */
