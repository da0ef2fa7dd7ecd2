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

/* Diagnostic: reads and clears the record that the scaled_mm kernel's bounded device waits report into.
 * out[0] = 0 when every wait completed, else the wait site; out[1] = block index. Synchronizes the device.
 * Returns 0 on success. No counterpart in the reference (its kernels have no device-side waits). */
int feather_scaled_mm_status(uint32_t* out);

#ifdef __cplusplus
}
#endif

#endif /* FEATHER_OPS_B200_H_ */
