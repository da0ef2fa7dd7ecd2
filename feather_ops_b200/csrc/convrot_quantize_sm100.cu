// ConvRot activation quantizer for sm_100a: per row, rotate every 256-wide group by the unnormalized regular
// Hadamard h4 (x) h4 (x) h4 (x) h4, round once to the input dtype, take the row absmax, and emit int8 codes
// with one fp32 scale per row.
//
// B200 counterpart of `convrot_quantize_kernel` / `launch_convrot_quantize` in the reference's
// csrc/hip_kernel_int8.cu (:646-704 the radix-4 rotation, :779-865 the kernel, :869-924 the C ABI).
// The arithmetic is reproduced operation for operation, because the int8 codes have to be reproducible:
//
//   * a group lives in one warp, eight consecutive values per lane (element = lane * 8 + i);
//   * four radix-4 stages, one per base-4 digit of the element index, lowest digit first; with the four
//     members of a butterfly in index order a0..a3, the member with digit d becomes
//     ((a0 + a1) + a2) + a3 - 2 * a[3 - d], all in fp32;
//   * the result is rounded to the input dtype (RNE), the row maximum of |rounded| gives
//     divisor = max(amax / 127, 1e-30), codes are clamp(rint(v * (1 / divisor)), -127, 127) and the stored
//     scale is divisor / 16 when rotating (the 1 / sqrt(256) normalization folded in), divisor otherwise;
//   * without rotation an optional per-column multiplier is applied first and rounded to the input dtype.
//
// The pass is HBM bound (2 bytes in, 1 byte out per element): lanes load 16 bytes and store 8, a warp
// keeps its groups in registers between the absmax and the quantize step (up to four groups, i.e. rows up
// to 32768 wide with 32 warps), and wider rows recompute the groups from global memory, which is L2
// resident by then. One CTA owns one or more whole rows, so the only reduction is a per-row maximum
// across the CTA's warps.
#include "feather_host.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace feather {
namespace quant {

constexpr int kGroup = 256;
constexpr int kPerLane = 8;
constexpr int kMaxWarpsPerRow = 32;
constexpr int kCachedGroups = 4;

template <bool kFp16>
__device__ __forceinline__ float to_float(uint16_t bits) {
    if constexpr (kFp16) {
        return __half2float(__ushort_as_half(bits));
    } else {
        return __uint_as_float(static_cast<uint32_t>(bits) << 16);
    }
}

// Round to the input dtype (nearest even) and come back to fp32.
template <bool kFp16>
__device__ __forceinline__ float round_to_input(float v) {
    if constexpr (kFp16) {
        return __half2float(__float2half_rn(v));
    } else {
        return __bfloat162float(__float2bfloat16_rn(v));
    }
}

__device__ __forceinline__ float butterfly(float a0, float a1, float a2, float a3, int digit) {
    const float mirrored = digit == 0 ? a3 : digit == 1 ? a2 : digit == 2 ? a1 : a0;
    return (((a0 + a1) + a2) + a3) - 2.0f * mirrored;
}

// In-register group-256 regular Hadamard. `v[i]` is element `lane * 8 + i`.
__device__ __forceinline__ void hadamard256(float (&v)[kPerLane], int lane) {
    // digit 0 (stride 1): members are four consecutive registers
    {
        float r[kPerLane];
#pragma unroll
        for (int i = 0; i < kPerLane; ++i) {
            const int b = i & 4;
            r[i] = butterfly(v[b], v[b + 1], v[b + 2], v[b + 3], i & 3);
        }
#pragma unroll
        for (int i = 0; i < kPerLane; ++i) v[i] = r[i];
    }
    // digit 1 (stride 4): registers {q, q + 4} of the even lane, then of the odd lane
    {
        float other[kPerLane];
#pragma unroll
        for (int i = 0; i < kPerLane; ++i) other[i] = __shfl_xor_sync(0xffffffffu, v[i], 1);
        const bool odd = (lane & 1) != 0;
        float r[kPerLane];
#pragma unroll
        for (int i = 0; i < kPerLane; ++i) {
            const int q = i & 3;
            const float a0 = odd ? other[q] : v[q];
            const float a1 = odd ? other[q + 4] : v[q + 4];
            const float a2 = odd ? v[q] : other[q];
            const float a3 = odd ? v[q + 4] : other[q + 4];
            const int digit = (odd ? 2 : 0) + (i >> 2);
            r[i] = butterfly(a0, a1, a2, a3, digit);
        }
#pragma unroll
        for (int i = 0; i < kPerLane; ++i) v[i] = r[i];
    }
    // digits 2 and 3 (strides 16 and 64): members sit in the same register of four different lanes
#pragma unroll
    for (int stage = 0; stage < 2; ++stage) {
        const int lane_step = 2 << (2 * stage);
        const int digit = (lane >> (1 + 2 * stage)) & 3;
        float r[kPerLane];
#pragma unroll
        for (int i = 0; i < kPerLane; ++i) {
            const float a0 = __shfl_xor_sync(0xffffffffu, v[i], lane_step * digit);
            const float a1 = __shfl_xor_sync(0xffffffffu, v[i], lane_step * (digit ^ 1));
            const float a2 = __shfl_xor_sync(0xffffffffu, v[i], lane_step * (digit ^ 2));
            const float a3 = __shfl_xor_sync(0xffffffffu, v[i], lane_step * (digit ^ 3));
            r[i] = butterfly(a0, a1, a2, a3, digit);
        }
#pragma unroll
        for (int i = 0; i < kPerLane; ++i) v[i] = r[i];
    }
}

// Load one group's eight values of this lane, apply the column multiplier or the rotation, and round to
// the input dtype. Returns the lane's maximum magnitude through `amax`.
template <bool kFp16>
__device__ __forceinline__ void produce(const uint16_t* __restrict__ x_row, const float* __restrict__ col_scale, int base, int lane,
                                        bool rotate, float (&v)[kPerLane], float& amax) {
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(x_row + base));
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
        v[i] = to_float<kFp16>(static_cast<uint16_t>(w[i / 2] >> (16 * (i % 2))));
    }
    if (!rotate && col_scale != nullptr) {
        const float4 s0 = __ldg(reinterpret_cast<const float4*>(col_scale + base));
        const float4 s1 = __ldg(reinterpret_cast<const float4*>(col_scale + base + 4));
        const float s[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
        for (int i = 0; i < kPerLane; ++i) v[i] = round_to_input<kFp16>(v[i] * s[i]);
    }
    if (rotate) hadamard256(v, lane);
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
        v[i] = round_to_input<kFp16>(v[i]);
        amax = fmaxf(amax, fabsf(v[i]));
    }
}

__device__ __forceinline__ int code_of(float v, float inv_divisor) {
    return static_cast<int>(fminf(fmaxf(rintf(v * inv_divisor), -127.0f), 127.0f));
}

__device__ __forceinline__ void store_codes(int8_t* __restrict__ q_row, int base, const float (&v)[kPerLane], float inv_divisor) {
    uint32_t packed[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        uint32_t word = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            word |= (static_cast<uint32_t>(code_of(v[4 * h + i], inv_divisor)) & 0xffu) << (8 * i);
        }
        packed[h] = word;
    }
    *reinterpret_cast<uint2*>(q_row + base) = make_uint2(packed[0], packed[1]);
}

// blockDim = (32, warps_per_row, rows_per_cta). `kCache`: every warp owns at most `kCachedGroups` groups of
// its row and keeps them in registers across the row maximum.
template <bool kFp16, bool kCache>
__global__ void convrot_quantize_kernel(const uint16_t* __restrict__ x, const float* __restrict__ col_scale, int8_t* __restrict__ q,
                                        float* __restrict__ row_scale, int64_t M, int K, int groups, bool rotate) {
    __shared__ float warp_max[kMaxWarpsPerRow];  // rows_per_cta * warps_per_row <= 32 entries
    const int lane = static_cast<int>(threadIdx.x);
    const int warp = static_cast<int>(threadIdx.y);
    const int warps = static_cast<int>(blockDim.y);
    const int local_row = static_cast<int>(threadIdx.z);
    const int64_t row = static_cast<int64_t>(blockIdx.x) * blockDim.z + local_row;
    const bool live = row < M;
    const uint16_t* const x_row = x + (live ? row : 0) * K;
    int8_t* const q_row = q + (live ? row : 0) * K;

    float cached[kCache ? kCachedGroups : 1][kPerLane];
    float amax = 0.0f;
    if (live) {
        if constexpr (kCache) {
#pragma unroll
            for (int j = 0; j < kCachedGroups; ++j) {
                const int g = warp + j * warps;
                if (g < groups) produce<kFp16>(x_row, col_scale, g * kGroup + lane * kPerLane, lane, rotate, cached[j], amax);
            }
        } else {
            for (int g = warp; g < groups; g += warps) {
                produce<kFp16>(x_row, col_scale, g * kGroup + lane * kPerLane, lane, rotate, cached[0], amax);
            }
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    if (lane == 0) warp_max[local_row * warps + warp] = amax;
    __syncthreads();
    if (!live) return;
    float row_max = 0.0f;
    for (int w = 0; w < warps; ++w) row_max = fmaxf(row_max, warp_max[local_row * warps + w]);
    const float divisor = fmaxf(row_max / 127.0f, 1e-30f);
    if (warp == 0 && lane == 0) row_scale[row] = rotate ? divisor * 0.0625f : divisor;
    const float inv_divisor = 1.0f / divisor;

    if constexpr (kCache) {
#pragma unroll
        for (int j = 0; j < kCachedGroups; ++j) {
            const int g = warp + j * warps;
            if (g < groups) store_codes(q_row, g * kGroup + lane * kPerLane, cached[j], inv_divisor);
        }
    } else {
        for (int g = warp; g < groups; g += warps) {
            float unused = 0.0f;
            produce<kFp16>(x_row, col_scale, g * kGroup + lane * kPerLane, lane, rotate, cached[0], unused);
            store_codes(q_row, g * kGroup + lane * kPerLane, cached[0], inv_divisor);
        }
    }
}

}  // namespace quant
}  // namespace feather

// C ABI, same signature as the reference's `launch_convrot_quantize` (csrc/hip_kernel_int8.cu:869-878).
// x: [M, K] fp16 (input_fp16 != 0) or bf16, K a multiple of 256; col_scale: [K] or NULL (used only when
// rotate is false); q: [M, K] int8; row_scale: [M]. Returns false when K is not a multiple of 256 or the
// launch failed. x, q (16 bytes) and col_scale (16 bytes) must be aligned as torch allocations are.
extern "C" bool launch_convrot_quantize(const void* x, const float* col_scale, int8_t* q, float* row_scale, int64_t M, int64_t K,
                                        int input_fp16, bool rotate, cudaStream_t stream) {
    using namespace feather::quant;
    if (K <= 0 || K % kGroup != 0 || K > (1ll << 30) || M < 0) return false;
    if (M == 0) return true;
    const int groups = static_cast<int>(K / kGroup);
    const int warps = groups < kMaxWarpsPerRow ? groups : kMaxWarpsPerRow;
    // short rows share a CTA so that a CTA is at least eight warps
    int rows_per_cta = 8 / warps;
    if (rows_per_cta < 1) rows_per_cta = 1;
    const bool cache = groups <= warps * kCachedGroups;
    const dim3 block(32, warps, rows_per_cta);
    const dim3 grid(static_cast<unsigned>((M + rows_per_cta - 1) / rows_per_cta));
    const uint16_t* const xp = static_cast<const uint16_t*>(x);
    if (input_fp16 != 0) {
        if (cache) {
            convrot_quantize_kernel<true, true><<<grid, block, 0, stream>>>(xp, col_scale, q, row_scale, M, static_cast<int>(K), groups, rotate);
        } else {
            convrot_quantize_kernel<true, false><<<grid, block, 0, stream>>>(xp, col_scale, q, row_scale, M, static_cast<int>(K), groups, rotate);
        }
    } else {
        if (cache) {
            convrot_quantize_kernel<false, true><<<grid, block, 0, stream>>>(xp, col_scale, q, row_scale, M, static_cast<int>(K), groups, rotate);
        } else {
            convrot_quantize_kernel<false, false><<<grid, block, 0, stream>>>(xp, col_scale, q, row_scale, M, static_cast<int>(K), groups, rotate);
        }
    }
    return cudaGetLastError() == cudaSuccess;
}
