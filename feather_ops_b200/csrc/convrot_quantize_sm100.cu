// ConvRot activation quantizer for sm_100a: per row, rotate every 256-wide group by the unnormalized regular
// Hadamard h4 (x) h4 (x) h4 (x) h4, round once to the input dtype, take the row absmax, and emit int8 codes
// with one fp32 scale per row.
//
// B200 counterpart of `convrot_quantize_kernel` / `launch_convrot_quantize` in the reference's
// csrc/hip_kernel_int8.cu (:646-704 the radix-4 rotation, :779-865 the kernel, :869-924 the C ABI).
// The arithmetic is reproduced operation for operation, because the int8 codes have to be reproducible:
//
//   * four radix-4 stages, one per base-4 digit of the element index, lowest digit first; with the four
//     members of a butterfly in index order a0..a3, the member with digit d becomes
//     ((a0 + a1) + a2) + a3 - 2 * a[3 - d], all in fp32;
//   * the result is rounded to the input dtype (RNE), the row maximum of |rounded| gives
//     divisor = max(amax / 127, 1e-30), codes are clamp(rint(v * (1 / divisor)), -127, 127) and the stored
//     scale is divisor / 16 when rotating (the 1 / sqrt(256) normalization folded in), divisor otherwise;
//   * without rotation an optional per-column multiplier is applied first and rounded to the input dtype.
//
// Data movement is where this differs from the reference. There a group lives in one wave, eight values per
// lane, and two of the four stages fetch their butterfly members with cross-lane shuffles (72 shuffles per
// lane and group). On B200 that makes the pass shuffle bound (one warp shuffle per clock and SM) at about an
// eighth of the HBM rate. Here a group lives in a half warp, sixteen consecutive values per lane, so two
// digits are inside the lane: stages 0 and 1 run on registers, the 16 x 16 value matrix is transposed
// through (bank-conflict-free, padded) shared memory, stages 2 and 3 run on registers again, and the
// rounded 16-bit results are transposed back so that every lane ends up with the sixteen consecutive
// outputs it stores as one 16-byte vector. No shuffle is used for the rotation.
//
// The floor of the pass is HBM traffic (2 bytes in, 1 byte out per element); as measured it is bound by instruction
// issue (about 26 warp instructions per value, a third of them the fp32 butterflies). A warp keeps its groups as packed 16-bit
// values in registers between the absmax and the quantize step (up to four rounds of two groups, i.e. rows
// up to 32768 wide with 16 warps per row); wider rows recompute the groups from global memory, which is L2
// resident by then. One CTA owns one or more whole rows, so the only reduction is a per-row maximum across
// the CTA's warps.
#include "feather_host.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace feather {
namespace quant {

constexpr int kGroup = 256;
constexpr int kPerLane = 16;          // consecutive values of one lane
constexpr int kMaxWarpsPerRow = 16;   // a warp handles two groups per round
constexpr int kCachedRounds = 4;
constexpr int kMaxWarpsPerCta = 16;
constexpr int kPadded = 20;           // row pitch (in words) of the transpose buffer: rows start on 16 bytes, and both a
                                      // quarter warp's 16-byte row stores and a half warp's column loads are conflict free
constexpr int kRegionWords = 16 * kPadded + 16;  // 16 mod 32: the two half warps of a warp read different banks

template <bool kFp16>
__device__ __forceinline__ float to_float(uint16_t bits) {
    if constexpr (kFp16) {
        return __half2float(__ushort_as_half(bits));
    } else {
        return __uint_as_float(static_cast<uint32_t>(bits) << 16);
    }
}

template <bool kFp16>
__device__ __forceinline__ uint16_t to_bits(float v) {
    if constexpr (kFp16) {
        return __half_as_ushort(__float2half_rn(v));
    } else {
        return __bfloat16_as_ushort(__float2bfloat16_rn(v));
    }
}

// Two values rounded to the input dtype (nearest even), packed low | high << 16. One instruction on the FMA
// pipe; the one-value conversions go through the quarter-rate conversion unit.
template <bool kFp16>
__device__ __forceinline__ uint32_t to_bits2(float lo, float hi) {
    if constexpr (kFp16) {
        const __half2 h = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<const uint32_t*>(&h);
    } else {
        const __nv_bfloat162 b = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<const uint32_t*>(&b);
    }
}

// Round to the input dtype (nearest even) and come back to fp32.
template <bool kFp16>
__device__ __forceinline__ float round_to_input(float v) {
    return to_float<kFp16>(to_bits<kFp16>(v));
}

// One radix-4 butterfly in place: member d becomes ((a0 + a1) + a2) + a3 - 2 * a[3 - d]. The sum is formed once,
// in the reference's order; 2 * a is exact, so the fused multiply-add rounds exactly like the subtraction.
__device__ __forceinline__ void butterfly4(float& a0, float& a1, float& a2, float& a3) {
    const float sum = ((a0 + a1) + a2) + a3;
    const float r0 = fmaf(-2.0f, a3, sum);
    const float r1 = fmaf(-2.0f, a2, sum);
    const float r2 = fmaf(-2.0f, a1, sum);
    const float r3 = fmaf(-2.0f, a0, sum);
    a0 = r0;
    a1 = r1;
    a2 = r2;
    a3 = r3;
}

// Two radix-4 stages over the sixteen values of a lane: first the low index digit (members are four
// consecutive registers), then the high one (members are registers q, q + 4, q + 8, q + 12).
__device__ __forceinline__ void two_stages(float (&v)[kPerLane]) {
#pragma unroll
    for (int b = 0; b < kPerLane; b += 4) butterfly4(v[b], v[b + 1], v[b + 2], v[b + 3]);
#pragma unroll
    for (int q = 0; q < 4; ++q) butterfly4(v[q], v[q + 4], v[q + 8], v[q + 12]);
}

// Produce one group for one half warp: load this lane's sixteen consecutive values, apply the column
// multiplier or the rotation, round to the input dtype. `packed` receives the lane's sixteen consecutive
// results as 16-bit patterns, `amax` the running maximum magnitude before that rounding. `region` is this half warp's transpose
// buffer. Every lane of the warp must call this together (it synchronizes the warp); `live` says whether
// the half warp has a group at all.
// This lane's sixteen consecutive input values as two 16-byte loads (zeros when the half warp has no group).
__device__ __forceinline__ void load_raw(const uint16_t* __restrict__ x_row, int base, bool live, uint4 (&raw)[2]) {
    raw[0] = make_uint4(0u, 0u, 0u, 0u);
    raw[1] = make_uint4(0u, 0u, 0u, 0u);
    if (live) {
        raw[0] = __ldg(reinterpret_cast<const uint4*>(x_row + base));
        raw[1] = __ldg(reinterpret_cast<const uint4*>(x_row + base + 8));
    }
}

template <bool kFp16>
__device__ __forceinline__ void produce_from(const uint4 (&raw)[2], const float* __restrict__ col_scale, int base, int l, bool live, bool rotate,
                                             float* region, uint32_t (&packed)[8], float& amax) {
    float v[kPerLane];
    {
        const uint32_t w[8] = {raw[0].x, raw[0].y, raw[0].z, raw[0].w, raw[1].x, raw[1].y, raw[1].z, raw[1].w};
#pragma unroll
        for (int i = 0; i < kPerLane; ++i) v[i] = to_float<kFp16>(static_cast<uint16_t>(w[i / 2] >> (16 * (i % 2))));
    }
    if (!rotate) {
        if (col_scale != nullptr && live) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const float4 s = __ldg(reinterpret_cast<const float4*>(col_scale + base + 4 * c));
                v[4 * c] = round_to_input<kFp16>(v[4 * c] * s.x);
                v[4 * c + 1] = round_to_input<kFp16>(v[4 * c + 1] * s.y);
                v[4 * c + 2] = round_to_input<kFp16>(v[4 * c + 2] * s.z);
                v[4 * c + 3] = round_to_input<kFp16>(v[4 * c + 3] * s.w);
            }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            amax = fmaxf(amax, fmaxf(fabsf(v[2 * i]), fabsf(v[2 * i + 1])));
            packed[i] = to_bits2<kFp16>(v[2 * i], v[2 * i + 1]);
        }
        return;
    }
    two_stages(v);  // digits 0 and 1: element index = l * 16 + i
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        *reinterpret_cast<float4*>(region + l * kPadded + 4 * c) = make_float4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
    }
    __syncwarp();
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) v[i] = region[i * kPadded + l];  // now element index = i * 16 + l
    __syncwarp();
    two_stages(v);  // digits 2 and 3
    uint16_t* const halves = reinterpret_cast<uint16_t*>(region);
#pragma unroll
    for (int i = 0; i < kPerLane; i += 2) {
        amax = fmaxf(amax, fmaxf(fabsf(v[i]), fabsf(v[i + 1])));
        const uint32_t pair = to_bits2<kFp16>(v[i], v[i + 1]);
        halves[i * 16 + l] = static_cast<uint16_t>(pair & 0xffffu);
        halves[(i + 1) * 16 + l] = static_cast<uint16_t>(pair >> 16);
    }
    __syncwarp();
    const uint4 lo = *reinterpret_cast<const uint4*>(halves + l * 16);
    const uint4 hi = *reinterpret_cast<const uint4*>(halves + l * 16 + 8);
    __syncwarp();
    packed[0] = lo.x;
    packed[1] = lo.y;
    packed[2] = lo.z;
    packed[3] = lo.w;
    packed[4] = hi.x;
    packed[5] = hi.y;
    packed[6] = hi.z;
    packed[7] = hi.w;
}

template <bool kFp16>
__device__ __forceinline__ void produce(const uint16_t* __restrict__ x_row, const float* __restrict__ col_scale, int base, int l, bool live,
                                        bool rotate, float* region, uint32_t (&packed)[8], float& amax) {
    uint4 raw[2];
    load_raw(x_row, base, live, raw);
    produce_from<kFp16>(raw, col_scale, base, l, live, rotate, region, packed, amax);
}

// clamp(rint(v * inv_divisor), -127, 127) as an integer in the low byte of the result. The clamp bounds are
// integers, so clamping first and rounding second gives the same value; adding 1.5 * 2^23 rounds to the nearest
// even integer exactly as rint does (|value| <= 127) and leaves it, in two's complement, in the low mantissa
// bits. No conversion instruction (quarter rate) is needed.
// Only the lower clamp is written out. |v| never exceeds the row maximum, so the product is at most
// 127 * (1 + 2^-22) in magnitude, which rounds to 127 without any clamp; the other possible product is NaN
// (a NaN input, or an infinite row maximum times the zero that 1 / inf gives), and fmaxf(NaN, -127) = -127 is
// what the two-sided clamp returned for it too.
__device__ __forceinline__ uint32_t code_of(float v, float inv_divisor) {
    const float clamped = fmaxf(v * inv_divisor, -127.0f);
    return __float_as_uint(clamped + 12582912.0f);
}

template <bool kFp16>
__device__ __forceinline__ void store_codes(int8_t* __restrict__ q_row, int base, const uint32_t (&packed)[8], float inv_divisor) {
    uint32_t out[4];
#pragma unroll
    for (int w = 0; w < 4; ++w) {
        const uint32_t p0 = packed[2 * w];
        const uint32_t p1 = packed[2 * w + 1];
        const uint32_t c0 = code_of(to_float<kFp16>(static_cast<uint16_t>(p0 & 0xffffu)), inv_divisor);
        const uint32_t c1 = code_of(to_float<kFp16>(static_cast<uint16_t>(p0 >> 16)), inv_divisor);
        const uint32_t c2 = code_of(to_float<kFp16>(static_cast<uint16_t>(p1 & 0xffffu)), inv_divisor);
        const uint32_t c3 = code_of(to_float<kFp16>(static_cast<uint16_t>(p1 >> 16)), inv_divisor);
        // low bytes of c0..c3 -> one word
        out[w] = __byte_perm(__byte_perm(c0, c1, 0x0040u), __byte_perm(c2, c3, 0x0040u), 0x5410u);
    }
    *reinterpret_cast<uint4*>(q_row + base) = make_uint4(out[0], out[1], out[2], out[3]);
}

// blockDim = (32, warps_per_row, rows_per_cta). A warp handles the groups 2 * (warp + j * warps) + half of its
// row in round j. `kCache`: at most kCachedRounds rounds, kept in registers across the row maximum.
template <bool kFp16, bool kCache>
__global__ void __launch_bounds__(32 * kMaxWarpsPerCta) convrot_quantize_kernel(const uint16_t* __restrict__ x, const float* __restrict__ col_scale,
                                                                               int8_t* __restrict__ q, float* __restrict__ row_scale, int64_t M, int K,
                                                                               int groups, bool rotate) {
    extern __shared__ __align__(16) float regions[];  // 2 * kRegionWords per warp of the CTA
    __shared__ float warp_max[kMaxWarpsPerCta];
    const int lane = static_cast<int>(threadIdx.x);
    const int half = lane >> 4;
    const int l = lane & 15;
    const int warp = static_cast<int>(threadIdx.y);
    const int warps = static_cast<int>(blockDim.y);
    const int local_row = static_cast<int>(threadIdx.z);
    const int cta_warp = local_row * warps + warp;
    float* const region = regions + (cta_warp * 2 + half) * kRegionWords;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * blockDim.z + local_row;
    const bool row_live = row < M;
    const uint16_t* const x_row = x + (row_live ? row : 0) * K;
    int8_t* const q_row = q + (row_live ? row : 0) * K;
    const int rounds = (groups + 2 * warps - 1) / (2 * warps);

    uint32_t cached[kCache ? kCachedRounds : 1][8];
    float amax = 0.0f;
    if constexpr (kCache) {
#pragma unroll
        for (int j = 0; j < kCachedRounds; ++j) {
            if (j < rounds) {
                const int g = 2 * (warp + j * warps) + half;
                produce<kFp16>(x_row, col_scale, g * kGroup + l * kPerLane, l, row_live && g < groups, rotate, region, cached[j], amax);
            }
        }
    } else {
        for (int j = 0; j < rounds; ++j) {
            const int g = 2 * (warp + j * warps) + half;
            produce<kFp16>(x_row, col_scale, g * kGroup + l * kPerLane, l, row_live && g < groups, rotate, region, cached[0], amax);
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    if (lane == 0) warp_max[cta_warp] = amax;
    __syncthreads();
    float row_max = 0.0f;
    for (int w = 0; w < warps; ++w) row_max = fmaxf(row_max, warp_max[local_row * warps + w]);
    // the maxima were taken before the rounding to the input dtype: rounding is monotonic, so the maximum of the
    // rounded magnitudes is the rounded maximum
    row_max = round_to_input<kFp16>(row_max);
    const float divisor = fmaxf(row_max / 127.0f, 1e-30f);
    if (row_live && warp == 0 && lane == 0) row_scale[row] = rotate ? divisor * 0.0625f : divisor;
    const float inv_divisor = 1.0f / divisor;

    if constexpr (kCache) {
#pragma unroll
        for (int j = 0; j < kCachedRounds; ++j) {
            const int g = 2 * (warp + j * warps) + half;
            if (j < rounds && row_live && g < groups) store_codes<kFp16>(q_row, g * kGroup + l * kPerLane, cached[j], inv_divisor);
        }
    } else {
        for (int j = 0; j < rounds; ++j) {
            const int g = 2 * (warp + j * warps) + half;
            float unused = 0.0f;
            produce<kFp16>(x_row, col_scale, g * kGroup + l * kPerLane, l, row_live && g < groups, rotate, region, cached[0], unused);
            if (row_live && g < groups) store_codes<kFp16>(q_row, g * kGroup + l * kPerLane, cached[0], inv_divisor);
        }
    }
}

// ---------------------------------------------------------------------------------------------------------
// Streaming kernel for rows up to 4 * 256 * blockDim.y wide (one round: every half warp has at most one PAIR of
// groups per row). A fixed number of resident CTAs walk the rows, and a CTA asks for its next row's values before it
// works on the current one: with one row per CTA lifetime the pass ran at the pace of one HBM latency per wave of
// CTAs, not at the HBM rate.
//
// The pass is bound by instruction issue, so this kernel halves the instructions of the arithmetic: a half warp
// rotates TWO adjacent groups (A and B) of its row at once, value i of A and value i of B sitting in one 64-bit
// register pair, and every butterfly runs on the packed fp32 pair instructions of sm_100a (add.f32x2, fma.rn.f32x2:
// two independent IEEE fp32 results per instruction, so every bit is what the scalar instruction gives). A pair
// never holds two members of one butterfly (its halves belong to different groups), and both halves always have the
// same member index, so the reference's operation order holds in each half. The pair also travels as a unit through
// the transposes: 8 bytes forward (16-byte stores, 8-byte column loads), and as one 32-bit word of two rounded
// 16-bit values back (4-byte stores, 16-byte row loads), so both transposes move twice the values per instruction.
// The per-row bookkeeping is kept short: the warp maximum is one `redux` on the bit pattern (magnitudes are
// non-negative, so they order like unsigned integers), the row maximum one shared-memory atomic per warp and one
// load per thread, and the two row buffers swap roles by unrolling.
// ---------------------------------------------------------------------------------------------------------
constexpr int kMaxRowsPerCta = 8;
constexpr int kPairPitchBytes = 16 * 8 + 16;           // forward transpose: a lane's sixteen 8-byte pairs + 16 bytes, so that the
                                                       // 16-byte stores of eight lanes fall into eight different bank groups
constexpr int kPairRegionBytes = 16 * kPairPitchBytes + 64;   // per half warp; the + 64 puts the two half warps of a warp 16 banks apart
constexpr int kBackPitchWords = 20;                    // backward transpose: rows of sixteen words, pitch 20 (16-byte row loads conflict free)
static_assert(16 * kBackPitchWords * 4 <= kPairRegionBytes, "the backward transpose reuses the forward buffer");

using f32x2 = unsigned long long;   // two fp32 values in one 64-bit register pair: low = group A, high = group B

__device__ __forceinline__ f32x2 pack2(float lo, float hi) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}

__device__ __forceinline__ void unpack2(f32x2 p, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(p));
}

__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
    f32x2 r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}

__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
    f32x2 r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}

__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
    f32x2 r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}

// butterfly4 on both halves of four pairs
__device__ __forceinline__ void butterfly4_pair(f32x2& a0, f32x2& a1, f32x2& a2, f32x2& a3, f32x2 minus_two) {
    const f32x2 sum = add2(add2(add2(a0, a1), a2), a3);
    const f32x2 r0 = fma2(minus_two, a3, sum);
    const f32x2 r1 = fma2(minus_two, a2, sum);
    const f32x2 r2 = fma2(minus_two, a1, sum);
    const f32x2 r3 = fma2(minus_two, a0, sum);
    a0 = r0;
    a1 = r1;
    a2 = r2;
    a3 = r3;
}

__device__ __forceinline__ void two_stages_pair(f32x2 (&v)[kPerLane], f32x2 minus_two) {
#pragma unroll
    for (int b = 0; b < kPerLane; b += 4) butterfly4_pair(v[b], v[b + 1], v[b + 2], v[b + 3], minus_two);
#pragma unroll
    for (int q = 0; q < 4; ++q) butterfly4_pair(v[q], v[q + 4], v[q + 8], v[q + 12], minus_two);
}

// Both halves of a pair rounded to the input dtype: group A in the low 16 bits, group B in the high 16 bits.
template <bool kFp16>
__device__ __forceinline__ uint32_t round_pair(f32x2 p) {
    float a, b;
    unpack2(p, a, b);
    return to_bits2<kFp16>(a, b);
}

template <bool kFp16, bool kRotate>
struct StreamRow {
    const float* col_scale;
    uint8_t* region;         // this half warp's transpose buffer
    uint32_t* row_max_bits;  // [3][kMaxRowsPerCta]: slot t % 3 collects row t, slot (t + 1) % 3 is cleared meanwhile
    float* row_scale;
    int l;
    int base_a;              // first element of this lane's sixteen values in group A; group B is kGroup further
    int local_row;
    bool a_live;
    bool b_live;
    bool writes_scale;

    // The lane's sixteen values of A and of B, paired: v[i] = (A[base_a + i], B[base_a + kGroup + i]) as fp32.
    __device__ __forceinline__ void load_pairs(const uint4 (&raw_a)[2], const uint4 (&raw_b)[2], f32x2 (&v)[kPerLane]) const {
        const uint32_t wa[8] = {raw_a[0].x, raw_a[0].y, raw_a[0].z, raw_a[0].w, raw_a[1].x, raw_a[1].y, raw_a[1].z, raw_a[1].w};
        const uint32_t wb[8] = {raw_b[0].x, raw_b[0].y, raw_b[0].z, raw_b[0].w, raw_b[1].x, raw_b[1].y, raw_b[1].z, raw_b[1].w};
#pragma unroll
        for (int i = 0; i < kPerLane; ++i) {
            v[i] = pack2(to_float<kFp16>(static_cast<uint16_t>(wa[i / 2] >> (16 * (i % 2)))), to_float<kFp16>(static_cast<uint16_t>(wb[i / 2] >> (16 * (i % 2)))));
        }
    }

    // One row: `raw_a` / `raw_b` hold its values, `q_row` / `row` say where the codes and the scale go.
    __device__ __forceinline__ void run(const uint4 (&raw_a)[2], const uint4 (&raw_b)[2], bool row_live, int8_t* q_row, int64_t row, uint32_t turn) const {
        f32x2 v[kPerLane];
        load_pairs(raw_a, raw_b, v);
        uint32_t words[kPerLane];   // element i of the lane's sixteen consecutive outputs: A in the low half, B in the high half
        float amax = 0.0f;
        if constexpr (kRotate) {
            const f32x2 minus_two = pack2(-2.0f, -2.0f);
            two_stages_pair(v, minus_two);   // digits 0 and 1: element index = l * 16 + i
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                *reinterpret_cast<ulonglong2*>(region + l * kPairPitchBytes + 16 * c) = make_ulonglong2(v[2 * c], v[2 * c + 1]);
            }
            __syncwarp();
#pragma unroll
            for (int i = 0; i < kPerLane; ++i) v[i] = *reinterpret_cast<const f32x2*>(region + i * kPairPitchBytes + 8 * l);   // now element index = i * 16 + l
            __syncwarp();
            two_stages_pair(v, minus_two);   // digits 2 and 3
            uint32_t* const back = reinterpret_cast<uint32_t*>(region);
#pragma unroll
            for (int i = 0; i < kPerLane; ++i) {
                float a, b;
                unpack2(v[i], a, b);
                amax = fmaxf(amax, fmaxf(fabsf(a), fabsf(b)));
                back[i * kBackPitchWords + l] = to_bits2<kFp16>(a, b);
            }
            __syncwarp();
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const uint4 w4 = *reinterpret_cast<const uint4*>(back + l * kBackPitchWords + 4 * c);
                words[4 * c] = w4.x;
                words[4 * c + 1] = w4.y;
                words[4 * c + 2] = w4.z;
                words[4 * c + 3] = w4.w;
            }
            __syncwarp();
        } else {
            if (col_scale != nullptr) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const float4 sa = a_live ? __ldg(reinterpret_cast<const float4*>(col_scale + base_a + 4 * c)) : make_float4(0.f, 0.f, 0.f, 0.f);
                    const float4 sb = b_live ? __ldg(reinterpret_cast<const float4*>(col_scale + base_a + kGroup + 4 * c)) : make_float4(0.f, 0.f, 0.f, 0.f);
                    v[4 * c] = mul2(v[4 * c], pack2(sa.x, sb.x));
                    v[4 * c + 1] = mul2(v[4 * c + 1], pack2(sa.y, sb.y));
                    v[4 * c + 2] = mul2(v[4 * c + 2], pack2(sa.z, sb.z));
                    v[4 * c + 3] = mul2(v[4 * c + 3], pack2(sa.w, sb.w));
                }
            }
#pragma unroll
            for (int i = 0; i < kPerLane; ++i) {
                float a, b;
                unpack2(v[i], a, b);
                amax = fmaxf(amax, fmaxf(fabsf(a), fabsf(b)));
                words[i] = to_bits2<kFp16>(a, b);
            }
        }
        const uint32_t warp_bits = __reduce_max_sync(0xffffffffu, __float_as_uint(amax));
        uint32_t* const slot = row_max_bits + turn * kMaxRowsPerCta + local_row;
        if (threadIdx.x == 0) atomicMax(slot, warp_bits);
        if (threadIdx.x == 1 && threadIdx.y == 0) row_max_bits[(turn == 2u ? 0u : turn + 1u) * kMaxRowsPerCta + local_row] = 0u;
        __syncthreads();
        // maxima were taken before the rounding to the input dtype, which is monotonic
        const float row_max = round_to_input<kFp16>(__uint_as_float(*slot));
        const float divisor = fmaxf(row_max / 127.0f, 1e-30f);
        if (row_live && writes_scale) row_scale[row] = kRotate ? divisor * 0.0625f : divisor;
        if (!row_live) return;
        // codes: clamp(rint(v / divisor)) for both halves of every word (see code_of); four words give four codes of A and four of B
        const float inv = 1.0f / divisor;
        const f32x2 inv2 = pack2(inv, inv);
        const f32x2 magic2 = pack2(12582912.0f, 12582912.0f);
        uint32_t out_a[4], out_b[4];
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            uint32_t ca[4], cb[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t word = words[4 * w + j];
                float a, b;
                if constexpr (kFp16) {
                    const float2 ab = __half22float2(*reinterpret_cast<const __half2*>(&word));
                    a = ab.x;
                    b = ab.y;
                } else {
                    a = __uint_as_float(word << 16);
                    b = __uint_as_float(word & 0xffff0000u);
                }
                float pa, pb;
                // The clamp sits between the multiplication and the addition on purpose: with the two packed instructions back
                // to back the assembler contracts them into one fused multiply-add, which rounds once and flips the codes
                // whose product rounds onto a .5 boundary (measured: 4382 of 12.6 M codes of the benchmark activation).
                unpack2(mul2(pack2(a, b), inv2), pa, pb);
                unpack2(add2(pack2(fmaxf(pa, -127.0f), fmaxf(pb, -127.0f)), magic2), pa, pb);
                ca[j] = __float_as_uint(pa);
                cb[j] = __float_as_uint(pb);
            }
            out_a[w] = __byte_perm(__byte_perm(ca[0], ca[1], 0x0040u), __byte_perm(ca[2], ca[3], 0x0040u), 0x5410u);
            out_b[w] = __byte_perm(__byte_perm(cb[0], cb[1], 0x0040u), __byte_perm(cb[2], cb[3], 0x0040u), 0x5410u);
        }
        if (a_live) *reinterpret_cast<uint4*>(q_row + base_a) = make_uint4(out_a[0], out_a[1], out_a[2], out_a[3]);
        if (b_live) *reinterpret_cast<uint4*>(q_row + base_a + kGroup) = make_uint4(out_b[0], out_b[1], out_b[2], out_b[3]);
    }
};

// blockDim = (32, warps_per_row, rows_per_cta); half warp h of warp w owns groups 4 w + 2 h (A) and 4 w + 2 h + 1 (B) of its row.
template <bool kFp16, bool kRotate>
__global__ void __launch_bounds__(32 * kMaxWarpsPerCta) convrot_quantize_stream_kernel(const uint16_t* __restrict__ x, const float* __restrict__ col_scale,
                                                                                      int8_t* __restrict__ q, float* __restrict__ row_scale, int64_t M, int K,
                                                                                      int groups) {
    extern __shared__ __align__(16) uint8_t pair_regions[];  // kPairRegionBytes per half warp of the CTA
    __shared__ uint32_t row_max_bits[3 * kMaxRowsPerCta];
    const int lane = static_cast<int>(threadIdx.x);
    const int half = lane >> 4;
    const int warp = static_cast<int>(threadIdx.y);
    const int warps = static_cast<int>(blockDim.y);
    const int local_row = static_cast<int>(threadIdx.z);
    const int group_a = 4 * warp + 2 * half;

    StreamRow<kFp16, kRotate> ctx;
    ctx.col_scale = col_scale;
    ctx.region = pair_regions + ((local_row * warps + warp) * 2 + half) * kPairRegionBytes;
    ctx.row_max_bits = row_max_bits;
    ctx.row_scale = row_scale;
    ctx.l = lane & 15;
    ctx.base_a = group_a * kGroup + ctx.l * kPerLane;
    ctx.local_row = local_row;
    ctx.a_live = group_a < groups;
    ctx.b_live = group_a + 1 < groups;
    ctx.writes_scale = warp == 0 && lane == 0;

    const int flat = (local_row * warps + warp) * 32 + lane;
    if (flat < 3 * kMaxRowsPerCta) row_max_bits[flat] = 0u;
    __syncthreads();

    const int64_t row_step = static_cast<int64_t>(gridDim.x) * blockDim.z;
    const int64_t step_elems = row_step * K;
    int64_t row = static_cast<int64_t>(blockIdx.x) * blockDim.z + local_row;
    int64_t first = static_cast<int64_t>(blockIdx.x) * blockDim.z;   // the CTA's lowest row: the same for all its threads
    const uint16_t* x_row = x + (row < M ? row : 0) * K;
    int8_t* q_row = q + (row < M ? row : 0) * K;
    uint4 raw_a0[2], raw_b0[2], raw_a1[2], raw_b1[2];
    load_raw(x_row, ctx.base_a, ctx.a_live && row < M, raw_a0);
    load_raw(x_row, ctx.base_a + kGroup, ctx.b_live && row < M, raw_b0);
    // The GEMM that consumes the codes may be launched as a programmatic dependent: let it set itself up (barriers, tensor
    // memory, descriptors) on SMs as they fall free; it waits for this grid to complete before it reads a code or a scale.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    uint32_t turn = 0;
    while (first < M) {
        load_raw(x_row + step_elems, ctx.base_a, ctx.a_live && row + row_step < M, raw_a1);
        load_raw(x_row + step_elems, ctx.base_a + kGroup, ctx.b_live && row + row_step < M, raw_b1);
        ctx.run(raw_a0, raw_b0, row < M, q_row, row, turn);
        turn = turn == 2u ? 0u : turn + 1u;
        first += row_step;
        row += row_step;
        x_row += step_elems;
        q_row += step_elems;
        if (first >= M) break;
        load_raw(x_row + step_elems, ctx.base_a, ctx.a_live && row + row_step < M, raw_a0);
        load_raw(x_row + step_elems, ctx.base_a + kGroup, ctx.b_live && row + row_step < M, raw_b0);
        ctx.run(raw_a1, raw_b1, row < M, q_row, row, turn);
        turn = turn == 2u ? 0u : turn + 1u;
        first += row_step;
        row += row_step;
        x_row += step_elems;
        q_row += step_elems;
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
    const uint16_t* const xp = static_cast<const uint16_t*>(x);
    const int k = static_cast<int>(K);
    if (groups <= 4 * kMaxWarpsPerRow) {
        // One round per row (a half warp takes two adjacent groups): resident CTAs walk the rows and prefetch the next one.
        const int warps = (groups + 3) / 4;
        // Small CTAs: every row costs its CTA one barrier (the row maximum), and many small CTAs per SM hide it better than
        // few large ones (4096 x 3072: 10.6 us with one row = three warps per CTA, 11.7 with three rows, 12.6 with four).
        // Rows narrower than three warps share a CTA so that a CTA is at least four warps.
        const int rows_per_cta = warps >= 3 ? 1 : 4 / warps;
        const dim3 block(32, warps, rows_per_cta);
        const int threads = 32 * warps * rows_per_cta;
        const size_t smem = static_cast<size_t>(warps) * rows_per_cta * 2 * kPairRegionBytes;
        using StreamKernel = void (*)(const uint16_t*, const float*, int8_t*, float*, int64_t, int, int);
        const StreamKernel kernel = input_fp16 != 0 ? (rotate ? convrot_quantize_stream_kernel<true, true> : convrot_quantize_stream_kernel<true, false>)
                                                    : (rotate ? convrot_quantize_stream_kernel<false, true> : convrot_quantize_stream_kernel<false, false>);
        // CTAs resident per SM for this block shape (the shared-memory size follows from it), asked once per device and shape
        static feather::PerDeviceState resident_per_sm[2][2][kMaxWarpsPerCta + 1];
        const int per_sm = resident_per_sm[input_fp16 != 0 ? 1 : 0][rotate ? 1 : 0][threads / 32].get([&] {
            if (smem > 48 * 1024 && cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024) != cudaSuccess) return 0;
            int value = 0;
            if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&value, kernel, threads, smem) != cudaSuccess || value < 1) {
                (void)cudaGetLastError();
                value = 1;
            }
            return value;
        });
        if (per_sm <= 0) return false;
        const int64_t resident = static_cast<int64_t>(per_sm) * feather::device_info().sm_count;
        const int64_t wanted = (M + rows_per_cta - 1) / rows_per_cta;
        const dim3 stream_grid(static_cast<unsigned>(wanted < resident ? wanted : resident));
        kernel<<<stream_grid, block, smem, stream>>>(xp, col_scale, q, row_scale, M, k, groups);
        return cudaGetLastError() == cudaSuccess;
    }
    // wider rows: several rounds per row, a half warp takes one group per round
    const int pairs = (groups + 1) / 2;
    const int warps = pairs < kMaxWarpsPerRow ? pairs : kMaxWarpsPerRow;
    const int rows_per_cta = 1;
    const bool cache = groups <= 2 * warps * kCachedRounds;
    const dim3 block(32, warps, rows_per_cta);
    const dim3 grid(static_cast<unsigned>((M + rows_per_cta - 1) / rows_per_cta));
    const size_t smem = static_cast<size_t>(warps) * rows_per_cta * 2 * kRegionWords * sizeof(float);
    if (input_fp16 != 0) {
        if (cache) {
            convrot_quantize_kernel<true, true><<<grid, block, smem, stream>>>(xp, col_scale, q, row_scale, M, k, groups, rotate);
        } else {
            convrot_quantize_kernel<true, false><<<grid, block, smem, stream>>>(xp, col_scale, q, row_scale, M, k, groups, rotate);
        }
    } else {
        if (cache) {
            convrot_quantize_kernel<false, true><<<grid, block, smem, stream>>>(xp, col_scale, q, row_scale, M, k, groups, rotate);
        } else {
            convrot_quantize_kernel<false, false><<<grid, block, smem, stream>>>(xp, col_scale, q, row_scale, M, k, groups, rotate);
        }
    }
    return cudaGetLastError() == cudaSuccess;
}
