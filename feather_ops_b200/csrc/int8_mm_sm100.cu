// int8 ConvRot GEMM for sm_100a, both directions over one prepacked weight:
//
//   forward   C[M, N] = A[M, K] @ W[N, K]^T,  out = cast(float(acc) * a_scale[m] * w_scale[n] + bias[n])
//   backward  C[M, K] = A[M, N] @ W[N, K],    out = cast(float(acc) * a_scale[m])      (`transposed_b`)
//
// The weight is the reference's 4x4 byte micro-tile prepack: micro-tile (k4, n4) is 16 bytes, byte
// (n % 4) * 4 + (k % 4) holds W[n][k], and micro-tile (k4, n4) sits at index k4 * (N / 4) + n4. The launcher
// receives the two micro-tile strides of the contraction and the output axis, so one kernel serves both
// directions. B200 counterpart of `int8_scaled_mm_kernel` / `launch_int8_scaled_mm` in the reference's
// csrc/hip_kernel_int8.cu (kernel :88-361, C ABI :413-471).
//
// Structure (one persistent CTA per SM, 128 x BN output tiles, 128 contraction bytes per pipeline slot):
//   * warp 0: TMA producer for the int8 activation tile (128 rows x 128 bytes, 128-byte swizzle, zero fill
//     past M and past the contraction length);
//   * eight re-layout warps: read the weight micro-tiles straight from global memory (L2), re-select
//     their bytes into K-major 16-byte rows (forward: four dwords of four consecutive k4; backward: a 4x4
//     byte transpose of four consecutive n4) and write the 128-byte swizzled UMMA operand tile;
//   * warp 1: one thread issues tcgen05.mma kind::i8 (M=128, N=BN, K=32) into one of two int32 TMEM
//     accumulators;
//   * four epilogue warps: int32 -> float, both scales, bias, one rounding, 16-byte stores.
// A ragged M is handled by the TMA zero fill and a row predicate on the stores, so there is no second
// launch for the M tail.
//
// 256-wide tiles run on CTA pairs instead (second half of this file): 256 x 256 tiles, the raw micro-tiles
// fetched by TMA and re-laid shared -> shared, about twice as fast per SM as the structure above.
#include "feather_host.h"
#include "feather_tiles_gen.h"
#include "sm100_ptx.cuh"

#include <cstdlib>

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace feather {
namespace i8mm {

constexpr int kBlockM = 128;
constexpr int kBlockK = 128;  // contraction bytes per slot: one 128-byte swizzle span
constexpr int kAStages = 4;
constexpr int kOperandStages = 3;
constexpr int kRelayoutWarps = 8;
constexpr int kEpilogueWarps = 4;
constexpr int kFirstEpilogueWarp = 2;
constexpr int kFirstRelayoutWarp = kFirstEpilogueWarp + kEpilogueWarps;
constexpr int kThreads = 32 * (kFirstRelayoutWarp + kRelayoutWarps);
constexpr int kATileBytes = kBlockM * kBlockK;

__device__ uint32_t g_status[2];

struct Params {
    const uint8_t* b;      // prepacked weight, 16-byte micro-tiles
    const float* a_scale;  // [M]
    const float* b_scale;  // [N_out] or null
    const uint16_t* bias;  // [N_out] or null
    uint16_t* c;           // [M, N_out]
    int M;
    int N_out;
    int K;                  // contraction length in bytes
    int64_t stride_kc;      // micro-tile stride of one 4-wide contraction step
    int64_t stride_out;     // micro-tile stride of one 4-wide output step
    int tiles_m;
    int tiles_n;
    uint32_t idesc;
    int band;               // pair kernel: row tiles per band of the tile walk
    int bulk_out;           // pair kernel: the output goes through shared-memory images and bulk tensor stores (N_out % 8 == 0, c 16-byte aligned)
    int tile_n;             // pair kernel: output columns per tile, a multiple of 16 up to 256 (below 256 only forward over the plain weight)
};

template <int BN>
struct Smem {
    static constexpr int kOperandBytes = BN * 128;
    static constexpr int kAOff = 0;
    static constexpr int kOperandOff = kAOff + kAStages * kATileBytes;
    static constexpr int kBarOff = kOperandOff + kOperandStages * kOperandBytes;
    static constexpr int kNumBars = 2 * kAStages + 2 * kOperandStages + 4;
    static constexpr int kTotal = kBarOff + kNumBars * 8 + 16;
    static constexpr int kDynamic = kTotal + 1024;
};

struct Ring {
    uint32_t idx = 0;
    uint32_t phase = 0;
    __device__ __forceinline__ void advance(uint32_t depth) {
        if (++idx == depth) {
            idx = 0;
            phase ^= 1u;
        }
    }
};

template <bool kOutBf16>
__device__ __forceinline__ uint32_t pack_out(float a, float b) {
    if constexpr (kOutBf16) {
        const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<const uint32_t*>(&v);
    } else {
        const __half2 v = __floats2half2_rn(a, b);
        return *reinterpret_cast<const uint32_t*>(&v);
    }
}

template <bool kOutBf16>
__device__ __forceinline__ float out_bits_to_float(uint16_t bits) {
    if constexpr (kOutBf16) {
        return __uint_as_float(static_cast<uint32_t>(bits) << 16);
    } else {
        return __half2float(__ushort_as_half(bits));
    }
}

// 4x4 byte transpose: in[i] byte j -> out[j] byte i.
__device__ __forceinline__ void transpose4x4(const uint32_t (&in)[4], uint32_t (&out)[4]) {
    const uint32_t t0 = __byte_perm(in[0], in[1], 0x5140u);
    const uint32_t t1 = __byte_perm(in[0], in[1], 0x7362u);
    const uint32_t t2 = __byte_perm(in[2], in[3], 0x5140u);
    const uint32_t t3 = __byte_perm(in[2], in[3], 0x7362u);
    out[0] = __byte_perm(t0, t2, 0x5410u);
    out[1] = __byte_perm(t0, t2, 0x7632u);
    out[2] = __byte_perm(t1, t3, 0x5410u);
    out[3] = __byte_perm(t1, t3, 0x7632u);
}

template <int BN, bool kTransposedB, bool kOutBf16>
__global__ void __launch_bounds__(kThreads, 1) int8_mm_kernel(const __grid_constant__ CUtensorMap map_a, const Params p) {
    using L = Smem<BN>;
    extern __shared__ uint8_t smem_dyn[];
    uint8_t* const smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~static_cast<uintptr_t>(1023));
    uint64_t* const bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
    uint64_t* const a_full = bars;
    uint64_t* const a_empty = a_full + kAStages;
    uint64_t* const operand_full = a_empty + kAStages;
    uint64_t* const operand_empty = operand_full + kOperandStages;
    uint64_t* const tmem_full = operand_empty + kOperandStages;
    uint64_t* const tmem_empty = tmem_full + 2;
    uint32_t* const tmem_slot = reinterpret_cast<uint32_t*>(bars + L::kNumBars);
    volatile uint32_t* const abort_flag = tmem_slot + 1;

    const int warp = static_cast<int>(threadIdx.x) / 32;
    const int lane = static_cast<int>(threadIdx.x) % 32;
    const WaitGuard guard{abort_flag, g_status};

    if (threadIdx.x == 0) {
        *abort_flag = 0u;
        for (int s = 0; s < kAStages; ++s) {
            mbar_init(&a_full[s], 1);
            mbar_init(&a_empty[s], 1);
        }
        for (int s = 0; s < kOperandStages; ++s) {
            mbar_init(&operand_full[s], kRelayoutWarps);
            mbar_init(&operand_empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&tmem_full[s], 1);
            mbar_init(&tmem_empty[s], kEpilogueWarps);
        }
        mbar_init_fence();
        tma_prefetch_desc(&map_a);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 2 * BN);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    const int num_tiles = p.tiles_m * p.tiles_n;
    const int num_kb = (p.K + kBlockK - 1) / kBlockK;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (activations)
        if (elect_one()) {
            Ring slot;
            bool ok = true;
            for (int tile = static_cast<int>(blockIdx.x); ok && tile < num_tiles; tile += static_cast<int>(gridDim.x)) {
                const int m0 = (tile % p.tiles_m) * kBlockM;
                for (int kb = 0; kb < num_kb; ++kb) {
                    ok = guard.wait(&a_empty[slot.idx], slot.phase ^ 1u, kSiteLoadEmpty);
                    if (!ok) break;
                    mbar_arrive_expect_tx(&a_full[slot.idx], kATileBytes);
                    tma_load_2d(smem + L::kAOff + slot.idx * kATileBytes, &map_a, &a_full[slot.idx], kb * kBlockK, m0);
                    slot.advance(kAStages);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (elect_one()) {
            Ring slot, operand, acc;
            bool ok = true;
            for (int tile = static_cast<int>(blockIdx.x); ok && tile < num_tiles; tile += static_cast<int>(gridDim.x)) {
                ok = guard.wait(&tmem_empty[acc.idx], acc.phase ^ 1u, kSiteTmemEmpty);
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t tmem_d = tmem_base + acc.idx * BN;
                for (int kb = 0; kb < num_kb; ++kb) {
                    ok = guard.wait(&a_full[slot.idx], slot.phase, kSiteLoadFull) &&
                         guard.wait(&operand_full[operand.idx], operand.phase, kSiteOperandFull);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint32_t a_addr = smem_u32(smem + L::kAOff + slot.idx * kATileBytes);
                    const uint32_t b_addr = smem_u32(smem + L::kOperandOff + operand.idx * L::kOperandBytes);
#pragma unroll
                    for (int k = 0; k < kBlockK / 32; ++k) {
                        umma_i8(tmem_d, make_desc_sw128_kmajor(a_addr + k * 32), make_desc_sw128_kmajor(b_addr + k * 32), p.idesc,
                                (kb | k) != 0 ? 1u : 0u);
                    }
                    umma_commit(&a_empty[slot.idx]);
                    umma_commit(&operand_empty[operand.idx]);
                    slot.advance(kAStages);
                    operand.advance(kOperandStages);
                }
                if (!ok) break;
                umma_commit(&tmem_full[acc.idx]);
                acc.advance(2);
            }
        }
    } else if (warp < kFirstRelayoutWarp) {
        // ------------------------------------------------------------------ epilogue
        const int quarter = warp % 4;
        const bool wide_rows = (p.N_out % 8) == 0;  // rows are 16-byte aligned
        Ring acc;
        bool ok = true;
        for (int tile = static_cast<int>(blockIdx.x); ok && tile < num_tiles; tile += static_cast<int>(gridDim.x)) {
            const int m0 = (tile % p.tiles_m) * kBlockM;
            const int n0 = (tile / p.tiles_m) * BN;
            ok = guard.wait(&tmem_full[acc.idx], acc.phase, kSiteTmemFull);
            if (!ok) break;
            tc_fence_after_sync();
            const int row = m0 + quarter * 32 + lane;
            const float row_scale = row < p.M ? __ldg(p.a_scale + row) : 0.0f;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc.idx * BN;
            uint16_t* const c_row = p.c + static_cast<int64_t>(row) * p.N_out;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t v[32];
                tmem_ld_32x32(taddr + c * 32, v);
                tmem_wait_ld();
                if (c == BN / 32 - 1) {
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&tmem_empty[acc.idx]);
                }
                const int col0 = n0 + c * 32;
#pragma unroll
                for (int g = 0; g < 8; ++g) {
                    const int col = col0 + g * 4;  // N_out is a multiple of 4
                    if (col >= p.N_out) continue;
                    float f[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        float value = static_cast<float>(static_cast<int32_t>(v[g * 4 + i])) * row_scale;
                        if constexpr (!kTransposedB) {
                            if (p.b_scale != nullptr) value *= __ldg(p.b_scale + col + i);
                            if (p.bias != nullptr) value += out_bits_to_float<kOutBf16>(__ldg(p.bias + col + i));
                        }
                        f[i] = value;
                    }
                    v[g * 4] = pack_out<kOutBf16>(f[0], f[1]);
                    v[g * 4 + 1] = pack_out<kOutBf16>(f[2], f[3]);
                }
                if (row < p.M) {
                    if (wide_rows) {
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            if (col0 + g * 8 < p.N_out) {
                                *reinterpret_cast<uint4*>(c_row + col0 + g * 8) = make_uint4(v[g * 8], v[g * 8 + 1], v[g * 8 + 4], v[g * 8 + 5]);
                            }
                        }
                    } else {
#pragma unroll
                        for (int g = 0; g < 8; ++g) {
                            if (col0 + g * 4 < p.N_out) {
                                *reinterpret_cast<uint2*>(c_row + col0 + g * 4) = make_uint2(v[g * 4], v[g * 4 + 1]);
                            }
                        }
                    }
                }
            }
            acc.advance(2);
        }
    } else {
        // ------------------------------------------------------------------ weight re-layout warps
        const int t = static_cast<int>(threadIdx.x) - kFirstRelayoutWarp * 32;
        const int k4_total = p.K / 4;
        if constexpr (!kTransposedB) {
            // Thread = operand row (output channel n). Dword (k4, n) of the prepack holds W[n][4 k4 .. 4 k4 + 3],
            // which is exactly four consecutive bytes of the K-major operand row, so the re-layout is a
            // 4-byte asynchronous copy per dword, straight from global (L2) to its swizzled position.
            // `kOperandStages - 1` slots of copies are kept in flight per thread.
            constexpr int kThreadsPerRow = (kRelayoutWarps * 32) / BN;
            constexpr int kChunksPerThread = 8 / kThreadsPerRow;
            constexpr int kInFlight = kOperandStages - 1;
            const uint32_t* const dwords = reinterpret_cast<const uint32_t*>(p.b);
            const int row = t % BN;
            const int first_chunk = (t / BN) * kChunksPerThread;
            Ring issue, landed;
            int tile = static_cast<int>(blockIdx.x);
            int kb = 0;
            bool ok = true;
            bool more = tile < num_tiles;
            int pending = 0;  // committed groups not yet published
            while (ok && (more || pending > 0)) {
                if (more) {
                    const int n = (tile / p.tiles_m) * BN + row;
                    const bool n_live = n < p.N_out;
                    const int64_t col_off = static_cast<int64_t>(n / 4) * p.stride_out * 4 + (n % 4);
                    ok = guard.wait(&operand_empty[issue.idx], issue.phase ^ 1u, kSiteOperandEmpty);
                    if (!ok) break;
                    const uint32_t dst = smem_u32(smem + L::kOperandOff + issue.idx * L::kOperandBytes);
#pragma unroll
                    for (int c = 0; c < kChunksPerThread; ++c) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const int k4 = kb * (kBlockK / 4) + (first_chunk + c) * 4 + j;
                            const bool live = n_live && k4 < k4_total;
                            const uint32_t* const src = live ? dwords + static_cast<int64_t>(k4) * p.stride_kc * 4 + col_off : dwords;
                            cp_async_4(dst + sw128_offset(row, first_chunk + c) + j * 4, src, live);
                        }
                    }
                    issue.advance(kOperandStages);
                    if (++kb == num_kb) {
                        kb = 0;
                        tile += static_cast<int>(gridDim.x);
                        more = tile < num_tiles;
                    }
                }
                cp_async_commit();
                ++pending;
                if (pending > kInFlight || !more) {
                    if (more) {
                        cp_async_wait<kInFlight>();
                    } else {
                        cp_async_wait<0>();
                    }
                    // everything but the newest `kInFlight` groups (all groups once the work is issued) has landed
                    const int publish = more ? 1 : pending;
                    for (int i = 0; i < publish; ++i) {
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&operand_full[landed.idx]);
                        landed.advance(kOperandStages);
                    }
                    pending -= publish;
                }
            }
        } else {
            // Thread = four operand rows (output columns 4 k4 .. 4 k4 + 3) x some 16-byte chunks.
            // Micro-tile (k4, n4) dword i holds W[4 n4 + i][4 k4 .. + 3]: the rows need byte r of every
            // dword, i.e. a 4x4 byte transpose per micro-tile, done in registers.
            constexpr int kColumns = BN / 4;
            constexpr int kThreadsPerColumn = (kRelayoutWarps * 32) / kColumns;
            constexpr int kChunksPerThread = (8 + kThreadsPerColumn - 1) / kThreadsPerColumn;
            const uint4* const tiles = reinterpret_cast<const uint4*>(p.b);
            const int column = t % kColumns;
            const int first_chunk = (t / kColumns) * kChunksPerThread;
            Ring operand;
            bool ok = true;
            for (int tile = static_cast<int>(blockIdx.x); ok && tile < num_tiles; tile += static_cast<int>(gridDim.x)) {
                const int out4 = ((tile / p.tiles_m) * BN) / 4 + column;
                const bool out_live = out4 * 4 < p.N_out;
                for (int kb = 0; kb < num_kb; ++kb) {
                    uint4 m[kChunksPerThread][4];
#pragma unroll
                    for (int c = 0; c < kChunksPerThread; ++c) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const int kc4 = kb * (kBlockK / 4) + (first_chunk + c) * 4 + j;
                            const bool live = out_live && kc4 < k4_total && first_chunk + c < 8;
                            m[c][j] = live ? __ldg(tiles + static_cast<int64_t>(kc4) * p.stride_kc + static_cast<int64_t>(out4) * p.stride_out)
                                           : make_uint4(0u, 0u, 0u, 0u);
                        }
                    }
                    ok = guard.wait(&operand_empty[operand.idx], operand.phase ^ 1u, kSiteOperandEmpty);
                    if (!ok) break;
                    uint8_t* const dst = smem + L::kOperandOff + operand.idx * L::kOperandBytes;
#pragma unroll
                    for (int c = 0; c < kChunksPerThread; ++c) {
                        if (first_chunk + c < 8) {
                            uint32_t rows[4][4];  // rows[j][r]: 4 contraction bytes of output row r from micro-tile j
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const uint32_t in[4] = {m[c][j].x, m[c][j].y, m[c][j].z, m[c][j].w};
                                transpose4x4(in, rows[j]);
                            }
#pragma unroll
                            for (int r = 0; r < 4; ++r) {
                                *reinterpret_cast<uint4*>(dst + sw128_offset(column * 4 + r, first_chunk + c)) =
                                    make_uint4(rows[0][r], rows[1][r], rows[2][r], rows[3][r]);
                            }
                        }
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&operand_full[operand.idx]);
                    operand.advance(kOperandStages);
                }
            }
        }
    }

    // ---------------------------------------------------------------------- teardown
    tc_fence_before_sync();
    __syncthreads();
    if (guard.aborted()) {
        const long long start = clock64();
        while (clock64() - start < 2000000LL) {
        }
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, 2 * BN);
    }
}

// ---------------------------------------------------------------------------------------------------------
// CTA-pair version (tcgen05 cta_group::2): a cluster of two CTAs owns a 256 x 256 output tile. CTA r loads
// activation rows [128 r, +128) and the raw micro-tiles of weight rows (output columns) [128 r, +128) of the
// tile by TMA; the UMMA (M = 256, N = 256, K = 32) is issued by CTA 0 and reads both CTAs' shared memory.
//
// Raw weight slab of one k block: 32 x 32 micro-tiles of 16 bytes, fetched as four boxes of 32 rows x 128
// bytes with the 128-byte swizzle. In global memory a slab row is one step of the slower micro-tile axis
// (forward: the contraction, backward: the output axis), so the same box shape serves both directions.
// The re-layout warps go shared -> registers -> shared: unit (group g = four operand rows, chunk c = 16
// contraction bytes) reads the four micro-tiles (contraction step 4 c + j, output step g), picks dwords
// (forward) or transposes 4x4 bytes (backward) and writes four 16-byte chunks of the swizzled K-major
// operand. The eight lanes of a quarter warp take g % 8 = l and c = l ^ t: both their 16-byte loads and
// their 16-byte stores then fall into eight different bank groups (the swizzle phases of the rows they touch
// differ in bit 2 exactly when l is odd), so neither side has bank conflicts. Global loads that feed
// registers directly (the previous version) ran at one k block per L2 latency whatever the prefetch depth.
// ---------------------------------------------------------------------------------------------------------
// Ring depths are multiples of the team count: a team always meets the same slots and sees every phase of the
// barriers it waits on.
#ifndef FEATHER_I8_LOAD_STAGES
#define FEATHER_I8_LOAD_STAGES 4
#endif
#ifndef FEATHER_I8_OPERAND_STAGES
#define FEATHER_I8_OPERAND_STAGES 4
#endif
#ifndef FEATHER_I8_TEAMS
#define FEATHER_I8_TEAMS 2
#endif
constexpr int kPairLoadStages = FEATHER_I8_LOAD_STAGES;
constexpr int kPairOperandStages = FEATHER_I8_OPERAND_STAGES;
constexpr int kPairTeams = FEATHER_I8_TEAMS;
static_assert(kPairLoadStages % kPairTeams == 0 && kPairOperandStages % kPairTeams == 0, "ring depths must be multiples of the team count");
constexpr int kPairHalfN = 128;
constexpr int kPairN = 2 * kPairHalfN;
constexpr int kPairRelayoutWarps = 8;
constexpr int kPairThreads = 32 * (kFirstRelayoutWarp + kPairRelayoutWarps);
constexpr int kRawBoxBytes = 32 * 128;

#ifndef FEATHER_I8_PLAIN_STAGES
#define FEATHER_I8_PLAIN_STAGES 6
#endif
constexpr int kPlainLoadStages = FEATHER_I8_PLAIN_STAGES;
constexpr int kPlainRelayWarp = kFirstEpilogueWarp + 2 * kEpilogueWarps;   // after two groups of epilogue warps
constexpr int kPlainThreads = 32 * (kPlainRelayWarp + 1);

// `kPlainB`: the weight is the released row-major `[N, K]` matrix, whose 128 x 128 byte boxes are UMMA operands as the copy engine
// delivers them (forward: K-major, backward: MN-major). No re-layout ring then, and a deeper load ring instead.
template <bool kPlainB>
struct PairSmemT {
    static constexpr int kLoadStages = kPlainB ? kPlainLoadStages : kPairLoadStages;
    static constexpr int kOperandStages = kPlainB ? 0 : kPairOperandStages;
    static constexpr int kOperandBars = kPlainB ? kPlainLoadStages : kPairOperandStages;   // plain: "both CTAs' loads have landed"
    static constexpr int kRawBytes = 4 * kRawBoxBytes;       // 16 KB: 32 x 32 micro-tiles, or one 128 x 128 box of the plain weight
    static constexpr int kOperandBytes = kPairHalfN * 128;  // 16 KB
    static constexpr int kAOff = 0;
    static constexpr int kRawOff = kAOff + kLoadStages * kATileBytes;
    static constexpr int kOperandOff = kRawOff + kLoadStages * kRawBytes;
    static constexpr int kColumnOff = kOperandOff + kOperandStages * kOperandBytes;  // 2 x (256 scales + 256 biases), fp32
    static constexpr int kImageBytes = kBlockM * 64;         // 128 rows x 32 output columns of 16 bits: four warps' images of 32 rows, one bulk tensor store each
    static constexpr int kImageOff = kColumnOff + 2 * 2 * kPairN * 4;   // eight warp images: two per warp used alternately, or one for each of eight warps
    static constexpr int kBarOff = kImageOff + 2 * kImageBytes;
    static constexpr int kNumBars = 2 * kLoadStages + 2 * kOperandBars + 6;
    static constexpr int kTotal = kBarOff + kNumBars * 8 + 16;
    static constexpr int kDynamic = kTotal + 1024;
    static_assert(kDynamic <= 227 * 1024, "the pair kernel's shared memory exceeds an SM's");
};
using PairSmem = PairSmemT<false>;

template <bool kTransposedB, bool kOutBf16, bool kPlainB>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
int8_mm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_c, const Params p) {
    using L = PairSmemT<kPlainB>;
    constexpr int kLoadStages = L::kLoadStages;
    constexpr int kOperandBars = L::kOperandBars;
    // Plain weight: the warps that would re-lay the weight are free, so two groups of four epilogue warps convert the two
    // 128-column halves of a tile at once (a tile's drain is half as long, which shows at the end of the launch).
    constexpr int kEpiWarps = kPlainB ? 2 * kEpilogueWarps : kEpilogueWarps;
    extern __shared__ uint8_t smem_dyn[];
    uint8_t* const smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~static_cast<uintptr_t>(1023));
    uint64_t* const bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
    uint64_t* const load_full = bars;                                // local: TMA bytes of this CTA's halves
    uint64_t* const load_empty = load_full + kLoadStages;        // signalled in both CTAs by CTA 0's commits
    uint64_t* const operand_full = load_empty + kLoadStages;     // CTA 0 only: both CTAs' warps arrive here
    uint64_t* const operand_empty = operand_full + kOperandBars;
    uint64_t* const tmem_full = operand_empty + kOperandBars;
    uint64_t* const tmem_empty = tmem_full + 2;                      // CTA 0 only
    uint64_t* const columns_full = tmem_empty + 2;                   // local: the tile's column scales and biases are staged
    uint32_t* const tmem_slot = reinterpret_cast<uint32_t*>(bars + L::kNumBars);
    volatile uint32_t* const abort_flag = tmem_slot + 1;

    const int warp = static_cast<int>(threadIdx.x) / 32;
    const int lane = static_cast<int>(threadIdx.x) % 32;
    const uint32_t cta = cluster_cta_rank();
    const WaitGuard guard{abort_flag, g_status};

    if (threadIdx.x == 0) {
        *abort_flag = 0u;
        for (int s = 0; s < kLoadStages; ++s) {
            mbar_init(&load_full[s], 1);
            mbar_init(&load_empty[s], 1);
        }
        for (int s = 0; s < kOperandBars; ++s) {
            // complete when the team's warps of both CTAs have written their halves; a warp arrives only after
            // its CTA's load (activation tile included) has landed, so the MMA thread needs no other wait.
            // Plain weight: one arrival per CTA, by the thread that watches that CTA's loads.
            mbar_init(&operand_full[s], kPlainB ? 2 : 2 * kPairRelayoutWarps / kPairTeams);
            mbar_init(&operand_empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&tmem_full[s], 1);
            mbar_init(&tmem_empty[s], 2 * kEpiWarps);
            mbar_init(&columns_full[s], kEpiWarps);
        }
        mbar_init_fence();
        tma_prefetch_desc(&map_a);
        tma_prefetch_desc(&map_b);
        if (p.bulk_out) tma_prefetch_desc(&map_c);
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, 2 * kPairN);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    const int tiles_m = (p.M + 2 * kBlockM - 1) / (2 * kBlockM);
    const int tiles_n = (p.N_out + p.tile_n - 1) / p.tile_n;
    const int num_tiles = tiles_m * tiles_n;
    const int num_kb = (p.K + kBlockK - 1) / kBlockK;
    const int first_tile = static_cast<int>(blockIdx.x) / 2;
    const int tile_step = static_cast<int>(gridDim.x) / 2;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (this CTA's halves)
        if (elect_one()) {
            // Launched as a programmatic dependent of the quantizer, everything above (barriers, tensor memory, descriptor
            // prefetch) has overlapped its tail; the activation codes are only read from here on.
            grid_dependency_wait();
            Ring slot;
            bool ok = true;
            for (int tile = first_tile; ok && tile < num_tiles; tile += tile_step) {
                int tile_m, tile_n;
                banded_tile(tile, tiles_m, tiles_n, p.band, tile_m, tile_n);
                const int m0 = tile_m * 2 * kBlockM + static_cast<int>(cta) * kBlockM;
                const int n0 = tile_n * p.tile_n + static_cast<int>(cta) * (p.tile_n / 2);
                // what the weight boxes of a k block deliver: plain forward one box of this CTA's output channels; plain backward one
                // full box; prepack forward one 4 KB box per 32 output channels; prepack backward four boxes of (channels / 4) rows
                const uint32_t half_cols = static_cast<uint32_t>(p.tile_n / 2);
                const uint32_t weight_bytes = kPlainB ? (kTransposedB ? static_cast<uint32_t>(L::kRawBytes) : half_cols * 128u) : half_cols * 128u;
                for (int kb = 0; kb < num_kb; ++kb) {
                    ok = guard.wait(&load_empty[slot.idx], slot.phase ^ 1u, kSiteLoadEmpty);
                    if (!ok) break;
                    mbar_arrive_expect_tx(&load_full[slot.idx], kATileBytes + weight_bytes);
                    tma_load_2d(smem + L::kAOff + slot.idx * kATileBytes, &map_a, &load_full[slot.idx], kb * kBlockK, m0);
                    // map_b: x = byte offset along the faster micro-tile axis, y = step of the slower one
                    const int x0 = kTransposedB ? kb * (kBlockK * 4) : n0 * 4;
                    const int y0 = kTransposedB ? n0 / 4 : kb * (kBlockK / 4);
                    uint8_t* const raw = smem + L::kRawOff + slot.idx * L::kRawBytes;
                    if constexpr (kPlainB) {
                        // map_b: x = weight column (the contraction forward, the output backward), y = weight row; one 128 x 128 box
                        if constexpr (kTransposedB) {
                            tma_load_2d(raw, &map_b, &load_full[slot.idx], n0, kb * kBlockK);
                        } else {
                            tma_load_2d(raw, &map_b, &load_full[slot.idx], kb * kBlockK, n0);
                        }
                    } else {
#pragma unroll
                        for (int box = 0; box < 4; ++box) {
                            // forward: box = 32 output channels (fewer boxes for a narrower tile); backward: box = 32 contraction steps
                            if (kTransposedB || box * 32 < static_cast<int>(half_cols)) {
                                tma_load_2d(raw + box * kRawBoxBytes, &map_b, &load_full[slot.idx], x0 + box * 128, y0);
                            }
                        }
                    }
                    slot.advance(kLoadStages);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (CTA 0 of the pair)
        if (cta == 0 && elect_one()) {
            Ring slot, operand, acc;
            bool ok = true;
            for (int tile = first_tile; ok && tile < num_tiles; tile += tile_step) {
                ok = guard.wait(&tmem_empty[acc.idx], acc.phase ^ 1u, kSiteTmemEmpty);
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t tmem_d = tmem_base + acc.idx * kPairN;
                for (int kb = 0; kb < num_kb; ++kb) {
                    ok = guard.wait(&operand_full[operand.idx], operand.phase, kSiteOperandFull);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint32_t a_addr = smem_u32(smem + L::kAOff + slot.idx * kATileBytes);
                    const uint32_t b_addr = kPlainB ? smem_u32(smem + L::kRawOff + slot.idx * L::kRawBytes)
                                                    : smem_u32(smem + L::kOperandOff + operand.idx * L::kOperandBytes);
#pragma unroll
                    for (int k = 0; k < kBlockK / 32; ++k) {
                        // plain weight, backward: the box holds 128 contraction rows of 128 output bytes, i.e. an MN-major operand
                        // whose 8-row groups are 1024 bytes apart; a 32-deep step is four of them
                        const uint64_t desc_b = kPlainB && kTransposedB ? make_desc_sw128_mnmajor(b_addr + k * 32 * 128) : make_desc_sw128_kmajor(b_addr + k * 32);
                        umma_i8_pair(tmem_d, make_desc_sw128_kmajor(a_addr + k * 32), desc_b, p.idesc, (kb | k) != 0 ? 1u : 0u);
                    }
#pragma unroll
                    for (uint32_t dst = 0; dst < 2; ++dst) {
                        umma_commit_pair(map_to_cta(smem_u32(&load_empty[slot.idx]), dst));
                        if constexpr (!kPlainB) umma_commit_pair(map_to_cta(smem_u32(&operand_empty[operand.idx]), dst));
                    }
                    slot.advance(kLoadStages);
                    operand.advance(kOperandBars);
                }
                if (!ok) break;
#pragma unroll
                for (uint32_t dst = 0; dst < 2; ++dst) umma_commit_pair(map_to_cta(smem_u32(&tmem_full[acc.idx]), dst));
                acc.advance(2);
            }
        }
    } else if (warp < kFirstEpilogueWarp + kEpiWarps) {
        // ------------------------------------------------------------------ epilogue (this CTA's 128 rows)
        // The column scales and biases of a tile are staged in shared memory once (each epilogue warp writes
        // a quarter, one barrier arrival per warp) instead of being fetched per element. Two buffers, used
        // alternately like the accumulators: a warp refills a buffer only after every warp has arrived for the
        // tile in between, i.e. has finished reading it.
        const int quarter = warp % 4;
        const int epi_warp = warp - kFirstEpilogueWarp;
        const int half = epi_warp / kEpilogueWarps;                 // plain weight: the 128 output columns this group converts
        const int chunks = (p.tile_n + 31) / 32;   // the last one may hold 16 columns only
        const int c_begin = kPlainB ? half * ((chunks + 1) / 2) : 0;
        const int c_end = kPlainB && half == 0 ? (chunks + 1) / 2 : chunks;
        const bool wide_rows = (p.N_out % 8) == 0;
        const bool has_scale = !kTransposedB && p.b_scale != nullptr;
        const bool has_bias = !kTransposedB && p.bias != nullptr;
        // With `bulk_out` a warp's 32 rows x 32 columns of a chunk go into a 64-byte-swizzled shared-memory image that its first lane
        // hands to the copy engine (which clips at M and N_out): a lane holds one row, so the direct stores are 32 requests of 16
        // bytes per warp instruction, 4096 per tile, and the drain of a pair's last tile has nothing to hide behind. One image per
        // warp, so that the warps never wait for one another: two used alternately, or (plain weight, eight warps) one.
        const int twist = (lane >> 1) & 3;   // 64-byte swizzle: the 16-byte chunk index is XORed with bits 7-8 of the address (the images are 2 KB apart)
        uint32_t stores = 0;
        Ring acc;
        bool ok = true;
        grid_dependency_wait();   // the row scales come from the kernel before this one
        for (int tile = first_tile; ok && tile < num_tiles; tile += tile_step) {
            int tile_m, tile_n;
            banded_tile(tile, tiles_m, tiles_n, p.band, tile_m, tile_n);
            const int m0 = tile_m * 2 * kBlockM + static_cast<int>(cta) * kBlockM;
            const int n0 = tile_n * p.tile_n;
            float* const col_scale = reinterpret_cast<float*>(smem + L::kColumnOff) + acc.idx * 2 * kPairN;
            float* const col_bias = col_scale + kPairN;
            if (has_scale || has_bias) {
#pragma unroll
                for (int i = 0; i < 8 / kEpiWarps; ++i) {
                    const int c = kPlainB ? epi_warp * 32 + lane : quarter * 64 + i * 32 + lane;
                    const int col = n0 + c;
                    col_scale[c] = has_scale && col < p.N_out ? __ldg(p.b_scale + col) : 1.0f;
                    col_bias[c] = has_bias && col < p.N_out ? out_bits_to_float<kOutBf16>(__ldg(p.bias + col)) : 0.0f;
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&columns_full[acc.idx]);
                ok = guard.wait(&columns_full[acc.idx], acc.phase, kSiteTmemFull, 3);
                if (!ok) break;
            }
            ok = guard.wait(&tmem_full[acc.idx], acc.phase, kSiteTmemFull);
            if (!ok) break;
            tc_fence_after_sync();
            const int row = m0 + quarter * 32 + lane;
            const float row_scale = row < p.M ? __ldg(p.a_scale + row) : 0.0f;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc.idx * kPairN;
            uint16_t* const c_row = p.c + static_cast<int64_t>(row) * p.N_out;
#pragma unroll 1
            for (int c = c_begin; c < c_end; ++c) {
                uint32_t v[32];
                tmem_ld_32x32(taddr + c * 32, v);
                tmem_wait_ld();
                if (c == c_end - 1) {
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tmem_empty[acc.idx]), 0));
                }
                const int col0 = n0 + c * 32;
#pragma unroll
                for (int g = 0; g < 8; ++g) {
                    float f[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) f[i] = static_cast<float>(static_cast<int32_t>(v[g * 4 + i])) * row_scale;
                    if (has_scale) {
                        const float4 s4 = *reinterpret_cast<const float4*>(col_scale + c * 32 + g * 4);
                        f[0] *= s4.x;
                        f[1] *= s4.y;
                        f[2] *= s4.z;
                        f[3] *= s4.w;
                    }
                    if (has_bias) {
                        const float4 b4 = *reinterpret_cast<const float4*>(col_bias + c * 32 + g * 4);
                        f[0] += b4.x;
                        f[1] += b4.y;
                        f[2] += b4.z;
                        f[3] += b4.w;
                    }
                    v[g * 4] = pack_out<kOutBf16>(f[0], f[1]);
                    v[g * 4 + 1] = pack_out<kOutBf16>(f[2], f[3]);
                }
                const int tile_cols = p.tile_n - c * 32;   // columns of this chunk that belong to the tile: 32, or 16 in a last half chunk
                if (p.bulk_out && tile_cols >= 32) {
                    if (col0 >= p.N_out) continue;
                    // before the warp overwrites an image its lane's store from it must have been read: all but the newest store
                    // with two images, every store with one
                    if (stores >= (kPlainB ? 1u : 2u)) {
                        if (lane == 0) {
                            if constexpr (kPlainB) {
                                tma_store_wait_read<0>();
                            } else {
                                tma_store_wait_read<1>();
                            }
                        }
                        __syncwarp();
                    }
                    uint8_t* const image = smem + L::kImageOff + (kPlainB ? epi_warp : static_cast<int>(stores & 1u) * kEpilogueWarps + quarter) * (32 * 64);
                    uint8_t* const image_row = image + lane * 64;
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        *reinterpret_cast<uint4*>(image_row + ((g ^ twist) << 4)) = make_uint4(v[g * 8], v[g * 8 + 1], v[g * 8 + 4], v[g * 8 + 5]);
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_2d(&map_c, image, col0, m0 + quarter * 32);
                        tma_store_commit();
                    }
                    ++stores;
                } else if (row < p.M) {
                    if (wide_rows) {
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            if (g * 8 < tile_cols && col0 + g * 8 < p.N_out) {
                                *reinterpret_cast<uint4*>(c_row + col0 + g * 8) = make_uint4(v[g * 8], v[g * 8 + 1], v[g * 8 + 4], v[g * 8 + 5]);
                            }
                        }
                    } else {
#pragma unroll
                        for (int g = 0; g < 8; ++g) {
                            if (g * 4 < tile_cols && col0 + g * 4 < p.N_out) {
                                *reinterpret_cast<uint2*>(c_row + col0 + g * 4) = make_uint2(v[g * 4], v[g * 4 + 1]);
                            }
                        }
                    }
                }
            }
            acc.advance(2);
        }
        if (p.bulk_out && lane == 0) tma_store_wait<0>();   // the images must outlive the copy engine's reads, and the stores the kernel
    } else if constexpr (kPlainB) {
        // ------------------------------------------------------------------ plain weight: one thread per CTA tells the MMA thread
        // (CTA 0) that this CTA's boxes of a k block have landed; the other warps of this role have nothing to do
        if (warp == kPlainRelayWarp && elect_one()) {
            Ring slot;
            bool ok = true;
            for (int tile = first_tile; ok && tile < num_tiles; tile += tile_step) {
                for (int kb = 0; kb < num_kb; ++kb) {
                    ok = guard.wait(&load_full[slot.idx], slot.phase, kSiteLoadFull, 2);
                    if (!ok) break;
                    mbar_arrive_cluster(map_to_cta(smem_u32(&operand_full[slot.idx]), 0));
                    slot.advance(kLoadStages);
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ weight re-layout warps (this CTA's 128 operand rows)
        constexpr int kTeamThreads = kPairRelayoutWarps * 32 / kPairTeams;
        constexpr int kUnitsPerThread = 256 / kTeamThreads;  // 32 groups x 8 chunks per k block
        const int relayout_thread = static_cast<int>(threadIdx.x) - kFirstRelayoutWarp * 32;
        const int team = relayout_thread / kTeamThreads;
        const int t = relayout_thread % kTeamThreads;
        const uint32_t l = static_cast<uint32_t>(t) & 7u;
        const uint32_t live_groups = static_cast<uint32_t>(p.tile_n / 8);   // groups of four operand rows in this CTA's half of the tile
        Ring slot, operand;
        bool ok = true;
        uint32_t turn = 0;  // k blocks since the start of the kernel, modulo the number of teams
        for (int tile = first_tile; ok && tile < num_tiles; tile += tile_step) {
            for (int kb = 0; kb < num_kb; ++kb) {
                if (turn == static_cast<uint32_t>(team)) {
                    ok = guard.wait(&load_full[slot.idx], slot.phase, kSiteLoadFull, 2) &&
                         guard.wait(&operand_empty[operand.idx], operand.phase ^ 1u, kSiteOperandEmpty);
                    if (!ok) break;
                    const uint8_t* const raw = smem + L::kRawOff + slot.idx * L::kRawBytes;
                    uint8_t* const dst = smem + L::kOperandOff + operand.idx * L::kOperandBytes;
                    uint4 m[kUnitsPerThread][4];
#pragma unroll
                    for (int i = 0; i < kUnitsPerThread; ++i) {
                        const uint32_t set = static_cast<uint32_t>(t + i * kTeamThreads) >> 3;  // 0..31
                        const uint32_t group = 8u * (set & 3u) + l;
                        if (group >= live_groups) continue;   // a narrower tile: fewer operand rows
                        const uint32_t chunk = l ^ (set >> 2);
#pragma unroll
                        for (uint32_t j = 0; j < 4; ++j) {
                            uint32_t offset;
                            if constexpr (kTransposedB) {
                                // slab row = output step, micro-tile column = contraction step 4 chunk + j
                                offset = (chunk >> 1) * kRawBoxBytes + sw128_offset(group, 4u * (chunk & 1u) + j);
                            } else {
                                // slab row = contraction step 4 chunk + j, micro-tile column = output step
                                offset = (group >> 3) * kRawBoxBytes + sw128_offset(4u * chunk + j, group & 7u);
                            }
                            m[i][j] = *reinterpret_cast<const uint4*>(raw + offset);
                        }
                    }
#pragma unroll
                    for (int i = 0; i < kUnitsPerThread; ++i) {
                        const uint32_t set = static_cast<uint32_t>(t + i * kTeamThreads) >> 3;
                        const uint32_t group = 8u * (set & 3u) + l;
                        if (group >= live_groups) continue;
                        const uint32_t chunk = l ^ (set >> 2);
                        uint32_t rows[4][4];  // rows[j][r]: contraction bytes 4 j .. 4 j + 3 of operand row 4 group + r
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const uint32_t in[4] = {m[i][j].x, m[i][j].y, m[i][j].z, m[i][j].w};
                            if constexpr (kTransposedB) {
                                transpose4x4(in, rows[j]);
                            } else {
#pragma unroll
                                for (int r = 0; r < 4; ++r) rows[j][r] = in[r];
                            }
                        }
#pragma unroll
                        for (uint32_t r = 0; r < 4; ++r) {
                            *reinterpret_cast<uint4*>(dst + sw128_offset(group * 4u + r, chunk)) = make_uint4(rows[0][r], rows[1][r], rows[2][r], rows[3][r]);
                        }
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&operand_full[operand.idx]), 0));
                }
                turn = turn + 1 == kPairTeams ? 0 : turn + 1;
                slot.advance(kPairLoadStages);
                operand.advance(kPairOperandStages);
            }
        }
    }

    // ---------------------------------------------------------------------- teardown
    tc_fence_before_sync();
    __syncthreads();
    if (guard.aborted()) {
        const long long start = clock64();
        while (clock64() - start < 2000000LL) {
        }
    }
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, 2 * kPairN);
    }
}

struct LaunchArgs {
    const int8_t* a;
    const uint8_t* b;
    const float* a_scale;
    const float* b_scale;
    const uint16_t* bias;
    uint16_t* c;
    int64_t M, N_out, K;
    int64_t stride_kc, stride_out;
    bool transposed_b;
    bool out_bf16;
    cudaStream_t stream;
    bool plain = false;   // `b` is the row-major [N, K] weight (the pair kernel only); the strides are unused
};

template <int BN, bool kTransposedB, bool kOutBf16>
bool launch_instance(const LaunchArgs& args) {
    using L = Smem<BN>;
    auto* kernel = &int8_mm_kernel<BN, kTransposedB, kOutBf16>;
    static PerDeviceState configured;
    if (configured.get([&] { return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic) == cudaSuccess ? 1 : 0; }) == 0) return false;
    CUtensorMap map_a;
    const uint64_t dims[2] = {static_cast<uint64_t>(args.K), static_cast<uint64_t>(args.M)};
    const uint64_t strides[1] = {static_cast<uint64_t>(args.K)};
    const uint32_t box[2] = {kBlockK, kBlockM};
    if (!encode_map(&map_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, args.a, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) return false;

    Params p{};
    p.b = args.b;
    p.a_scale = args.a_scale;
    p.b_scale = args.b_scale;
    p.bias = args.bias;
    p.c = args.c;
    p.M = static_cast<int>(args.M);
    p.N_out = static_cast<int>(args.N_out);
    p.K = static_cast<int>(args.K);
    p.stride_kc = args.stride_kc;
    p.stride_out = args.stride_out;
    p.tiles_m = static_cast<int>((args.M + kBlockM - 1) / kBlockM);
    p.tiles_n = static_cast<int>((args.N_out + BN - 1) / BN);
    p.idesc = make_idesc(kAccS32, kFmtS8, kFmtS8, kBlockM, BN);
    const int num_tiles = p.tiles_m * p.tiles_n;
    const int sms = device_info().sm_count;
    const int grid = num_tiles < sms ? num_tiles : sms;
    kernel<<<grid, kThreads, L::kDynamic, args.stream>>>(map_a, p);
    return cudaGetLastError() == cudaSuccess;
}

// FEATHER_INT8_PDL_OFF=1 launches the pair kernel without programmatic dependent launch (A/B measurements). Read once per process.
inline bool pdl_off() {
    static const bool off = env_switch("FEATHER_INT8_PDL_OFF");
    return off;
}

// FEATHER_INT8_BULK_OUT_OFF=1 keeps the pair kernel's direct output stores (A/B measurements). Read once per process.
inline bool bulk_out_off() {
    static const bool off = env_switch("FEATHER_INT8_BULK_OUT_OFF");
    return off;
}

// FEATHER_INT8_TILE_WIDTH_OFF=1 keeps 256-column tiles for every shape (A/B measurements). Read once per process.
inline bool tile_width_off() {
    static const bool off = env_switch("FEATHER_INT8_TILE_WIDTH_OFF");
    return off;
}

// Output columns per tile for the forward product over the plain weight. That kernel is bound by the tensor pipe, so a tile's time
// goes with its width, and a narrower tile can fill the last round of the persistent grid: 4096 x 3072 with 256-wide tiles are 192
// tiles = 2.6 rounds of 74 pairs, which take three; 176-wide ones are 288 tiles = 3.9 rounds of 0.69 the length. Cost of a launch:
// rounds x (width + a fixed part per tile, in columns); the widest tile wins a tie.
// `step`: 16 forward. Backward 64: a CTA's half of the tile's columns is the x coordinate of its weight boxes, which the copy engine wants on
// a 16-byte boundary (so 32 at least), and an MN-major operand of 80 or 112 columns per CTA was measured a third slower than one of 96 or 128.
inline int plain_tile_width(int64_t M, int64_t N_out, int pairs, int step = 16, int fixed_columns = 0) {
    // the part of a tile's time that does not go with its width, in columns: small forward; backward a 192-column tile was measured at 0.84 of a
    // 256-column one (its boxes still fetch 128-byte rows)
    const int kFixedColumns = fixed_columns > 0 ? fixed_columns : (step == 16 ? 24 : 144);
    if (tile_width_off() || pairs <= 0) return kPairN;
    // FEATHER_INT8_TILE_WIDTH=<multiple of 16 in 128..256> forces the width (measurements). Read once per process.
    static const int forced = [] {
        const char* text = std::getenv("FEATHER_INT8_TILE_WIDTH");
        const int value = text != nullptr ? std::atoi(text) : 0;
        return value >= kPairN / 2 && value <= kPairN && value % 16 == 0 ? value : 0;
    }();
    if (forced != 0) return forced % step == 0 ? forced : kPairN;
    // backward with a few rows streams the weight once and is bound by that: a narrower tile's boxes still fetch 128-byte rows, so it
    // would only fetch more (16 x 5376 x 5376: 17.6 us at 256 columns, 22.8 at 128)
    if (step != 16 && fixed_columns == 0 && M <= 64) return kPairN;
    const int64_t tiles_m = (M + 2 * kBlockM - 1) / (2 * kBlockM);
    int best = kPairN;
    int64_t best_cost = 0;
    int64_t full_cost = 0;
    for (int width = kPairN; width >= kPairN / 2; width -= step) {
        const int64_t tiles = tiles_m * ((N_out + width - 1) / width);
        const int64_t cost = ((tiles + pairs - 1) / pairs) * (width + kFixedColumns);
        if (width == kPairN) full_cost = cost;
        if (width == kPairN || cost < best_cost) {
            best = width;
            best_cost = cost;
        }
    }
    // a narrower tile must promise at least 4 %: below that the model's error decides
    return best_cost * 100 <= full_cost * 96 ? best : kPairN;
}

// The same choice for the kernel over the prepack, among 128, 192 and 256 columns (a weight box is 32 output channels forward). That kernel
// is bound by the shared-memory traffic of a k block, a third of which (the activation tile in and out) does not go with the tile's width.
inline int prepack_tile_width(int64_t M, int64_t N_out, int pairs) { return plain_tile_width(M, N_out, pairs, 64, 128); }

template <bool kTransposedB, bool kOutBf16, bool kPlainB>
bool launch_pair_instance(const LaunchArgs& args) {
    using L = PairSmemT<kPlainB>;
    auto* kernel = &int8_mm_pair_kernel<kTransposedB, kOutBf16, kPlainB>;
    // once per device: the shared-memory limit and how many CTA pairs fit at once (a persistent grid must be resident as a
    // whole, and a pair needs both SMs of a TPC)
    static PerDeviceState resident_pairs;
    const int pairs = resident_pairs.get([&] {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic) != cudaSuccess) return 0;
        cudaLaunchConfig_t config = {};
        config.gridDim = dim3(static_cast<unsigned>(device_info().sm_count / 2 * 2));
        config.blockDim = dim3(kPlainB ? kPlainThreads : kPairThreads);
        config.dynamicSmemBytes = L::kDynamic;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        config.attrs = attr;
        config.numAttrs = 1;
        int clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &config) != cudaSuccess || clusters <= 0) {
            (void)cudaGetLastError();
            clusters = device_info().sm_count / 2;
        }
        return clusters;
    });
    if (pairs <= 0) return false;
    CUtensorMap map_a;
    const uint64_t dims[2] = {static_cast<uint64_t>(args.K), static_cast<uint64_t>(args.M)};
    const uint64_t strides[1] = {static_cast<uint64_t>(args.K)};
    const uint32_t box[2] = {kBlockK, kBlockM};
    if (!encode_map(&map_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, args.a, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) return false;
    // weight as a 2-D byte array: x runs along the micro-tile axis with stride 1 (forward: output steps,
    // backward: contraction steps), y along the other one
    const int tile_n = kPlainB ? plain_tile_width(args.M, args.N_out, pairs, kTransposedB ? 64 : 16) : prepack_tile_width(args.M, args.N_out, pairs);
    CUtensorMap map_b;
    if constexpr (kPlainB) {
        // the row-major weight: x = column (the layer's input axis), y = row (its output axis)
        const uint64_t weight_cols = static_cast<uint64_t>(kTransposedB ? args.N_out : args.K);
        const uint64_t weight_rows = static_cast<uint64_t>(kTransposedB ? args.K : args.N_out);
        const uint64_t b_dims[2] = {weight_cols, weight_rows};
        const uint64_t b_strides[1] = {weight_cols};
        const uint32_t b_box[2] = {128, kTransposedB ? 128u : static_cast<uint32_t>(tile_n / 2)};   // forward: this CTA's output channels
        if (!encode_map(&map_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, args.b, b_dims, b_strides, b_box, CU_TENSOR_MAP_SWIZZLE_128B)) return false;
    } else {
        const uint64_t fast_tiles = static_cast<uint64_t>((kTransposedB ? args.K : args.N_out) / 4);
        const uint64_t slow_tiles = static_cast<uint64_t>((kTransposedB ? args.N_out : args.K) / 4);
        const uint64_t slow_stride = static_cast<uint64_t>(kTransposedB ? args.stride_out : args.stride_kc);
        const uint64_t b_dims[2] = {fast_tiles * 16, slow_tiles};
        const uint64_t b_strides[1] = {slow_stride * 16};
        // forward: 32 contraction steps of 32 output channels (one box per 32 channels of the CTA's half); backward: 32 contraction steps
        // (128 bytes) of all the CTA's output steps
        const uint32_t b_box[2] = {128, kTransposedB ? static_cast<uint32_t>(tile_n / 8) : 32u};
        if (!encode_map(&map_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, args.b, b_dims, b_strides, b_box, CU_TENSOR_MAP_SWIZZLE_128B)) return false;
    }

    Params p{};
    p.b = args.b;
    p.a_scale = args.a_scale;
    p.b_scale = args.b_scale;
    p.bias = args.bias;
    p.c = args.c;
    p.M = static_cast<int>(args.M);
    p.N_out = static_cast<int>(args.N_out);
    p.K = static_cast<int>(args.K);
    p.stride_kc = args.stride_kc;
    p.stride_out = args.stride_out;
    p.tiles_m = static_cast<int>((args.M + 2 * kBlockM - 1) / (2 * kBlockM));
    {
        // as many row tiles per band as keep one band of activations around 32 MB
        int64_t band = (32ll << 20) / (2 * kBlockM * args.K);
        if (band < 4) band = 4;
        if (band > p.tiles_m) band = p.tiles_m;
        p.band = static_cast<int>(band < 1 ? 1 : band);
    }
    p.tile_n = tile_n;
    p.tiles_n = static_cast<int>((args.N_out + tile_n - 1) / tile_n);
    p.idesc = make_idesc(kAccS32, kFmtS8, kFmtS8, 2 * kBlockM, static_cast<uint32_t>(tile_n)) | (kPlainB && kTransposedB ? kIdescBMajorMN : 0u);
    // the output as a 2-D tensor with a box of 32 columns x 128 rows (64-byte swizzle): what the epilogue's bulk stores write
    CUtensorMap map_c = map_a;   // unused without bulk_out
    p.bulk_out = (args.N_out % 8 == 0 && (reinterpret_cast<uintptr_t>(args.c) & 15u) == 0 && !bulk_out_off()) ? 1 : 0;
    if (p.bulk_out) {
        const uint64_t c_dims[2] = {static_cast<uint64_t>(args.N_out), static_cast<uint64_t>(args.M)};
        const uint64_t c_strides[1] = {static_cast<uint64_t>(args.N_out) * 2};
        const uint32_t c_box[2] = {32, 32};   // one epilogue warp's rows of a 32-column chunk
        if (!encode_map(&map_c, kOutBf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, args.c, c_dims, c_strides, c_box, CU_TENSOR_MAP_SWIZZLE_64B)) return false;
    }
    const int num_tiles = p.tiles_m * p.tiles_n;
    const int grid = 2 * (num_tiles < pairs ? num_tiles : pairs);
    // Programmatic dependent launch: the kernel may start while the one before it in the stream (in the ConvRot linear
    // layer: the activation quantizer) is still running, and waits for it (griddepcontrol.wait) before it reads the
    // activations or the row scales. After a kernel that never signals its dependents this is an ordinary launch.
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(static_cast<unsigned>(grid));
    config.blockDim = dim3(kPlainB ? kPlainThreads : kPairThreads);   // plain: one warp watches the loads
    config.dynamicSmemBytes = L::kDynamic;
    config.stream = args.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl_off() ? 0 : 1;
    config.attrs = attr;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, kernel, map_a, map_b, map_c, p) == cudaSuccess;
}

// ---------------------------------------------------------------------------------------------------------
// Warp-MMA version of the forward direction for at most 64 rows (a text band, a decode step): tcgen05 has no shape
// below 64 rows and a CTA-pair launch costs more than streaming a few MB of weight, so this case runs on mma.sync
// m16n8k32 (int8, exact int32 accumulation). A warp owns 32 output columns for one eighth of the contraction; the
// eight warps' int32 partial sums are added through shared memory (integer addition: any order gives the same bits).
// The contraction index inside a 32-deep block is permuted identically for both operands (fragment bytes 4t..4t+3
// and 16+4t..16+4t+3 take k = 8t..8t+7), so a lane's A fragment is eight consecutive activation bytes and its B
// fragment two dwords of the prepack (contraction steps 2t and 2t+1 of one output column): no shuffles, no staging.
// ---------------------------------------------------------------------------------------------------------
constexpr int kWmmaMaxRows = 64;    // two grid rows of 32: beyond that the pair kernel wins (128 rows at K = 12288: 54 against 38 us)
constexpr int kWmmaTwoTileMaxN = 8192;   // 17..32 rows: from this width on the CTA-pair kernel has enough tiles and wins
constexpr int kWmmaWarps = 8;

__device__ __forceinline__ void mma_m16n8k32_s8(int32_t (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// kRowTiles 16-row tiles per warp (1 or 2: up to 32 rows); every weight dword is fetched once and used for all of them.
// Four tiles per warp (64 rows) were measured slower than the CTA-pair kernel at every shape tried: 128 registers, one
// block in flight.
// `kPlainW`: `b` is the row-major [N, K] weight instead of the prepack. A lane's B fragment is then eight consecutive bytes of
// weight row n (the same eight contraction indices as its A fragment), one 8-byte load; the strides are unused.
template <int kRowTiles, bool kOutBf16, bool kPlainW>
__global__ void __launch_bounds__(32 * kWmmaWarps, kRowTiles == 1 ? 3 : 2)
int8_mm_wmma_kernel(const int8_t* __restrict__ a, const uint8_t* __restrict__ b, const float* __restrict__ a_scale, const float* __restrict__ b_scale,
                    const uint16_t* __restrict__ bias, uint16_t* __restrict__ c, int M, int N, int K, int64_t stride_kc, int64_t stride_out) {
    constexpr int kUnroll = 2;   // 32-deep blocks in flight per warp (8 weight dwords per lane each)
    __shared__ int32_t partial[kWmmaWarps][4][4][32];   // [warp][8-column block][fragment register][lane], one row tile at a time
    const int warp = static_cast<int>(threadIdx.x) / 32;
    const int lane = static_cast<int>(threadIdx.x) % 32;
    const int g = lane >> 2;   // fragment row (and row + 8), B column inside an 8-column block
    const int t = lane & 3;    // which eight k of the 32-deep block
    const int n0 = static_cast<int>(blockIdx.x) * 32;
    const int row0 = static_cast<int>(blockIdx.y) * 16 * kRowTiles;   // more rows than a warp's tiles: one grid row per block of them
    const int blocks = K / 32 + (K % 32 != 0 ? 1 : 0);   // K is a multiple of 16: the last block may be half
    const int per_warp = (blocks + kWmmaWarps - 1) / kWmmaWarps;
    const int s_begin = warp * per_warp;
    const int s_end = s_begin + per_warp < blocks ? s_begin + per_warp : blocks;
    const int k4_total = K / 4;

    int32_t acc[kRowTiles][4][4];
#pragma unroll
    for (int rt = 0; rt < kRowTiles; ++rt) {
#pragma unroll
        for (int blk = 0; blk < 4; ++blk) {
#pragma unroll
            for (int r = 0; r < 4; ++r) acc[rt][blk][r] = 0;
        }
    }
    // rows of this lane's A fragments: 16 rt + g and 16 rt + g + 8
    bool row_live[kRowTiles][2];
    const int8_t* a_row[kRowTiles][2];
#pragma unroll
    for (int rt = 0; rt < kRowTiles; ++rt) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = row0 + 16 * rt + g + 8 * h;
            row_live[rt][h] = row < M;
            a_row[rt][h] = a + static_cast<int64_t>(row_live[rt][h] ? row : 0) * K + 8 * t;
        }
    }
    // dword (contraction step k4, output column n) of the prepack: micro-tile (k4, n / 4), dword n % 4
    const uint8_t* w_col[4];
    bool col_live[4];
#pragma unroll
    for (int blk = 0; blk < 4; ++blk) {
        const int n = n0 + 8 * blk + g;
        col_live[blk] = n < N;
        if constexpr (kPlainW) {
            w_col[blk] = b + static_cast<int64_t>(col_live[blk] ? n : 0) * K + 8 * t;
        } else {
            w_col[blk] = b + (static_cast<int64_t>(col_live[blk] ? n / 4 : 0) * stride_out) * 16 + (n % 4) * 4;
        }
    }

    for (int s0 = s_begin; s0 < s_end; s0 += kUnroll) {
        uint32_t w[kUnroll][4][2];
        uint2 x[kUnroll][kRowTiles][2];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int k4 = (s0 + u) * 8 + 2 * t;            // this lane's two contraction steps of the block
            const bool live = s0 + u < s_end && k4 < k4_total;   // k4 + 1 exists as well: K / 4 is a multiple of 4
#pragma unroll
            for (int blk = 0; blk < 4; ++blk) {
                if constexpr (kPlainW) {
                    const uint2 pair = (live && col_live[blk]) ? __ldg(reinterpret_cast<const uint2*>(w_col[blk] + (s0 + u) * 32)) : make_uint2(0u, 0u);
                    w[u][blk][0] = pair.x;
                    w[u][blk][1] = pair.y;
                } else {
                    const uint8_t* const src = w_col[blk] + static_cast<int64_t>(k4) * stride_kc * 16;
                    w[u][blk][0] = (live && col_live[blk]) ? __ldg(reinterpret_cast<const uint32_t*>(src)) : 0u;
                    w[u][blk][1] = (live && col_live[blk]) ? __ldg(reinterpret_cast<const uint32_t*>(src + stride_kc * 16)) : 0u;
                }
            }
#pragma unroll
            for (int rt = 0; rt < kRowTiles; ++rt) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    x[u][rt][h] = (live && row_live[rt][h]) ? __ldg(reinterpret_cast<const uint2*>(a_row[rt][h] + (s0 + u) * 32)) : make_uint2(0u, 0u);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
#pragma unroll
            for (int rt = 0; rt < kRowTiles; ++rt) {
                // A fragment: {row g: k 8t..8t+3}, {row g+8: same}, {row g: k 8t+4..8t+7}, {row g+8: same}
                const uint32_t af[4] = {x[u][rt][0].x, x[u][rt][1].x, x[u][rt][0].y, x[u][rt][1].y};
#pragma unroll
                for (int blk = 0; blk < 4; ++blk) mma_m16n8k32_s8(acc[rt][blk], af, w[u][blk][0], w[u][blk][1]);
            }
        }
    }
    // per row tile: the eight warps' partial sums meet in shared memory, warp blk adds those of column block blk and
    // writes it: accumulator registers 0, 1 are row g, columns 2t and 2t+1 of the block; registers 2, 3 the same
    // columns of row g + 8
    const int col = n0 + 8 * (warp & 3) + 2 * t;
    const bool writes = warp < 4 && col < N;  // N is a multiple of 4 and col is even: col + 1 exists as well
    const float s0 = (writes && b_scale != nullptr) ? __ldg(b_scale + col) : 1.0f;
    const float s1 = (writes && b_scale != nullptr) ? __ldg(b_scale + col + 1) : 1.0f;
    const float z0 = (writes && bias != nullptr) ? out_bits_to_float<kOutBf16>(__ldg(bias + col)) : 0.0f;
    const float z1 = (writes && bias != nullptr) ? out_bits_to_float<kOutBf16>(__ldg(bias + col + 1)) : 0.0f;
#pragma unroll
    for (int rt = 0; rt < kRowTiles; ++rt) {
        if (rt > 0) __syncthreads();   // the previous row tile's sums have been read
#pragma unroll
        for (int blk = 0; blk < 4; ++blk) {
#pragma unroll
            for (int r = 0; r < 4; ++r) partial[warp][blk][r][lane] = acc[rt][blk][r];
        }
        __syncthreads();
        if (warp < 4) {
            int32_t sum[4] = {0, 0, 0, 0};
#pragma unroll
            for (int w2 = 0; w2 < kWmmaWarps; ++w2) {
#pragma unroll
                for (int r = 0; r < 4; ++r) sum[r] += partial[w2][warp][r][lane];
            }
            if (writes) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int row = row0 + 16 * rt + g + 8 * h;
                    if (row >= M) continue;
                    const float rs = __ldg(a_scale + row);
                    float v0 = static_cast<float>(sum[2 * h]) * rs;
                    float v1 = static_cast<float>(sum[2 * h + 1]) * rs;
                    if (b_scale != nullptr) {
                        v0 *= s0;
                        v1 *= s1;
                    }
                    if (bias != nullptr) {
                        v0 += z0;
                        v1 += z1;
                    }
                    *reinterpret_cast<uint32_t*>(c + static_cast<int64_t>(row) * N + col) = pack_out<kOutBf16>(v0, v1);
                }
            }
        }
    }
}

// True when the warp-MMA kernel takes the problem: forward direction, at most 16 rows (64 for outputs narrower than
// 8192 columns: measured 6.9-10.3 against 13.7-14.3 us at 3072 x 3072, 18.4-30.4 against 36 at 3072 x 12288, but 15.7-18.6
// against 15.1 at 12288 x 3072, where the pair kernel has 48 tiles to spread), operands aligned for its 8-byte
// activation loads, dword weight loads and 4-byte stores.
// FEATHER_INT8_WMMA_OFF=1 keeps few-row problems on the tcgen05 kernels (A/B measurements). Read once per process.
inline bool wmma_off() {
    static const bool off = env_switch("FEATHER_INT8_WMMA_OFF");
    return off;
}

bool wmma_eligible(const LaunchArgs& args) {
    return !args.transposed_b && args.M <= kWmmaMaxRows && (args.M <= 16 || args.N_out < kWmmaTwoTileMaxN) && args.N_out >= 256 && args.K % 16 == 0 && args.N_out % 4 == 0 &&
           (reinterpret_cast<uintptr_t>(args.a) & 7u) == 0 && (reinterpret_cast<uintptr_t>(args.b) & (args.plain ? 7u : 3u)) == 0 &&
           (reinterpret_cast<uintptr_t>(args.c) & 3u) == 0 && !wmma_off();
}

bool launch_wmma(const LaunchArgs& args) {
    const int row_tiles = args.M <= 16 ? 1 : 2;
    const dim3 grid(static_cast<unsigned>((args.N_out + 31) / 32), static_cast<unsigned>((args.M + 16 * row_tiles - 1) / (16 * row_tiles)));
#define FEATHER_I8_WMMA_CASE(RT, OUT, PLAIN)                                                                                       \
    if (row_tiles == RT && args.out_bf16 == OUT && args.plain == PLAIN) {                                                          \
        int8_mm_wmma_kernel<RT, OUT, PLAIN><<<grid, 32 * kWmmaWarps, 0, args.stream>>>(args.a, args.b, args.a_scale, args.b_scale, args.bias, args.c, \
                                                                                        static_cast<int>(args.M), static_cast<int>(args.N_out), \
                                                                                        static_cast<int>(args.K), args.stride_kc, args.stride_out); \
        return cudaGetLastError() == cudaSuccess;                                                                                  \
    }
    FEATHER_I8_WMMA_CASE(1, true, false)
    FEATHER_I8_WMMA_CASE(1, false, false)
    FEATHER_I8_WMMA_CASE(2, true, false)
    FEATHER_I8_WMMA_CASE(2, false, false)
    FEATHER_I8_WMMA_CASE(1, true, true)
    FEATHER_I8_WMMA_CASE(1, false, true)
    FEATHER_I8_WMMA_CASE(2, true, true)
    FEATHER_I8_WMMA_CASE(2, false, true)
#undef FEATHER_I8_WMMA_CASE
    return false;
}

// The pair kernel fetches the weight by TMA: the micro-tile axis that its boxes run along must be contiguous,
// the other stride must fit a tensor map, and the base must be 16-byte aligned.
bool pair_eligible(const LaunchArgs& args) {
    const int64_t fast = args.transposed_b ? args.stride_kc : args.stride_out;
    const int64_t slow = args.transposed_b ? args.stride_out : args.stride_kc;
    const int64_t fast_tiles = (args.transposed_b ? args.K : args.N_out) / 4;
    return fast == 1 && slow >= fast_tiles && slow < (int64_t{1} << 34) && (reinterpret_cast<uintptr_t>(args.b) & 15u) == 0;
}

bool launch_pair(const LaunchArgs& args) {
    if (args.plain) {
        if (args.transposed_b) {
            return args.out_bf16 ? launch_pair_instance<true, true, true>(args) : launch_pair_instance<true, false, true>(args);
        }
        return args.out_bf16 ? launch_pair_instance<false, true, true>(args) : launch_pair_instance<false, false, true>(args);
    }
    if (args.transposed_b) {
        return args.out_bf16 ? launch_pair_instance<true, true, false>(args) : launch_pair_instance<true, false, false>(args);
    }
    return args.out_bf16 ? launch_pair_instance<false, true, false>(args) : launch_pair_instance<false, false, false>(args);
}

template <int BN>
bool launch_for_block_n(const LaunchArgs& args) {
    if (args.transposed_b) {
        return args.out_bf16 ? launch_instance<BN, true, true>(args) : launch_instance<BN, true, false>(args);
    }
    return args.out_bf16 ? launch_instance<BN, false, true>(args) : launch_instance<BN, false, false>(args);
}

}  // namespace i8mm
}  // namespace feather

// C ABI, same signature as the reference's `launch_int8_scaled_mm` (csrc/hip_kernel_int8.cu:413-432).
// `b_stride_kc` / `b_stride_out` are the micro-tile strides of one 4-wide step along the contraction
// and the output axis of the weight. `output_dtype`: 0 = fp16, 1 = bf16. `a` must be 16-byte aligned and
// `K_contract` a multiple of 16; `N_out` a multiple of 4. Returns false for an unknown tile tuple.
extern "C" bool launch_int8_scaled_mm(const int8_t* a, const uint8_t* b, const float* a_scale, const float* b_scale, const uint16_t* bias,
                                      uint16_t* c, int64_t M, int64_t N_out, int64_t K_contract, int64_t b_stride_kc, int64_t b_stride_out,
                                      bool transposed_b, int block_warps_m, int block_warps_n, int unroll_k, int repeat_m, int repeat_n,
                                      int output_dtype, cudaStream_t stream) {
    using namespace feather;
    const int block_n = int8_tile_block_n(block_warps_m, block_warps_n, unroll_k, repeat_m, repeat_n);
    if (block_n == 0) return false;
    if (M < 0 || N_out <= 0 || K_contract <= 0 || N_out % 4 != 0 || K_contract % 16 != 0) return false;
    if (M > (1 << 30) || N_out > (1 << 30) || K_contract > (1 << 30)) return false;
    if (M == 0) return true;
    const i8mm::LaunchArgs args{a, b, a_scale, b_scale, bias, c, M, N_out, K_contract, b_stride_kc, b_stride_out,
                                transposed_b, output_dtype != 0, stream};
    if (i8mm::wmma_eligible(args)) return i8mm::launch_wmma(args);
    if (block_n >= 256) {
        // The pair kernel also serves a single row tile: its second CTA then multiplies zero rows, but the weight
        // re-layout is shared by two SMs and streams through TMA, which the single-CTA kernel's is not (a 256-wide
        // single-CTA tile costs four times as much per k block).
        if (i8mm::pair_eligible(args)) return i8mm::launch_pair(args);
        return i8mm::launch_for_block_n<256>(args);
    }
    if (block_n >= 128) return i8mm::launch_for_block_n<128>(args);
    return i8mm::launch_for_block_n<64>(args);
}

// The same product over the released row-major weight `w` = `[N, K]` int8 (no prepack): forward `C[M, N] = A[M, K] W^T` with both
// scales and the bias, backward (`transposed_b`) `C[M, K] = A[M, N] W` with the row scale only. The copy engine's 128 x 128 boxes of
// `w` are tensor-core operands as they land, so the kernel has no re-layout stage. `a`, `w` and `c` must be 16-byte aligned, `K` a
// multiple of 16 and `N` of 4 (backward: of 16, it is the activation's row length). No counterpart in the reference, whose kernels read the micro-tile prepack only. Returns false if the
// arguments do not fit.
extern "C" bool launch_int8_scaled_mm_plain(const int8_t* a, const int8_t* w, const float* a_scale, const float* b_scale, const uint16_t* bias,
                                            uint16_t* c, int64_t M, int64_t N, int64_t K, bool transposed_b, int output_dtype, cudaStream_t stream) {
    using namespace feather;
    if (M < 0 || N <= 0 || K <= 0 || N % (transposed_b ? 16 : 4) != 0 || K % 16 != 0) return false;
    if (M > (1 << 30) || N > (1 << 30) || K > (1 << 30)) return false;
    if (((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(c)) & 15u) != 0) return false;
    if (transposed_b && (b_scale != nullptr || bias != nullptr)) return false;
    if (M == 0) return true;
    i8mm::LaunchArgs args{a, reinterpret_cast<const uint8_t*>(w), a_scale, b_scale, bias, c, M, transposed_b ? K : N, transposed_b ? N : K, 0, 0,
                          transposed_b, output_dtype != 0, stream};
    args.plain = true;
    if (i8mm::wmma_eligible(args)) return i8mm::launch_wmma(args);   // a few rows, forward: the warp-MMA kernel reads the rows of w directly
    return i8mm::launch_pair(args);
}

// Output columns per tile that `launch_int8_scaled_mm_plain` picks for a product of `M` rows and `N` output columns (backward: the weight's
// input features) on a device with `pairs` resident CTA pairs (74 on a B200). For tests and logs.
extern "C" int feather_int8_plain_tile_width(int64_t M, int64_t N, int pairs, bool transposed_b) {
    return feather::i8mm::plain_tile_width(M, N, pairs, transposed_b ? 64 : 16);
}

// Reads and clears the int8 GEMM's wait-status record (see feather_scaled_mm_status).
extern "C" int feather_int8_mm_status(uint32_t* out) {
    uint32_t zero[2] = {0u, 0u};
    if (cudaDeviceSynchronize() != cudaSuccess) return 1;
    if (cudaMemcpyFromSymbol(out, feather::i8mm::g_status, sizeof(zero)) != cudaSuccess) return 1;
    if (cudaMemcpyToSymbol(feather::i8mm::g_status, zero, sizeof(zero)) != cudaSuccess) return 1;
    return 0;
}
