// scaled_mm for sm_100a: C[M,N] = cast(cast((A[M,K] @ upcast(B)) * scale) + bias)
//
//   A     fp16 or bf16, row-major, K contiguous
//   B     fp8 (e5m2 or e4m3fn), prepacked as [K_pad/16][N][16] bytes: the 16 bytes of one (k16, n) cell are the
//         sixteen consecutive k of column n, and K is zero padded to a multiple of 128
//   C     fp16 or bf16, row-major
//
// This is the B200 counterpart of `scaled_mm_kernel` / `launch_scaled_mm` in the reference's
// csrc/hip_kernel.cu (kernel :148-572, C ABI :687-713). Same contract, different machine:
//
//   * one persistent CTA per SM walks 128 x BN output tiles (m fastest so concurrently running CTAs share
//     a weight panel in L2);
//   * warp 0 is the TMA producer: per 64-wide k block it brings a 128 x 64 activation tile (128-byte
//     swizzle, zero fill past M and K) and the raw fp8 cells (boxes of 4 slabs x up to 128 cells, 2 KB
//     contiguous per box row) into a ring of load slots;
//   * sixteen upcast warps turn the raw cells into a K-major, 128-byte swizzled fp16 operand tile
//     (e5m2 -> fp16 is a byte placement, e4m3 -> fp16 one cvt per pair; both exact for every code)
//     in a second, shorter ring, fence it for the async proxy and hand it to the MMA warp;
//   * one thread of warp 1 issues tcgen05.mma kind::f16 (M=128, N=BN, K=16) into one of two TMEM
//     accumulators and commits to the barriers that recycle the slots;
//   * four epilogue warps read the finished accumulator (thread = output row), apply the scale, round,
//     add the bias in the output dtype, round again and store 64 contiguous bytes per thread per
//     32-column step, while the MMA warp already fills the other accumulator.
//
// That is the general kernel. Three relatives follow it in this file: the CTA-pair kernel (256 x 256 tiles over
// tcgen05 cta_group::2, used for M > 128 with the 256-wide tile: the headline path), the skinny kernel for M <= 128
// (64-wide tiles, two CTAs per SM, optional deterministic split-K) and the entry point that keeps the split-K
// scratch in the library's own device memory.
//
// The UMMA wants both operands in one 16-bit format (a bf16 x fp16 instruction descriptor is rejected as an
// illegal instruction), so the weights are decoded to the activation's format: fp16 by byte placement,
// bf16 through an exact fp16 -> fp32 -> bf16 conversion. Nothing is rounded before the fp32 accumulation.
#include "feather_host.h"
#include "feather_tiles_gen.h"
#include "sm100_ptx.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <cstdio>
#include <cstdlib>
#include <atomic>
#include <mutex>

namespace feather {
namespace smm {

constexpr int kBlockM = 128;
constexpr int kBlockK = 64;            // one 128-byte swizzle span of 16-bit elements
constexpr int kSlabsPerBlock = kBlockK / 16;
constexpr int kLoadStages = 4;
constexpr int kUpcastWarps = 16;
constexpr int kEpilogueWarps = 4;
constexpr int kFirstEpilogueWarp = 2;
constexpr int kFirstUpcastWarp = kFirstEpilogueWarp + kEpilogueWarps;
constexpr int kThreads = 32 * (kFirstUpcastWarp + kUpcastWarps);
constexpr int kATileBytes = kBlockM * kBlockK * 2;

__device__ uint32_t g_status[2];

struct Params {
    const float* scale;
    const uint16_t* bias;
    uint16_t* c;
    int M;
    int N;
    int K;
    int tiles_m;
    int tiles_n;
    uint32_t idesc;
    int bias_vec;  // bias pointer is 16-byte aligned
    int band;      // pair kernel: row tiles per band of the tile walk
    // one-CTA kernel with K split `splits` ways (1 = no split, the other three are then unused)
    int splits;
    int kb_per_split;
    float* partials;      // [splits][M][N] fp32
    uint32_t* counters;   // [tiles_m * tiles_n] tickets, zero before the launch and zero again after it
    int single_item;      // every CTA has exactly one (tile, split) item: the whole CTA adds the partials, not four warps
    int bulk_out;         // pair kernel: the output goes through shared-memory images and bulk tensor stores
    int cluster_reduce;   // pair kernel with a K split: the CTAs of a tile form one cluster and exchange partials through distributed shared memory
    int tile_n;           // pair kernel without a K split: output columns per tile, a multiple of 32 from 128 to 256
};

template <int BN>
struct Smem {
    static constexpr int kRawBytes = kSlabsPerBlock * BN * 16;
    static constexpr int kBoxCells = BN < 128 ? BN : 128;          // 16-byte cells per TMA box row
    static constexpr int kBoxes = BN / kBoxCells;                   // weight boxes per slot
    static constexpr int kBoxBytes = kSlabsPerBlock * kBoxCells * 16;
    static constexpr int kOperandBytes = BN * 128;
    // the upcast warps work as kTeams teams taking k blocks in turn (their barrier hand-offs overlap); ring depths are
    // multiples of the team count, and the widest tile only has room for two operand slots
    static constexpr int kTeams = 2;
    static constexpr int kOperandStages = BN == 256 ? 2 : 4;
    static_assert(kLoadStages % kTeams == 0 && kOperandStages % kTeams == 0, "ring depths must be multiples of the team count");
    static constexpr int kAOff = 0;
    static constexpr int kOperandOff = kAOff + kLoadStages * kATileBytes;
    static constexpr int kRawOff = kOperandOff + kOperandStages * kOperandBytes;
    static constexpr int kBarOff = kRawOff + kLoadStages * kRawBytes;
    // load full/empty, operand full/empty, tmem full/empty
    static constexpr int kNumBars = 2 * kLoadStages + 2 * kOperandStages + 4;
    static constexpr int kTotal = kBarOff + kNumBars * 8 + 16;
    static constexpr int kDynamic = kTotal + 1024;  // slack for the 1024-byte alignment of the base
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

// Two fp8 bytes -> two fp16 in one register. `kE5M2`: the byte is the high byte of the fp16 pattern.
template <bool kE5M2>
__device__ __forceinline__ void fp8x4_to_f16x4(uint32_t p, uint32_t& lo, uint32_t& hi) {
    if constexpr (kE5M2) {
        lo = __byte_perm(p, 0u, 0x1404u);
        hi = __byte_perm(p, 0u, 0x3424u);
    } else {
        const __half2_raw l = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(p & 0xffffu), __NV_E4M3);
        const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(p >> 16), __NV_E4M3);
        lo = static_cast<uint32_t>(l.x) | (static_cast<uint32_t>(l.y) << 16);
        hi = static_cast<uint32_t>(h.x) | (static_cast<uint32_t>(h.y) << 16);
    }
}

// fp16 pair -> bf16 pair, exact for every value an fp8 code can take (used only when the activation and
// weight operand formats have to match).
__device__ __forceinline__ uint32_t f16x2_to_bf16x2(uint32_t v) {
    const __half2 h = *reinterpret_cast<const __half2*>(&v);
    const float2 f = __half22float2(h);
    const __nv_bfloat162 b = __floats2bfloat162_rn(f.x, f.y);
    return *reinterpret_cast<const uint32_t*>(&b);
}

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
__device__ __forceinline__ float2 unpack_out(uint32_t v) {
    if constexpr (kOutBf16) {
        return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v));
    } else {
        return __half22float2(*reinterpret_cast<const __half2*>(&v));
    }
}

// Thirty-two consecutive accumulator columns of one output row (fp32 bit patterns): scale, round, add the bias,
// round again, store. Shared by the direct epilogue and the split-K reduction of the one-CTA kernel.
template <bool kOutBf16>
__device__ __forceinline__ void finish_columns(const Params& p, const uint32_t (&v)[32], float scale, int row, int col0, uint16_t* c_row) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        const int col = col0 + g * 8;
        uint32_t o[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            o[i] = pack_out<kOutBf16>(__uint_as_float(v[g * 8 + 2 * i]) * scale, __uint_as_float(v[g * 8 + 2 * i + 1]) * scale);
        }
        if (p.bias != nullptr && col < p.N) {
            uint32_t bw[4];
            if (p.bias_vec) {
                const uint4 b4 = __ldg(reinterpret_cast<const uint4*>(p.bias + col));
                bw[0] = b4.x;
                bw[1] = b4.y;
                bw[2] = b4.z;
                bw[3] = b4.w;
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    bw[i] = static_cast<uint32_t>(__ldg(p.bias + col + 2 * i)) | (static_cast<uint32_t>(__ldg(p.bias + col + 2 * i + 1)) << 16);
                }
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 x = unpack_out<kOutBf16>(o[i]);
                const float2 b = unpack_out<kOutBf16>(bw[i]);
                o[i] = pack_out<kOutBf16>(x.x + b.x, x.y + b.y);
            }
        }
        if (row < p.M && col < p.N) {
            *reinterpret_cast<uint4*>(c_row + col) = make_uint4(o[0], o[1], o[2], o[3]);
        }
    }
}

// kSplitK: the variant whose work items are (tile, K split); compiled apart so that the plain kernel keeps its registers.
template <int BN, bool kE5M2, bool kOperandBf16, bool kOutBf16, bool kSplitK>
__global__ void __launch_bounds__(kThreads, 1)
scaled_mm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const Params p) {
    using L = Smem<BN>;
    extern __shared__ uint8_t smem_dyn[];
    uint8_t* const smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~static_cast<uintptr_t>(1023));
    uint64_t* const bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
    uint64_t* const load_full = bars;
    uint64_t* const load_empty = load_full + kLoadStages;
    uint64_t* const operand_full = load_empty + kLoadStages;
    uint64_t* const operand_empty = operand_full + L::kOperandStages;
    uint64_t* const tmem_full = operand_empty + L::kOperandStages;
    uint64_t* const tmem_empty = tmem_full + 2;
    uint32_t* const tmem_slot = reinterpret_cast<uint32_t*>(bars + L::kNumBars);
    volatile uint32_t* const abort_flag = tmem_slot + 1;
    volatile uint32_t* const last_flag = tmem_slot + 2;  // split K: this CTA drew a tile's last ticket

    const int warp = static_cast<int>(threadIdx.x) / 32;
    const int lane = static_cast<int>(threadIdx.x) % 32;
    const WaitGuard guard{abort_flag, g_status};

    if (threadIdx.x == 0) {
        *abort_flag = 0u;
        *last_flag = 0u;
        for (int s = 0; s < kLoadStages; ++s) {
            mbar_init(&load_full[s], 1);
            mbar_init(&load_empty[s], 1);
        }
        for (int s = 0; s < L::kOperandStages; ++s) {
            mbar_init(&operand_full[s], kUpcastWarps / L::kTeams);
            mbar_init(&operand_empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&tmem_full[s], 1);
            mbar_init(&tmem_empty[s], kEpilogueWarps);
        }
        mbar_init_fence();
        tma_prefetch_desc(&map_a);
        tma_prefetch_desc(&map_b);
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
    // work item = (tile, K split); without a split an item is a tile and covers every k block
    const int splits = (kSplitK && p.splits > 1) ? p.splits : 1;
    const int kb_per_split = splits > 1 ? p.kb_per_split : num_kb;
    const int num_items = num_tiles * splits;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (elect_one()) {
            Ring slot;
            bool ok = true;
            for (int item = static_cast<int>(blockIdx.x); ok && item < num_items; item += static_cast<int>(gridDim.x)) {
                const int tile = item / splits;
                const int kb_begin = (item - tile * splits) * kb_per_split;
                const int kb_end = kb_begin + kb_per_split < num_kb ? kb_begin + kb_per_split : num_kb;
                const int m0 = (tile % p.tiles_m) * kBlockM;
                const int n0 = (tile / p.tiles_m) * BN;
                for (int kb = kb_begin; kb < kb_end; ++kb) {
                    ok = guard.wait(&load_empty[slot.idx], slot.phase ^ 1u, kSiteLoadEmpty);
                    if (!ok) break;
                    mbar_arrive_expect_tx(&load_full[slot.idx], kATileBytes + L::kRawBytes);
                    tma_load_2d(smem + L::kAOff + slot.idx * kATileBytes, &map_a, &load_full[slot.idx], kb * kBlockK, m0);
#pragma unroll
                    for (int box = 0; box < L::kBoxes; ++box) {
                        tma_load_2d(smem + L::kRawOff + slot.idx * L::kRawBytes + box * L::kBoxBytes, &map_b, &load_full[slot.idx],
                                    (n0 + box * L::kBoxCells) * 2, kb * kSlabsPerBlock);
                    }
                    slot.advance(kLoadStages);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (elect_one()) {
            Ring slot, operand, acc;
            bool ok = true;
            for (int item = static_cast<int>(blockIdx.x); ok && item < num_items; item += static_cast<int>(gridDim.x)) {
                ok = guard.wait(&tmem_empty[acc.idx], acc.phase ^ 1u, kSiteTmemEmpty);
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t tmem_d = tmem_base + acc.idx * BN;
                const int kb_begin = (item % splits) * kb_per_split;
                const int kb_end = kb_begin + kb_per_split < num_kb ? kb_begin + kb_per_split : num_kb;
                for (int kb = kb_begin; kb < kb_end; ++kb) {
                    ok = guard.wait(&load_full[slot.idx], slot.phase, kSiteLoadFull, 1) &&
                         guard.wait(&operand_full[operand.idx], operand.phase, kSiteOperandFull);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint32_t a_addr = smem_u32(smem + L::kAOff + slot.idx * kATileBytes);
                    const uint32_t b_addr = smem_u32(smem + L::kOperandOff + operand.idx * L::kOperandBytes);
#pragma unroll
                    for (int k = 0; k < kBlockK / 16; ++k) {
                        umma_f16(tmem_d, make_desc_sw128_kmajor(a_addr + k * 32), make_desc_sw128_kmajor(b_addr + k * 32), p.idesc,
                                 (kb != kb_begin || k != 0) ? 1u : 0u);
                    }
                    umma_commit(&load_empty[slot.idx]);
                    umma_commit(&operand_empty[operand.idx]);
                    slot.advance(kLoadStages);
                    operand.advance(L::kOperandStages);
                }
                if (!ok) break;
                umma_commit(&tmem_full[acc.idx]);
                acc.advance(2);
            }
        }
    } else if (warp < kFirstUpcastWarp) {
        // ------------------------------------------------------------------ epilogue
        const int quarter = warp % 4;  // the TMEM lane quarter this warp is allowed to read
        const float scale = p.scale != nullptr ? __ldg(p.scale) : 1.0f;
        Ring acc;
        bool ok = true;
        for (int item = static_cast<int>(blockIdx.x); ok && item < num_items; item += static_cast<int>(gridDim.x)) {
            const int tile = item / splits;
            const int split = item - tile * splits;
            const int m0 = (tile % p.tiles_m) * kBlockM;
            const int n0 = (tile / p.tiles_m) * BN;
            const bool got = guard.wait(&tmem_full[acc.idx], acc.phase, kSiteTmemFull);
            if ((!kSplitK || splits == 1) && !got) {
                ok = false;
                break;
            }
            tc_fence_after_sync();
            const int row = m0 + quarter * 32 + lane;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc.idx * BN;
            uint16_t* const c_row = p.c + static_cast<int64_t>(row) * p.N;
            if (!kSplitK || splits == 1) {
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    uint32_t v[32];
                    tmem_ld_32x32(taddr + c * 32, v);
                    tmem_wait_ld();
                    if (c == BN / 32 - 1) {
                        // the accumulator is in registers: hand the TMEM buffer back before the stores
                        tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&tmem_empty[acc.idx]);
                    }
                    finish_columns<kOutBf16>(p, v, scale, row, n0 + c * 32, c_row);
                }
            } else if constexpr (kSplitK) {
                // K split: this CTA's fp32 partial goes to scratch, a ticket per tile says which CTA came last, and
                // that one adds the partials in split order (so the sum does not depend on who it was) and finishes.
                // The four epilogue warps meet at two named barriers per item, so none of them may leave the loop
                // between the two: a warp whose wait ran out skips the work, and the second barrier tells all four.
                // Scratch layout: [split][tile][32-column chunk][4-column group][row of the tile][4], so that the 32
                // lanes of a warp (32 rows) write and read 512 consecutive bytes per instruction.
                constexpr int kTileFloats = kBlockM * BN;
                const int slot_row = (quarter * 32 + lane) * 4;
                float* const part_tile = p.partials + (static_cast<int64_t>(split) * num_tiles + tile) * kTileFloats;
#pragma unroll 1
                for (int c = 0; got && c < BN / 32; ++c) {
                    uint32_t v[32];
                    tmem_ld_32x32(taddr + c * 32, v);
                    tmem_wait_ld();
                    if (c == BN / 32 - 1) {
                        // the accumulator is in registers: hand the TMEM buffer back before the stores
                        tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&tmem_empty[acc.idx]);
                    }
                    // with one item per CTA the chunks this CTA adds itself stay in tensor memory (nothing reuses the buffer)
                    if (p.single_item != 0 && c % splits == split) continue;
#pragma unroll
                    for (int g = 0; g < 8; ++g) {
                        __stcg(reinterpret_cast<uint4*>(part_tile + (c * 8 + g) * (kBlockM * 4) + slot_row),
                               make_uint4(v[4 * g], v[4 * g + 1], v[4 * g + 2], v[4 * g + 3]));
                    }
                }
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (threadIdx.x == kFirstEpilogueWarp * 32) {
                    if (p.single_item != 0) {
                        // one item per CTA: count this split in; the tile's CTAs share the reduction after the role loops
                        if (got) {
                            __threadfence();
                            atomicAdd(p.counters + tile, 1u);
                        }
                    } else {
                        const uint32_t ticket = atomicAdd(p.counters + tile, 1u);
                        const bool last = ticket == static_cast<uint32_t>(splits - 1);
                        if (last) p.counters[tile] = 0u;  // every other split has drawn its ticket: ready for the next launch
                        *last_flag = last ? 1u : 0u;
                    }
                }
                uint32_t any_failed;
                asm volatile(
                    "{\n\t"
                    ".reg .pred P, Q;\n\t"
                    "setp.ne.u32 P, %1, 0;\n\t"
                    "bar.red.or.pred Q, 1, 128, P;\n\t"
                    "selp.u32 %0, 1, 0, Q;\n\t"
                    "}"
                    : "=r"(any_failed)
                    : "r"(got ? 0u : 1u)
                    : "memory");
                if (any_failed != 0u) {
                    ok = false;
                    break;
                }
                if (p.single_item != 0) {
                    // the whole CTA adds the partials after the role loops (below): twenty warps instead of four
                } else if (*last_flag != 0u) {
                    // Holding the accumulator back so that the last CTA could add its own partial from tensor memory
                    // was measured slower than reading all of them from the scratch: the MMA warp waits for the buffer.
                    __threadfence();
                    // (Sixteen columns at a time with the loads of four splits in flight before the first add was measured
                    // too: not faster, 20.6 against 19.5 us at 128 x 4096 x 4096 with four splits.)
#pragma unroll 1
                    for (int c = 0; c < BN / 32; ++c) {
                        float sum[32];
#pragma unroll
                        for (int i = 0; i < 32; ++i) sum[i] = 0.0f;
                        for (int sp = 0; sp < splits; ++sp) {
                            const float* const src = p.partials + (static_cast<int64_t>(sp) * num_tiles + tile) * kTileFloats + slot_row;
#pragma unroll
                            for (int g = 0; g < 8; ++g) {
                                const float4 x = __ldcg(reinterpret_cast<const float4*>(src + (c * 8 + g) * (kBlockM * 4)));
                                sum[4 * g] += x.x;
                                sum[4 * g + 1] += x.y;
                                sum[4 * g + 2] += x.z;
                                sum[4 * g + 3] += x.w;
                            }
                        }
                        uint32_t v[32];
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(sum[i]);
                        finish_columns<kOutBf16>(p, v, scale, row, n0 + c * 32, c_row);
                    }
                }
            }
            acc.advance(2);
        }
    } else {
        // ------------------------------------------------------------------ upcast warps
        // Work unit = one 16-byte cell (row n, slab j): unit u = t + i * threads, row = u % BN, slab = u / BN.
        const int t = static_cast<int>(threadIdx.x) - kFirstUpcastWarp * 32;
        constexpr int kTeamThreads = kUpcastWarps * 32 / L::kTeams;
        constexpr int kUnits = BN * kSlabsPerBlock;
        constexpr int kUnitsPerThread = (kUnits + kTeamThreads - 1) / kTeamThreads;
        const int team = t / kTeamThreads;
        const int tt = t % kTeamThreads;
        Ring slot, operand;
        bool ok = true;
        uint32_t turn = 0;  // k blocks since the start of the kernel, modulo the number of teams
        for (int item = static_cast<int>(blockIdx.x); ok && item < num_items; item += static_cast<int>(gridDim.x)) {
            const int kb_begin = (item % splits) * kb_per_split;
            const int kb_end = kb_begin + kb_per_split < num_kb ? kb_begin + kb_per_split : num_kb;
            for (int kb = kb_begin; kb < kb_end; ++kb) {
                if (turn == static_cast<uint32_t>(team)) {
                    ok = guard.wait(&load_full[slot.idx], slot.phase, kSiteLoadFull, 2) &&
                         guard.wait(&operand_empty[operand.idx], operand.phase ^ 1u, kSiteOperandEmpty);
                    if (!ok) break;
                    const uint8_t* const raw = smem + L::kRawOff + slot.idx * L::kRawBytes;
                    uint8_t* const dst = smem + L::kOperandOff + operand.idx * L::kOperandBytes;
                    uint4 cells[kUnitsPerThread];
#pragma unroll
                    for (int i = 0; i < kUnitsPerThread; ++i) {
                        const int u = tt + i * kTeamThreads;
                        if (kUnits % kTeamThreads == 0 || u < kUnits) {
                            const int row = u % BN;
                            const int slab = u / BN;
                            cells[i] = *reinterpret_cast<const uint4*>(raw + (row / L::kBoxCells) * L::kBoxBytes + (slab * L::kBoxCells + row % L::kBoxCells) * 16);
                        }
                    }
#pragma unroll
                    for (int i = 0; i < kUnitsPerThread; ++i) {
                        const int u = tt + i * kTeamThreads;
                        if (kUnits % kTeamThreads != 0 && u >= kUnits) continue;
                        const int row = u % BN;
                        const int slab = u / BN;
                        const uint32_t w[4] = {cells[i].x, cells[i].y, cells[i].z, cells[i].w};
                        uint32_t h[8];
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            fp8x4_to_f16x4<kE5M2>(w[q], h[2 * q], h[2 * q + 1]);
                            if constexpr (kOperandBf16) {
                                h[2 * q] = f16x2_to_bf16x2(h[2 * q]);
                                h[2 * q + 1] = f16x2_to_bf16x2(h[2 * q + 1]);
                            }
                        }
                        *reinterpret_cast<uint4*>(dst + sw128_offset(row, 2 * slab)) = make_uint4(h[0], h[1], h[2], h[3]);
                        *reinterpret_cast<uint4*>(dst + sw128_offset(row, 2 * slab + 1)) = make_uint4(h[4], h[5], h[6], h[7]);
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&operand_full[operand.idx]);
                }
                turn = turn + 1 == L::kTeams ? 0 : turn + 1;
                slot.advance(kLoadStages);
                operand.advance(L::kOperandStages);
            }
        }
    }

    if constexpr (kSplitK) {
        if (p.single_item != 0 && splits > 1) {
            // One item per CTA, all of them resident at once: every role loop has ended. Wait (bounded) until every split of the
            // tile is in, then add the partials of THIS CTA's share of the 32-column chunks (chunk c belongs to split c % splits)
            // in split order, twenty warps at work. One CTA adding a whole tile reads all its partials through its own L2 port
            // (six splits of a 128 x 128 tile: 384 KB, 6 us); spread over the tile's CTAs it is a sixth of that each.
            __syncthreads();
            const int tile = static_cast<int>(blockIdx.x) / splits;
            const int split = static_cast<int>(blockIdx.x) - tile * splits;
            if (threadIdx.x == 0 && !guard.aborted()) {
                const uint32_t* const in_counter = p.counters + tile;
                const long long start = clock64();
                while (true) {
                    uint32_t seen;
                    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(in_counter) : "memory");
                    if (seen >= static_cast<uint32_t>(splits)) break;
                    if (clock64() - start > kWaitLimitCycles) {
                        guard.give_up(kSiteStore, 7);
                        break;
                    }
                    __nanosleep(64);
                }
                __threadfence();
            }
            __syncthreads();
            if (!guard.aborted() && threadIdx.x >= kFirstEpilogueWarp * 32) {
                constexpr int kTileFloats = kBlockM * BN;
                constexpr int kGroups = (kThreads - kFirstEpilogueWarp * 32) / kBlockM;   // 128 threads (one per row) each
                const int t = static_cast<int>(threadIdx.x) - kFirstEpilogueWarp * 32;
                const int group = t / kBlockM;
                // a warp reads the tensor-memory lanes 32 * (warp % 4) .. + 31, so its threads take those rows of the tile
                const int r = (warp % 4) * 32 + lane;
                const uint32_t own_taddr = tmem_base + (static_cast<uint32_t>((warp % 4) * 32) << 16);   // the item's accumulator: buffer 0
                tc_fence_after_sync();
                const int row = (tile % p.tiles_m) * kBlockM + r;
                const int n0 = (tile / p.tiles_m) * BN;
                const float scale = p.scale != nullptr ? __ldg(p.scale) : 1.0f;
                uint16_t* const c_row = p.c + static_cast<int64_t>(row) * p.N;
                int owned = 0;
#pragma unroll 1
                for (int c = split; c < BN / 32; c += splits, ++owned) {
                    if (group >= kGroups || owned % kGroups != group) continue;
                    float sum[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) sum[i] = 0.0f;
                    for (int sp = 0; sp < splits; ++sp) {  // split order: the sum does not depend on who adds it
                        if (sp == split) {
                            // this CTA's own partial of the chunk never left tensor memory
                            uint32_t own[32];
                            tmem_ld_32x32(own_taddr + c * 32, own);
                            tmem_wait_ld();
#pragma unroll
                            for (int i = 0; i < 32; ++i) sum[i] += __uint_as_float(own[i]);
                            continue;
                        }
                        const float* const src = p.partials + (static_cast<int64_t>(sp) * num_tiles + tile) * kTileFloats + r * 4;
#pragma unroll
                        for (int g = 0; g < 8; ++g) {
                            const float4 x = __ldcg(reinterpret_cast<const float4*>(src + (c * 8 + g) * (kBlockM * 4)));
                            sum[4 * g] += x.x;
                            sum[4 * g + 1] += x.y;
                            sum[4 * g + 2] += x.z;
                            sum[4 * g + 3] += x.w;
                        }
                    }
                    uint32_t v[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(sum[i]);
                    finish_columns<kOutBf16>(p, v, scale, row, n0 + c * 32, c_row);
                }
            }
            __syncthreads();
            if (threadIdx.x == 0) {
                // this CTA has read what it needs: the last of the tile's CTAs puts both tickets back to zero
                __threadfence();
                uint32_t* const done = p.counters + num_tiles + tile;
                if (atomicAdd(done, 1u) == static_cast<uint32_t>(splits - 1)) {
                    p.counters[tile] = 0u;
                    *done = 0u;
                }
            }
        }
    }

    // ---------------------------------------------------------------------- teardown
    tc_fence_before_sync();
    __syncthreads();
    if (guard.aborted()) {
        // give copies and MMAs that were in flight when a wait ran out time to land before the CTA's
        // shared and tensor memory go away
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
// CTA-pair version (tcgen05 cta_group::2): a cluster of two CTAs owns a 256 x 256 output tile. CTA r of the
// pair loads activation rows [128 r, 128 r + 128) and weight columns [128 r, 128 r + 128) of the tile,
// converts only that half of the weight tile, and receives accumulator rows [128 r, 128 r + 128) x 256
// columns in its own tensor memory. The UMMA (M = 256, N = 256, K = 16) is issued by CTA 0 and reads both
// CTAs' shared memory, so per SM the converted-operand traffic and the conversion work are half of the
// one-CTA kernel's for the same number of flops. Barriers that CTA 0's MMA thread waits on live in CTA 0
// and are arrived on remotely by CTA 1's warps; barriers that release slots or publish an accumulator are
// signalled in both CTAs by two commits.
// ---------------------------------------------------------------------------------------------------------
// Both ring depths are multiples of the number of upcast teams: a team then always meets the same slots and
// sees every phase of the barriers it waits on (a waiter that skipped phases could mistake an old phase of the
// same parity for the one it needs).
constexpr int kPairLoadStages = 6;
constexpr int kPairOperandStages = 4;
constexpr int kPairTeams = 2;   // upcast teams taking k blocks in turn (measured: 1 team 1.27, 2 or 4 teams 1.35 PFLOP/s)
static_assert(kPairLoadStages % kPairTeams == 0 && kPairOperandStages % kPairTeams == 0, "ring depths must be multiples of the team count");
constexpr int kPairHalfN = 128;
constexpr int kPairN = 2 * kPairHalfN;

struct PairSmem {
    static constexpr int kRawBytes = kSlabsPerBlock * kPairHalfN * 16;   // 8 KB
    static constexpr int kOperandBytes = kPairHalfN * 128;               // 16 KB
    static constexpr int kAOff = 0;
    static constexpr int kOperandOff = kAOff + kPairLoadStages * kATileBytes;
    static constexpr int kRawOff = kOperandOff + kPairOperandStages * kOperandBytes;
    static constexpr int kImageBytes = kBlockM * 64;   // 128 rows x 32 output columns of 16 bits: four warps' slices of 32 rows, one bulk tensor store each
    static constexpr int kImageOff = kRawOff + kPairLoadStages * kRawBytes;   // two images: a warp writes its slice of one while the copy engine reads that of the other
    static constexpr int kBarOff = kImageOff + 2 * kImageBytes;
    static constexpr int kNumBars = 2 * kPairLoadStages + 2 * kPairOperandStages + 4;
    static constexpr int kTotal = kBarOff + kNumBars * 8 + 16;
    static constexpr int kDynamic = kTotal + 1024;
    static_assert(kImageOff % 1024 == 0, "swizzled images sit on a 1 KB boundary");
    static_assert(kDynamic <= 227 * 1024, "a CTA's shared memory");
};

// kSplitK: every pair has exactly ONE work item (tile, K split) instead of walking tiles; compiled apart so that the plain
// kernel keeps its registers. A pair writes its fp32 partial tile to scratch and counts itself in; then every CTA of the tile
// (two per split) waits, with a limit, until all splits of its half of the rows are in, and adds the partials of ITS share
// of the 32-column chunks in split order: the reduction is spread over all the CTAs that worked on the tile instead of one
// CTA reading every partial through its own L2 port. All pairs of the grid are resident at once (the launcher checks), so the
// wait cannot starve. Scratch: [tile][row half][split][chunk][4-column group][row][4] fp32; tickets: two "in" counters per tile
// (one per row half) and one "done" counter, whose last arriver puts all three back to zero for the next launch.
// With at most four splits, and when every cluster of the launch fits the device at once, the pairs of a tile are launched as ONE
// cluster instead (`cluster_reduce`): partials go from tensor memory straight into the shared memory of the CTA that adds them, and
// neither scratch nor tickets are touched. Both ways add in split order, so they give the same bits.
template <bool kE5M2, bool kOperandBf16, bool kOutBf16, bool kSplitK = false>
__global__ void __launch_bounds__(kThreads, 1)
scaled_mm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_c, const Params p) {
    using L = PairSmem;
    extern __shared__ uint8_t smem_dyn[];
    uint8_t* const smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~static_cast<uintptr_t>(1023));
    uint64_t* const bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
    uint64_t* const load_full = bars;
    uint64_t* const load_empty = load_full + kPairLoadStages;
    uint64_t* const operand_full = load_empty + kPairLoadStages;      // used in CTA 0 only
    uint64_t* const operand_empty = operand_full + kPairOperandStages;
    uint64_t* const tmem_full = operand_empty + kPairOperandStages;
    uint64_t* const tmem_empty = tmem_full + 2;                        // used in CTA 0 only
    uint32_t* const tmem_slot = reinterpret_cast<uint32_t*>(bars + L::kNumBars);
    volatile uint32_t* const abort_flag = tmem_slot + 1;

    const int warp = static_cast<int>(threadIdx.x) / 32;
    const int lane = static_cast<int>(threadIdx.x) % 32;
    // The cluster is one CTA pair, or with `cluster_reduce` all the pairs of a tile: ranks 2 i and 2 i + 1 are pair i.
    const uint32_t cluster_rank = cluster_cta_rank();
    const uint32_t cta = cluster_rank & 1u;
    const uint32_t pair_base = cluster_rank & ~1u;
    const WaitGuard guard{abort_flag, g_status};

    if (threadIdx.x == 0) {
        *abort_flag = 0u;
        for (int s = 0; s < kPairLoadStages; ++s) {
            mbar_init(&load_full[s], 1);
            mbar_init(&load_empty[s], 1);
        }
        for (int s = 0; s < kPairOperandStages; ++s) {
            mbar_init(&operand_full[s], 2 * kUpcastWarps / kPairTeams);
            mbar_init(&operand_empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&tmem_full[s], 1);
            mbar_init(&tmem_empty[s], 2 * kEpilogueWarps);
        }
        mbar_init_fence();
        tma_prefetch_desc(&map_a);
        tma_prefetch_desc(&map_b);
        if (!kSplitK && p.bulk_out) tma_prefetch_desc(&map_c);
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, 2 * kPairN);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();  // the peer's barriers are initialised before anything is signalled across CTAs
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    const int tiles_m = (p.M + 2 * kBlockM - 1) / (2 * kBlockM);
    const int tile_cols = kSplitK ? kPairN : p.tile_n;   // output columns per tile; each CTA stages half of them as weight rows
    const int tiles_n = (p.N + tile_cols - 1) / tile_cols;
    const int num_tiles = tiles_m * tiles_n;
    const int num_kb = (p.K + kBlockK - 1) / kBlockK;
    // plain: pair i walks tiles i, i + pairs, ...; split K: pair i has the one item (tile i / splits, split i % splits)
    const int item = static_cast<int>(blockIdx.x) / 2;
    const int my_split = kSplitK ? item % p.splits : 0;
    const int first_tile = kSplitK ? item / p.splits : item;
    const int tile_step = kSplitK ? num_tiles : static_cast<int>(gridDim.x) / 2;
    const int kb_begin = kSplitK ? my_split * p.kb_per_split : 0;
    const int kb_end = kSplitK ? (kb_begin + p.kb_per_split < num_kb ? kb_begin + p.kb_per_split : num_kb) : num_kb;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (this CTA's halves)
        if (elect_one()) {
            Ring slot;
            bool ok = true;
            for (int tile = first_tile; ok && tile < num_tiles; tile += tile_step) {
                int tile_m, tile_n;
                banded_tile(tile, tiles_m, tiles_n, p.band, tile_m, tile_n);
                const int m0 = tile_m * 2 * kBlockM + static_cast<int>(cta) * kBlockM;
                const int n0 = tile_n * tile_cols + static_cast<int>(cta) * (tile_cols / 2);
                const uint32_t raw_bytes = static_cast<uint32_t>(kSlabsPerBlock * (tile_cols / 2) * 16);   // the box: [slab][this CTA's columns][16]
                for (int kb = kb_begin; kb < kb_end; ++kb) {
                    ok = guard.wait(&load_empty[slot.idx], slot.phase ^ 1u, kSiteLoadEmpty);
                    if (!ok) break;
                    mbar_arrive_expect_tx(&load_full[slot.idx], kATileBytes + raw_bytes);
                    tma_load_2d(smem + L::kAOff + slot.idx * kATileBytes, &map_a, &load_full[slot.idx], kb * kBlockK, m0);
                    tma_load_2d(smem + L::kRawOff + slot.idx * L::kRawBytes, &map_b, &load_full[slot.idx], n0 * 2, kb * kSlabsPerBlock);
                    slot.advance(kPairLoadStages);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (CTA 0 of the pair)
        if (cta == 0 && elect_one()) {
            Ring slot, operand, acc;
            bool ok = true;
            // every barrier the UMMA completion has to reach, in this CTA and at the same offset in the peer
            for (int tile = first_tile; ok && tile < num_tiles; tile += tile_step) {
                ok = guard.wait(&tmem_empty[acc.idx], acc.phase ^ 1u, kSiteTmemEmpty);
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t tmem_d = tmem_base + acc.idx * kPairN;
                for (int kb = kb_begin; kb < kb_end; ++kb) {
                    ok = guard.wait(&load_full[slot.idx], slot.phase, kSiteLoadFull, 1) &&
                         guard.wait(&operand_full[operand.idx], operand.phase, kSiteOperandFull);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint32_t a_addr = smem_u32(smem + L::kAOff + slot.idx * kATileBytes);
                    const uint32_t b_addr = smem_u32(smem + L::kOperandOff + operand.idx * L::kOperandBytes);
#pragma unroll
                    for (int k = 0; k < kBlockK / 16; ++k) {
                        umma_f16_pair(tmem_d, make_desc_sw128_kmajor(a_addr + k * 32), make_desc_sw128_kmajor(b_addr + k * 32), p.idesc,
                                      (kb != kb_begin || k != 0) ? 1u : 0u);
                    }
#pragma unroll
                    for (uint32_t dst = 0; dst < 2; ++dst) {
                        umma_commit_pair(map_to_cta(smem_u32(&load_empty[slot.idx]), pair_base + dst));
                        umma_commit_pair(map_to_cta(smem_u32(&operand_empty[operand.idx]), pair_base + dst));
                    }
                    slot.advance(kPairLoadStages);
                    operand.advance(kPairOperandStages);
                }
                if (!ok) break;
#pragma unroll
                for (uint32_t dst = 0; dst < 2; ++dst) umma_commit_pair(map_to_cta(smem_u32(&tmem_full[acc.idx]), pair_base + dst));
                acc.advance(2);
            }
        }
    } else if (warp < kFirstUpcastWarp) {
        // ------------------------------------------------------------------ epilogue (this CTA's 128 rows)
        const int quarter = warp % 4;
        const float scale = p.scale != nullptr ? __ldg(p.scale) : 1.0f;
        // With `bulk_out` a warp's 32 rows x 32 columns of a chunk go into a 64-byte-swizzled shared-memory image that its first lane
        // hands to the copy engine (which clips at M and N): a lane holds one row, so the direct stores are 32 requests of 16 bytes
        // per warp instruction, and the drain of a pair's last tile has nothing to hide behind. One image per warp rather than one
        // per chunk: the four warps then never wait for one another (two hand-offs per chunk cost a quarter of the epilogue's time).
        const int twist = (lane >> 1) & 3;   // 64-byte swizzle: the 16-byte chunk index is XORed with bits 7-8 of the address (the slices are 2 KB apart)
        uint32_t stores = 0;
        Ring acc;
        bool ok = true;
        for (int tile = first_tile; ok && tile < num_tiles; tile += tile_step) {
            int tile_m, tile_n;
            banded_tile(tile, tiles_m, tiles_n, p.band, tile_m, tile_n);
            const int m0 = tile_m * 2 * kBlockM + static_cast<int>(cta) * kBlockM;
            const int n0 = tile_n * tile_cols;
            ok = guard.wait(&tmem_full[acc.idx], acc.phase, kSiteTmemFull);
            if (!kSplitK && !ok) break;   // the K-split path below meets its named barrier whatever the wait returned
            tc_fence_after_sync();
            const int row = m0 + quarter * 32 + lane;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc.idx * kPairN;
            uint16_t* const c_row = p.c + static_cast<int64_t>(row) * p.N;
            if constexpr (kSplitK) {
                if (p.cluster_reduce) break;   // the accumulator is complete; the exchange below reads it from tensor memory
                // this pair's partial of the tile goes to scratch; a warp writes 512 consecutive bytes per instruction
                float* const part = p.partials + ((static_cast<int64_t>(tile) * 2 + cta) * p.splits + my_split) * (kBlockM * kPairN) + (quarter * 32 + lane) * 4;
#pragma unroll 1
                for (int c = 0; ok && c < kPairN / 32; ++c) {
                    if (c % p.splits == my_split) continue;   // this CTA adds these chunks itself and takes its own share from tensor memory
                    uint32_t v[32];
                    tmem_ld_32x32(taddr + c * 32, v);
                    tmem_wait_ld();
#pragma unroll
                    for (int g = 0; g < 8; ++g) {
                        __stcg(reinterpret_cast<uint4*>(part + (c * 8 + g) * (kBlockM * 4)), make_uint4(v[4 * g], v[4 * g + 1], v[4 * g + 2], v[4 * g + 3]));
                    }
                }
                __threadfence();
                // the four epilogue warps: this CTA's half of the partial is out. Every warp comes here, also one whose wait gave
                // up (it wrote nothing and the tile is not counted in: the reducers then run out of their own bounded wait).
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (threadIdx.x == kFirstEpilogueWarp * 32 && !guard.aborted()) {
                    __threadfence();
                    atomicAdd(p.counters + tile * 2 + static_cast<int>(cta), 1u);
                }
                break;   // one item per pair
            }
            const int chunks = tile_cols / 32;
#pragma unroll 1
            for (int c = 0; c < chunks; ++c) {
                uint32_t v[32];
                tmem_ld_32x32(taddr + c * 32, v);
                tmem_wait_ld();
                if (c == chunks - 1) {
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tmem_empty[acc.idx]), pair_base));
                }
                const int col0 = n0 + c * 32;
                uint32_t out_words[16];
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    const int col = col0 + g * 8;
                    uint32_t* const o = out_words + 4 * g;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        o[i] = pack_out<kOutBf16>(__uint_as_float(v[g * 8 + 2 * i]) * scale, __uint_as_float(v[g * 8 + 2 * i + 1]) * scale);
                    }
                    if (p.bias != nullptr && col < p.N) {
                        uint32_t bw[4];
                        if (p.bias_vec) {
                            const uint4 b4 = __ldg(reinterpret_cast<const uint4*>(p.bias + col));
                            bw[0] = b4.x;
                            bw[1] = b4.y;
                            bw[2] = b4.z;
                            bw[3] = b4.w;
                        } else {
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                bw[i] = static_cast<uint32_t>(__ldg(p.bias + col + 2 * i)) | (static_cast<uint32_t>(__ldg(p.bias + col + 2 * i + 1)) << 16);
                            }
                        }
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const float2 x = unpack_out<kOutBf16>(o[i]);
                            const float2 b = unpack_out<kOutBf16>(bw[i]);
                            o[i] = pack_out<kOutBf16>(x.x + b.x, x.y + b.y);
                        }
                    }
                    if (!p.bulk_out && row < p.M && col < p.N) {
                        *reinterpret_cast<uint4*>(c_row + col) = make_uint4(o[0], o[1], o[2], o[3]);
                    }
                }
                if (p.bulk_out) {
                    if (col0 >= p.N) continue;
                    // a warp's 32 rows of the chunk are an image of their own (2 KB, two of them used alternately) that the warp's
                    // first lane hands to the copy engine: no hand-off between the warps, only the lane's own stores to wait for
                    const uint32_t img = stores & 1u;
                    if (stores >= 2) {
                        if (lane == 0) tma_store_wait_read<1>();   // all but this lane's newest store have been read: this image's last one too
                        __syncwarp();
                    }
                    uint8_t* const image = smem + L::kImageOff + img * L::kImageBytes + quarter * (32 * 64);
                    uint8_t* const image_row = image + lane * 64;
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        *reinterpret_cast<uint4*>(image_row + ((g ^ twist) << 4)) = make_uint4(out_words[4 * g], out_words[4 * g + 1], out_words[4 * g + 2], out_words[4 * g + 3]);
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_2d(&map_c, image, col0, m0 + quarter * 32);
                        tma_store_commit();
                    }
                    ++stores;
                }
            }
            acc.advance(2);
        }
        if (!kSplitK && p.bulk_out && lane == 0) tma_store_wait<0>();   // the images must outlive the copy engine's reads, and the stores the kernel
    } else {
        // ------------------------------------------------------------------ upcast warps (this CTA's weight half)
        // The warps form kPairTeams teams that take the k blocks in turn, so a team has kPairTeams k-block times
        // for its chain (wait, shared load, convert, shared store, proxy fence, arrive) and the chains of
        // consecutive k blocks overlap. Within a team: cell u = (slab u / 128, row u % 128), u = t + i * team size.
        constexpr int kTeamThreads = kUpcastWarps * 32 / kPairTeams;
        const int upcast_thread = static_cast<int>(threadIdx.x) - kFirstUpcastWarp * 32;
        const int team = upcast_thread / kTeamThreads;
        const int t = upcast_thread % kTeamThreads;
        constexpr int kUnits = kPairHalfN * kSlabsPerBlock;
        constexpr int kUnitsPerThread = kUnits / kTeamThreads;
        static_assert(kUnits % kTeamThreads == 0, "the weight half tile must split evenly over a team");
        // a narrower tile has fewer cells per k block: cell u sits at byte 16 u of the box, and where it goes does not depend on the k block
        const int half_cols = tile_cols / 2;
        const int units = half_cols * kSlabsPerBlock;
        uint32_t dst_offset[kUnitsPerThread];
#pragma unroll
        for (int i = 0; i < kUnitsPerThread; ++i) {
            const int u = t + i * kTeamThreads;
            dst_offset[i] = sw128_offset(static_cast<uint32_t>(u % half_cols), 2u * static_cast<uint32_t>(u / half_cols));
        }
        Ring slot, operand;
        bool ok = true;
        uint32_t turn = 0;  // k blocks since the start of the kernel, modulo the number of teams
        for (int tile = first_tile; ok && tile < num_tiles; tile += tile_step) {
            for (int kb = kb_begin; kb < kb_end; ++kb) {
                if (turn == static_cast<uint32_t>(team)) {
                    ok = guard.wait(&load_full[slot.idx], slot.phase, kSiteLoadFull, 2) &&
                         guard.wait(&operand_empty[operand.idx], operand.phase ^ 1u, kSiteOperandEmpty);
                    if (!ok) break;
                    const uint8_t* const raw = smem + L::kRawOff + slot.idx * L::kRawBytes;
                    uint8_t* const dst = smem + L::kOperandOff + operand.idx * L::kOperandBytes;
                    uint4 cells[kUnitsPerThread];
#pragma unroll
                    for (int i = 0; i < kUnitsPerThread; ++i) {
                        if (t + i * kTeamThreads < units) cells[i] = *reinterpret_cast<const uint4*>(raw + (t + i * kTeamThreads) * 16);
                    }
#pragma unroll
                    for (int i = 0; i < kUnitsPerThread; ++i) {
                        if (t + i * kTeamThreads >= units) continue;
                        const uint32_t w[4] = {cells[i].x, cells[i].y, cells[i].z, cells[i].w};
                        uint32_t h[8];
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            fp8x4_to_f16x4<kE5M2>(w[q], h[2 * q], h[2 * q + 1]);
                            if constexpr (kOperandBf16) {
                                h[2 * q] = f16x2_to_bf16x2(h[2 * q]);
                                h[2 * q + 1] = f16x2_to_bf16x2(h[2 * q + 1]);
                            }
                        }
                        *reinterpret_cast<uint4*>(dst + dst_offset[i]) = make_uint4(h[0], h[1], h[2], h[3]);
                        *reinterpret_cast<uint4*>(dst + (dst_offset[i] ^ 16u)) = make_uint4(h[4], h[5], h[6], h[7]);
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&operand_full[operand.idx]), pair_base));
                }
                turn = turn + 1 == kPairTeams ? 0 : turn + 1;
                slot.advance(kPairLoadStages);
                operand.advance(kPairOperandStages);
            }
        }
    }

    if constexpr (kSplitK) {
      if (p.cluster_reduce) {
        // The cluster holds every CTA of the tile (pair s = split s). Each CTA sends the 32-column chunks it does not add itself
        // (chunk c belongs to split c % splits) from tensor memory straight into the owner's shared memory, which the main loop
        // no longer needs, and then adds what it received to its own chunks in split order: no scratch, no tickets, and the
        // partials never pass through the L2. Receive buffer of a CTA: [source split][owned chunk c / splits][4-column group]
        // [row][4] fp32, so that the 32 lanes of a warp (32 rows) write and read 512 consecutive bytes per instruction.
        constexpr int kGroups = (kThreads - kFirstEpilogueWarp * 32) / kBlockM;   // 128 threads (one per row) each
        constexpr int kChunkBytes = 8 * kBlockM * 16;                              // one chunk of 128 rows x 32 columns
        const int max_owned = (kPairN / 32 + p.splits - 1) / p.splits;
        const int t = static_cast<int>(threadIdx.x) - kFirstEpilogueWarp * 32;
        const int group = t / kBlockM;
        // a warp reads the tensor-memory lanes 32 * (warp % 4) .. + 31, so its threads take those rows of the tile
        const int r = (warp % 4) * 32 + lane;
        const uint32_t own_taddr = tmem_base + (static_cast<uint32_t>((warp % 4) * 32) << 16);   // one item per pair: accumulator buffer 0
        __syncthreads();
        cluster_sync_all();   // every CTA of the tile has left its role loops: its operand rings are free
        if (t >= 0) {
            tc_fence_after_sync();
            int sent = 0;
            for (int c = 0; c < kPairN / 32; ++c) {
                const int owner = c % p.splits;
                if (owner == my_split) continue;
                if (sent++ % kGroups != group) continue;
                uint32_t v[32];
                tmem_ld_32x32(own_taddr + c * 32, v);
                tmem_wait_ld();
                const uint32_t local = smem_u32(smem + (my_split * max_owned + c / p.splits) * kChunkBytes + r * 16);
                const uint32_t remote = map_to_cta(local, static_cast<uint32_t>(2 * owner) + cta);
#pragma unroll
                for (int g = 0; g < 8; ++g) st_shared_cluster_v4(remote + g * (kBlockM * 16), v[4 * g], v[4 * g + 1], v[4 * g + 2], v[4 * g + 3]);
            }
        }
        cluster_sync_all();   // release / acquire over the cluster: every partial has landed
        if (t >= 0 && !guard.aborted()) {
            const int tile = first_tile;
            int tile_m, tile_n;
            banded_tile(tile, tiles_m, tiles_n, p.band, tile_m, tile_n);
            const int row = tile_m * 2 * kBlockM + static_cast<int>(cta) * kBlockM + r;
            const int n0 = tile_n * kPairN;
            const float scale = p.scale != nullptr ? __ldg(p.scale) : 1.0f;
            uint16_t* const c_row = p.c + static_cast<int64_t>(row) * p.N;
            int owned = 0;
            for (int c = my_split; c < kPairN / 32; c += p.splits, ++owned) {
                if (owned % kGroups != group) continue;
                float sum[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) sum[i] = 0.0f;
                for (int sp = 0; sp < p.splits; ++sp) {   // split order: the sum does not depend on who adds it
                    if (sp == my_split) {
                        uint32_t own[32];
                        tmem_ld_32x32(own_taddr + c * 32, own);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; ++i) sum[i] += __uint_as_float(own[i]);
                        continue;
                    }
                    const uint8_t* const src = smem + (sp * max_owned + owned) * kChunkBytes + r * 16;
#pragma unroll
                    for (int g = 0; g < 8; ++g) {
                        const float4 x = *reinterpret_cast<const float4*>(src + g * (kBlockM * 16));
                        sum[4 * g] += x.x;
                        sum[4 * g + 1] += x.y;
                        sum[4 * g + 2] += x.z;
                        sum[4 * g + 3] += x.w;
                    }
                }
                uint32_t v[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(sum[i]);
                finish_columns<kOutBf16>(p, v, scale, row, n0 + c * 32, c_row);
            }
        }
      } else {
        // Every role loop has ended. Wait until all splits of this CTA's half of the tile are in (bounded), then add the
        // partials of this CTA's share of the chunks: chunk c belongs to split c % splits. Twenty warps, one row per thread.
        __syncthreads();
        const int tile = first_tile;
        if (threadIdx.x == 0 && !guard.aborted()) {
            const uint32_t* const in_counter = p.counters + tile * 2 + static_cast<int>(cta);
            const long long start = clock64();
            while (true) {
                uint32_t seen;
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(in_counter) : "memory");
                if (seen >= static_cast<uint32_t>(p.splits)) break;
                if (clock64() - start > kWaitLimitCycles) {
                    guard.give_up(kSiteStore, 7);
                    break;
                }
                __nanosleep(64);
            }
            __threadfence();
        }
        __syncthreads();
        if (!guard.aborted() && threadIdx.x >= kFirstEpilogueWarp * 32) {
            constexpr int kGroups = (kThreads - kFirstEpilogueWarp * 32) / kBlockM;   // 128 threads (one per row) each
            const int t = static_cast<int>(threadIdx.x) - kFirstEpilogueWarp * 32;
            const int group = t / kBlockM;
            // a warp reads the tensor-memory lanes 32 * (warp % 4) .. + 31, so its threads take those rows of the tile
            const int r = (warp % 4) * 32 + lane;
            const uint32_t own_taddr = tmem_base + (static_cast<uint32_t>((warp % 4) * 32) << 16);   // one item per pair: accumulator buffer 0
            tc_fence_after_sync();
            int tile_m, tile_n;
            banded_tile(tile, tiles_m, tiles_n, p.band, tile_m, tile_n);
            const int row = tile_m * 2 * kBlockM + static_cast<int>(cta) * kBlockM + r;
            const int n0 = tile_n * kPairN;
            const float scale = p.scale != nullptr ? __ldg(p.scale) : 1.0f;
            uint16_t* const c_row = p.c + static_cast<int64_t>(row) * p.N;
            const float* const half_base = p.partials + (static_cast<int64_t>(tile) * 2 + cta) * p.splits * (kBlockM * kPairN) + r * 4;
            int owned = 0;
            for (int c = my_split; c < kPairN / 32; c += p.splits, ++owned) {
                if (group >= kGroups || owned % kGroups != group) continue;
                float sum[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) sum[i] = 0.0f;
                for (int sp = 0; sp < p.splits; ++sp) {   // split order: the sum does not depend on who adds it
                    if (sp == my_split) {
                        // this CTA's own partial of the chunk never left tensor memory
                        uint32_t own[32];
                        tmem_ld_32x32(own_taddr + c * 32, own);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; ++i) sum[i] += __uint_as_float(own[i]);
                        continue;
                    }
                    const float* const src = half_base + static_cast<int64_t>(sp) * (kBlockM * kPairN);
#pragma unroll
                    for (int g = 0; g < 8; ++g) {
                        const float4 x = __ldcg(reinterpret_cast<const float4*>(src + (c * 8 + g) * (kBlockM * 4)));
                        sum[4 * g] += x.x;
                        sum[4 * g + 1] += x.y;
                        sum[4 * g + 2] += x.z;
                        sum[4 * g + 3] += x.w;
                    }
                }
                uint32_t v[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(sum[i]);
                finish_columns<kOutBf16>(p, v, scale, row, n0 + c * 32, c_row);
            }
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            // this CTA has read every partial it needs: the last of the tile's 2 x splits CTAs resets the tickets
            __threadfence();
            uint32_t* const done = p.counters + 2 * num_tiles + tile;
            if (atomicAdd(done, 1u) == static_cast<uint32_t>(2 * p.splits - 1)) {
                p.counters[tile * 2] = 0u;
                p.counters[tile * 2 + 1] = 0u;
                *done = 0u;
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
    }
    cluster_sync_all();  // neither CTA frees tensor memory while the pair's UMMAs may still write to it
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, 2 * kPairN);
    }
}

// ---------------------------------------------------------------------------------------------------------
// Skinny-M version (M <= 128, HBM bound on the weight): one CTA per (64-column tile, K split), two CTAs
// resident per SM, so that a few hundred CTAs stream the weight concurrently. With `splits` > 1 every CTA
// writes its fp32 partial tile to a scratch buffer [splits][M][N], takes a ticket from a per-tile counter,
// and the CTA that draws the last ticket sums the partials in split order (deterministic), applies the
// epilogue, writes C and puts the counter back to zero. With `splits` == 1 nothing is staged.
// ---------------------------------------------------------------------------------------------------------
constexpr int kSkinnyN = 64;
constexpr int kSkinnyUpcastWarps = 8;   // 256 cells per k block, one per thread
constexpr int kSkinnyThreads = 32 * (kFirstUpcastWarp + kSkinnyUpcastWarps);
constexpr int kSkinnyRawBytes = kSlabsPerBlock * kSkinnyN * 16;   // 4 KB of fp8 cells per k block
constexpr int kSkinnyOperandBytes = kSkinnyN * 128;               // 8 KB converted operand
constexpr int kSkinnyMaxStages = 12;
constexpr int kSkinnyTeams = 2;
constexpr int kSkinnyOperandStages = 6;   // per k block there is almost no work: the barrier hand-offs have to overlap
constexpr int kSkinnySmemBudget = 100 * 1024;                     // two CTAs per SM

struct SkinnyParams {
    Params base;
    float* partials;      // [splits][M][N] fp32, only touched when splits > 1
    uint32_t* counters;   // [tiles_n], zero before the launch and zero again after it
    int splits;
    int kb_per_split;
    uint32_t a_slot_bytes;  // bytes of one activation box and slot: only ceil(M / 8) * 8 rows are fetched and kept
    uint32_t load_stages;   // depth of the load ring: as many slots as fit beside a second CTA on the SM
};

template <bool kE5M2, bool kOperandBf16, bool kOutBf16>
__global__ void __launch_bounds__(kSkinnyThreads, 2)
scaled_mm_skinny_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const SkinnyParams sp) {
    constexpr int BN = kSkinnyN;
    const Params& p = sp.base;
    extern __shared__ uint8_t smem_dyn[];
    uint8_t* const smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~static_cast<uintptr_t>(1023));
    // [activation slots, packed at a_slot_bytes][operand slots][raw weight slots][barriers]. An activation slot only
    // holds the rows that exist; the UMMA reads 128 rows from its start, i.e. on into the following slots and
    // buffers (at least 16 KB follow the last slot), and what it finds there only reaches accumulator rows >= M.
    const uint32_t stages = sp.load_stages;
    uint8_t* const a_smem = smem;
    uint8_t* const operand_smem = a_smem + stages * sp.a_slot_bytes;
    uint8_t* const raw_smem = operand_smem + kSkinnyOperandStages * kSkinnyOperandBytes;
    uint64_t* const bars = reinterpret_cast<uint64_t*>(raw_smem + stages * kSkinnyRawBytes);
    uint64_t* const load_full = bars;
    uint64_t* const load_empty = load_full + stages;
    uint64_t* const operand_full = load_empty + stages;
    uint64_t* const operand_empty = operand_full + kSkinnyOperandStages;
    uint64_t* const tmem_full = operand_empty + kSkinnyOperandStages;
    uint32_t* const tmem_slot = reinterpret_cast<uint32_t*>(tmem_full + 1);
    volatile uint32_t* const abort_flag = tmem_slot + 1;
    volatile uint32_t* const last_flag = tmem_slot + 2;

    const int warp = static_cast<int>(threadIdx.x) / 32;
    const int lane = static_cast<int>(threadIdx.x) % 32;
    const WaitGuard guard{abort_flag, g_status};

    if (threadIdx.x == 0) {
        *abort_flag = 0u;
        *last_flag = 0u;
        for (uint32_t s = 0; s < stages; ++s) {
            mbar_init(&load_full[s], 1);
            mbar_init(&load_empty[s], 1);
        }
        for (int s = 0; s < kSkinnyOperandStages; ++s) {
            mbar_init(&operand_full[s], kSkinnyUpcastWarps / kSkinnyTeams);
            mbar_init(&operand_empty[s], 1);
        }
        mbar_init(&tmem_full[0], 1);
        mbar_init_fence();
        tma_prefetch_desc(&map_a);
        tma_prefetch_desc(&map_b);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, BN);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    const int tile = static_cast<int>(blockIdx.x) / sp.splits;   // splits of one tile are neighbours in the grid
    const int split = static_cast<int>(blockIdx.x) % sp.splits;
    const int n0 = tile * BN;
    const int num_kb = (p.K + kBlockK - 1) / kBlockK;
    const int kb_begin = split * sp.kb_per_split;
    const int kb_end = kb_begin + sp.kb_per_split < num_kb ? kb_begin + sp.kb_per_split : num_kb;

    if (warp == 0) {
        if (elect_one()) {
            Ring slot;
            for (int kb = kb_begin; kb < kb_end; ++kb) {
                if (!guard.wait(&load_empty[slot.idx], slot.phase ^ 1u, kSiteLoadEmpty)) break;
                // The activation box only covers the rows that exist (rounded up to 8): rows of a 128-row box that lie
                // past M are zero filled but still cross the L2 -> SM fabric. The UMMA reads 128 rows of the slot all
                // the same; what the missing rows hold only reaches accumulator rows that are never stored.
                mbar_arrive_expect_tx(&load_full[slot.idx], sp.a_slot_bytes + kSkinnyRawBytes);
                tma_load_2d(a_smem + slot.idx * sp.a_slot_bytes, &map_a, &load_full[slot.idx], kb * kBlockK, 0);
                tma_load_2d(raw_smem + slot.idx * kSkinnyRawBytes, &map_b, &load_full[slot.idx], n0 * 2, kb * kSlabsPerBlock);
                slot.advance(stages);
            }
        }
    } else if (warp == 1) {
        if (elect_one()) {
            Ring slot, operand;
            bool ok = true;
            for (int kb = kb_begin; kb < kb_end; ++kb) {
                ok = guard.wait(&load_full[slot.idx], slot.phase, kSiteLoadFull, 1) &&
                     guard.wait(&operand_full[operand.idx], operand.phase, kSiteOperandFull);
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t a_addr = smem_u32(a_smem + slot.idx * sp.a_slot_bytes);
                const uint32_t b_addr = smem_u32(operand_smem + operand.idx * kSkinnyOperandBytes);
#pragma unroll
                for (int k = 0; k < kBlockK / 16; ++k) {
                    umma_f16(tmem_base, make_desc_sw128_kmajor(a_addr + k * 32), make_desc_sw128_kmajor(b_addr + k * 32), p.idesc,
                             (kb > kb_begin || k > 0) ? 1u : 0u);
                }
                umma_commit(&load_empty[slot.idx]);
                umma_commit(&operand_empty[operand.idx]);
                slot.advance(stages);
                operand.advance(kSkinnyOperandStages);
            }
            if (ok) umma_commit(&tmem_full[0]);
        }
    } else if (warp < kFirstUpcastWarp) {
        // ------------------------------------------------------------------ epilogue (+ split reduction)
        const int quarter = warp % 4;
        const int row = quarter * 32 + lane;
        const bool row_live = row < p.M;
        const float scale = p.scale != nullptr ? __ldg(p.scale) : 1.0f;
        const bool ok = guard.wait(&tmem_full[0], 0u, kSiteTmemFull);
        tc_fence_after_sync();
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
        uint16_t* const c_row = p.c + static_cast<int64_t>(row) * p.N;

        // scale, round, bias, round, store: 32 consecutive columns of this thread's row
        auto finish = [&](const float (&acc)[32], int col0) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                const int col = col0 + g * 8;
                if (col >= p.N) continue;
                uint32_t o[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) o[i] = pack_out<kOutBf16>(acc[g * 8 + 2 * i] * scale, acc[g * 8 + 2 * i + 1] * scale);
                if (p.bias != nullptr) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint32_t bw = static_cast<uint32_t>(__ldg(p.bias + col + 2 * i)) | (static_cast<uint32_t>(__ldg(p.bias + col + 2 * i + 1)) << 16);
                        const float2 x = unpack_out<kOutBf16>(o[i]);
                        const float2 b = unpack_out<kOutBf16>(bw);
                        o[i] = pack_out<kOutBf16>(x.x + b.x, x.y + b.y);
                    }
                }
                *reinterpret_cast<uint4*>(c_row + col) = make_uint4(o[0], o[1], o[2], o[3]);
            }
        };

        if (ok) {
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t v[32];
                tmem_ld_32x32(taddr + c * 32, v);
                tmem_wait_ld();
                float acc[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) acc[i] = __uint_as_float(v[i]);
                if (!row_live) continue;
                if (sp.splits == 1) {
                    finish(acc, n0 + c * 32);
                } else {
                    float* const dst = sp.partials + (static_cast<int64_t>(split) * p.M + row) * p.N + n0 + c * 32;
#pragma unroll
                    for (int g = 0; g < 8; ++g) {
                        if (n0 + c * 32 + g * 4 < p.N) *reinterpret_cast<float4*>(dst + g * 4) = make_float4(acc[g * 4], acc[g * 4 + 1], acc[g * 4 + 2], acc[g * 4 + 3]);
                    }
                }
            }
        }
        if (sp.splits > 1) {
            __threadfence();
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (warp == kFirstEpilogueWarp && lane == 0) {
                const uint32_t ticket = atomicAdd(sp.counters + tile, 1u);
                *last_flag = (ticket == static_cast<uint32_t>(sp.splits - 1)) ? 1u : 0u;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (*last_flag != 0u) {
                __threadfence();
                if (row_live) {
#pragma unroll 1
                    for (int c = 0; c < BN / 32; ++c) {
                        float acc[32];
#pragma unroll
                        for (int i = 0; i < 32; ++i) acc[i] = 0.0f;
                        for (int s = 0; s < sp.splits; ++s) {  // fixed order: the sum does not depend on which CTA finishes last
                            const float* const src = sp.partials + (static_cast<int64_t>(s) * p.M + row) * p.N + n0 + c * 32;
#pragma unroll
                            for (int g = 0; g < 8; ++g) {
                                if (n0 + c * 32 + g * 4 < p.N) {
                                    const float4 t4 = __ldcg(reinterpret_cast<const float4*>(src + g * 4));
                                    acc[g * 4] += t4.x;
                                    acc[g * 4 + 1] += t4.y;
                                    acc[g * 4 + 2] += t4.z;
                                    acc[g * 4 + 3] += t4.w;
                                }
                            }
                        }
                        finish(acc, n0 + c * 32);
                    }
                }
                if (warp == kFirstEpilogueWarp && lane == 0) sp.counters[tile] = 0u;  // ready for the next launch
            }
        }
    } else {
        // ------------------------------------------------------------------ upcast warps
        // Two teams of four warps take the k blocks in turn (a k block is 256 cells, two per thread of a team):
        // there is almost no work per k block, so what has to overlap is the chain of barrier hand-offs. Both
        // ring depths are even, so a team always meets the same slots and sees every phase of their barriers.
        constexpr int kTeams = kSkinnyTeams;
        constexpr int kTeamThreads = kSkinnyUpcastWarps * 32 / kTeams;
        constexpr int kUnits = BN * kSlabsPerBlock;
        constexpr int kUnitsPerThread = kUnits / kTeamThreads;
        const int upcast_thread = static_cast<int>(threadIdx.x) - kFirstUpcastWarp * 32;
        const int team = upcast_thread / kTeamThreads;
        const int t = upcast_thread % kTeamThreads;
        Ring slot, operand;
        for (int kb = kb_begin; kb < kb_end; ++kb) {
            if (((kb - kb_begin) % kTeams) == team) {
                if (!(guard.wait(&load_full[slot.idx], slot.phase, kSiteLoadFull, 2) &&
                      guard.wait(&operand_empty[operand.idx], operand.phase ^ 1u, kSiteOperandEmpty))) {
                    break;
                }
                const uint8_t* const raw = raw_smem + slot.idx * kSkinnyRawBytes;
                uint8_t* const dst = operand_smem + operand.idx * kSkinnyOperandBytes;
                uint4 cells[kUnitsPerThread];
#pragma unroll
                for (int i = 0; i < kUnitsPerThread; ++i) cells[i] = *reinterpret_cast<const uint4*>(raw + (t + i * kTeamThreads) * 16);
#pragma unroll
                for (int i = 0; i < kUnitsPerThread; ++i) {
                    const int u = t + i * kTeamThreads;
                    const int row = u % BN;
                    const int slab = u / BN;
                    const uint32_t w[4] = {cells[i].x, cells[i].y, cells[i].z, cells[i].w};
                    uint32_t h[8];
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        fp8x4_to_f16x4<kE5M2>(w[q], h[2 * q], h[2 * q + 1]);
                        if constexpr (kOperandBf16) {
                            h[2 * q] = f16x2_to_bf16x2(h[2 * q]);
                            h[2 * q + 1] = f16x2_to_bf16x2(h[2 * q + 1]);
                        }
                    }
                    *reinterpret_cast<uint4*>(dst + sw128_offset(row, 2 * slab)) = make_uint4(h[0], h[1], h[2], h[3]);
                    *reinterpret_cast<uint4*>(dst + sw128_offset(row, 2 * slab + 1)) = make_uint4(h[4], h[5], h[6], h[7]);
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(&operand_full[operand.idx]);
            }
            slot.advance(stages);
            operand.advance(kSkinnyOperandStages);
        }
    }

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
        tmem_dealloc(tmem_base, BN);
    }
}

// SMs that the persistent scaled_mm kernels leave free (feather_scaled_mm_set_sm_margin): a collective that runs beside
// the product needs SMs of its own, because a persistent CTA holds its SM's shared memory until the kernel ends.
std::atomic<int> g_sm_margin{0};

struct LaunchArgs {
    const uint16_t* a;
    const uint8_t* b;
    const float* scale;
    const uint16_t* bias;
    uint16_t* c;
    int64_t M, N, K;
    bool e5m2, a_bf16, out_bf16;
    cudaStream_t stream;
    // K split of the one-CTA kernel (1 = none): fp32 scratch [splits][M][N] and one zeroed ticket per tile
    int splits = 1;
    float* partials = nullptr;
    uint32_t* counters = nullptr;
};

inline int effective_splits(int64_t K, int splits);

template <int BN, bool kE5M2, bool kOperandBf16, bool kOutBf16>
bool launch_instance(const LaunchArgs& args) {
    using L = Smem<BN>;
    const bool split = args.splits > 1 && args.partials != nullptr && args.counters != nullptr && effective_splits(args.K, args.splits) > 1;
    auto* kernel = split ? &scaled_mm_kernel<BN, kE5M2, kOperandBf16, kOutBf16, true> : &scaled_mm_kernel<BN, kE5M2, kOperandBf16, kOutBf16, false>;
    static PerDeviceState configured[2];
    if (configured[split ? 1 : 0].get([&] { return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic) == cudaSuccess ? 1 : 0; }) == 0) {
        return false;
    }

    CUtensorMap map_a, map_b;
    {
        const uint64_t dims[2] = {static_cast<uint64_t>(args.K), static_cast<uint64_t>(args.M)};
        const uint64_t strides[1] = {static_cast<uint64_t>(args.K) * 2};
        const uint32_t box[2] = {kBlockK, kBlockM};
        if (!encode_map(&map_a, args.a_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, args.a, dims, strides, box,
                        CU_TENSOR_MAP_SWIZZLE_128B)) {
            return false;
        }
    }
    {
        // One slab row of the prepack is N contiguous 16-byte cells. Described as 8-byte elements so that a
        // box row is up to 2048 contiguous bytes (128 cells) instead of one 16-byte cell per box row.
        const uint64_t k16_rows = static_cast<uint64_t>((args.K + 127) / 128) * 8;  // the prepack pads K to 128
        const uint64_t dims[2] = {static_cast<uint64_t>(args.N) * 2, k16_rows};
        const uint64_t strides[1] = {static_cast<uint64_t>(args.N) * 16};
        const uint32_t box[2] = {static_cast<uint32_t>(L::kBoxCells * 2), kSlabsPerBlock};
        if (!encode_map(&map_b, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, args.b, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE)) return false;
    }

    Params p{};
    p.scale = args.scale;
    p.bias = args.bias;
    p.c = args.c;
    p.M = static_cast<int>(args.M);
    p.N = static_cast<int>(args.N);
    p.K = static_cast<int>(args.K);
    p.tiles_m = static_cast<int>((args.M + kBlockM - 1) / kBlockM);
    p.tiles_n = static_cast<int>((args.N + BN - 1) / BN);
    p.idesc = make_idesc(kAccF32, args.a_bf16 ? kFmtBF16 : kFmtF16, kOperandBf16 ? kFmtBF16 : kFmtF16, kBlockM, BN);
    p.bias_vec = (reinterpret_cast<uintptr_t>(args.bias) & 0xfu) == 0u ? 1 : 0;

    p.splits = 1;
    if (split) {
        const int num_kb = static_cast<int>((args.K + kBlockK - 1) / kBlockK);
        p.splits = effective_splits(args.K, args.splits);
        p.kb_per_split = (num_kb + p.splits - 1) / p.splits;
        p.partials = args.partials;
        p.counters = args.counters;
    }
    const int64_t num_items = static_cast<int64_t>(p.tiles_m) * p.tiles_n * p.splits;
    if (num_items > (1 << 30)) return false;
    const int margin = g_sm_margin.load(std::memory_order_relaxed);
    const int sms = device_info().sm_count - margin > 0 ? device_info().sm_count - margin : 1;
    const int grid = num_items < sms ? static_cast<int>(num_items) : sms;
    p.single_item = (split && num_items <= sms) ? 1 : 0;
    kernel<<<grid, kThreads, L::kDynamic, args.stream>>>(map_a, map_b, p);
    return cudaGetLastError() == cudaSuccess;
}

// FEATHER_SCALED_MM_PAIR=0 keeps the one-CTA kernel for every shape (A/B measurements).
// Row tiles per band of the pair kernels' tile walk: as many as keep one band of activations around 32 MB.
inline int tile_band(int64_t bytes_per_row_tile, int tiles_m) {
    int64_t band = (32ll << 20) / (bytes_per_row_tile > 0 ? bytes_per_row_tile : 1);
    if (band < 4) band = 4;
    if (band > tiles_m) band = tiles_m;
    return static_cast<int>(band < 1 ? 1 : band);
}

inline bool pair_kernel_enabled() {
    static const bool enabled = [] {
        const char* v = getenv("FEATHER_SCALED_MM_PAIR");
        return v == nullptr || v[0] != '0';
    }();
    return enabled;
}

// FEATHER_SKINNY_WMMA_OFF=1 keeps few-row problems on the tcgen05 kernel with 64-wide tiles (A/B measurements).
// Read once per process.
inline bool skinny_wmma_off() {
    static const bool off = env_switch("FEATHER_SKINNY_WMMA_OFF");
    return off;
}

// Pair tiles (256 x 256) of a problem, and whether a K split of the pair kernel fits: every (tile, split) item needs a pair
// of its own, all resident at once, because the CTAs of a tile wait for one another's partials.
inline int64_t pair_tiles(int64_t M, int64_t N) { return ((M + 2 * kBlockM - 1) / (2 * kBlockM)) * ((N + kPairN - 1) / kPairN); }
constexpr int kPairMaxSplits = kPairN / 32;   // a split owns at least one 32-column chunk of the reduction

// FEATHER_SCALED_MM_CLUSTER_REDUCE_OFF=1 keeps the K split of the pair kernel on scratch and tickets (A/B measurements). Read once per process.
inline bool cluster_reduce_off() {
    static const bool off = env_switch("FEATHER_SCALED_MM_CLUSTER_REDUCE_OFF");
    return off;
}

// The pair kernel takes its cluster size from the launch: 2 (one CTA pair), or all the pairs of a tile when they reduce a K
// split among themselves. `cluster_reduce` is stored in the parameters the kernel sees. False if the launch is refused (a
// cluster of that size does not fit the device), with the error cleared.
template <typename Kernel>
bool launch_clustered(Kernel* kernel, int cluster_ctas, unsigned grid, bool cluster_reduce, cudaStream_t stream, const CUtensorMap& map_a, const CUtensorMap& map_b,
                      const CUtensorMap& map_c, Params p, int margin_sms = 0) {
    p.cluster_reduce = cluster_reduce ? 1 : 0;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(grid);
    config.blockDim = dim3(kThreads);
    config.dynamicSmemBytes = PairSmem::kDynamic;
    config.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = static_cast<unsigned>(cluster_ctas);
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    config.attrs = attr;
    config.numAttrs = 1;
    if (cluster_ctas > 2) {
        // Every cluster of the launch has to be resident at once, or a second wave of clusters waits for the first (a cluster
        // needs up to eight free SMs of ONE GPC with 214 KB of shared memory each, so fewer fit than SMs / size): asked once per
        // device, kernel and cluster size.
        static PerDeviceState fits[9];
        const int resident = fits[cluster_ctas].get([&] {   // clusters that fit + 1
            int clusters = 0;
            if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &config) != cudaSuccess || clusters < 0) {
                (void)cudaGetLastError();
                clusters = 0;
            }
            return clusters + 1;
        }) - 1;
        const int needed = static_cast<int>(grid) / cluster_ctas;
        if (needed > resident - (margin_sms + cluster_ctas - 1) / cluster_ctas) return false;
    }
    if (cudaLaunchKernelEx(&config, kernel, map_a, map_b, map_c, p) != cudaSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    return true;
}

// FEATHER_SCALED_MM_BULK_OUT_OFF=1 keeps the pair kernel's direct output stores (A/B measurements). Read once per process.
inline bool bulk_out_off() {
    static const bool off = env_switch("FEATHER_SCALED_MM_BULK_OUT_OFF");
    return off;
}

// FEATHER_SCALED_MM_TILE_WIDTH_OFF=1 keeps 256-column tiles for every shape, FEATHER_SCALED_MM_TILE_WIDTH=<multiple of 32 in 128..256>
// forces a width (A/B measurements). Read once per process.
inline int forced_tile_width() {
    static const int forced = [] {
        if (env_switch("FEATHER_SCALED_MM_TILE_WIDTH_OFF")) return kPairN;
        const char* text = std::getenv("FEATHER_SCALED_MM_TILE_WIDTH");
        const int value = text != nullptr ? std::atoi(text) : 0;
        return value >= kPairN / 2 && value <= kPairN && value % 32 == 0 ? value : 0;
    }();
    return forced;
}

// Output columns per tile of the pair kernel without a K split. A tile fetches its 256 activation rows whatever its width, so its time is
// modelled as a part that goes with the width and an equal part that does not; a narrower tile pays when it fills the last round of the
// persistent grid (1024 x 12288: 192 tiles of 256 columns are 2.6 rounds of 74 pairs and take three, 220 tiles of 224 columns are 2.97).
// The widest tile wins a tie.
inline int pair_tile_width(int64_t M, int64_t N, int pairs) {
    const int forced = forced_tile_width();
    if (forced != 0) return forced;
    if (pairs <= 0) return kPairN;
    const int64_t tiles_m = (M + 2 * kBlockM - 1) / (2 * kBlockM);
    int best = kPairN;
    int64_t best_cost = 0;
    int64_t full_cost = 0;
    for (int width = kPairN; width >= kPairN / 2; width -= 32) {
        const int64_t tiles = tiles_m * ((N + width - 1) / width);
        const int64_t cost = ((tiles + pairs - 1) / pairs) * (width + kPairN + 48);
        if (width == kPairN) full_cost = cost;
        if (width == kPairN || cost < best_cost) {
            best = width;
            best_cost = cost;
        }
    }
    // a narrower tile must promise at least 4 %: below that the model's error decides
    return best_cost * 100 <= full_cost * 96 ? best : kPairN;
}

template <bool kE5M2, bool kOperandBf16, bool kOutBf16, bool kSplitK = false>
bool launch_pair_instance(const LaunchArgs& args) {
    using L = PairSmem;
    auto* kernel = &scaled_mm_pair_kernel<kE5M2, kOperandBf16, kOutBf16, kSplitK>;
    // Set-up once per device: the shared-memory limit, and how many CTA pairs can be resident at once. A persistent
    // grid must not exceed that: pairs need both SMs of a TPC, and parts with an odd number of enabled SMs in some
    // TPCs hold fewer pairs than sm_count / 2.
    static PerDeviceState resident_pairs;
    const int pairs = resident_pairs.get([&] {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic) != cudaSuccess) return 0;
        cudaLaunchConfig_t config = {};
        config.gridDim = dim3(static_cast<unsigned>(device_info().sm_count / 2 * 2));
        config.blockDim = dim3(kThreads);
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
    const int margin_pairs = (g_sm_margin.load(std::memory_order_relaxed) + 1) / 2;
    const int usable = pairs - margin_pairs > 0 ? pairs - margin_pairs : 1;
    const int tile_n = kSplitK ? kPairN : pair_tile_width(args.M, args.N, usable);
    CUtensorMap map_a, map_b;
    {
        const uint64_t dims[2] = {static_cast<uint64_t>(args.K), static_cast<uint64_t>(args.M)};
        const uint64_t strides[1] = {static_cast<uint64_t>(args.K) * 2};
        const uint32_t box[2] = {kBlockK, kBlockM};
        if (!encode_map(&map_a, args.a_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, args.a, dims, strides, box,
                        CU_TENSOR_MAP_SWIZZLE_128B)) {
            return false;
        }
    }
    {
        const uint64_t k16_rows = static_cast<uint64_t>((args.K + 127) / 128) * 8;
        const uint64_t dims[2] = {static_cast<uint64_t>(args.N) * 2, k16_rows};
        const uint64_t strides[1] = {static_cast<uint64_t>(args.N) * 16};
        const uint32_t box[2] = {static_cast<uint32_t>(tile_n), kSlabsPerBlock};   // a CTA's half of the tile's columns, two 8-byte words each
        if (!encode_map(&map_b, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, args.b, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE)) return false;
    }
    Params p{};
    p.scale = args.scale;
    p.bias = args.bias;
    p.c = args.c;
    p.M = static_cast<int>(args.M);
    p.N = static_cast<int>(args.N);
    p.K = static_cast<int>(args.K);
    p.tiles_m = static_cast<int>((args.M + 2 * kBlockM - 1) / (2 * kBlockM));
    p.band = tile_band(2 * kBlockM * args.K * 2, p.tiles_m);
    p.tile_n = tile_n;
    p.tiles_n = static_cast<int>((args.N + tile_n - 1) / tile_n);
    p.idesc = make_idesc(kAccF32, args.a_bf16 ? kFmtBF16 : kFmtF16, kOperandBf16 ? kFmtBF16 : kFmtF16, 2 * kBlockM, static_cast<uint32_t>(tile_n));
    p.bias_vec = (reinterpret_cast<uintptr_t>(args.bias) & 0xfu) == 0u ? 1 : 0;
    // the output as a 2-D tensor with a box of 32 columns x 128 rows (64-byte swizzle): what the epilogue's bulk stores write
    CUtensorMap map_c = map_a;   // unused without bulk_out
    p.bulk_out = (!kSplitK && args.N % 8 == 0 && (reinterpret_cast<uintptr_t>(args.c) & 15u) == 0 && !bulk_out_off()) ? 1 : 0;
    if (p.bulk_out) {
        const uint64_t c_dims[2] = {static_cast<uint64_t>(args.N), static_cast<uint64_t>(args.M)};
        const uint64_t c_strides[1] = {static_cast<uint64_t>(args.N) * 2};
        const uint32_t c_box[2] = {32, 32};   // one epilogue warp's rows of a 32-column chunk
        if (!encode_map(&map_c, kOutBf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, args.c, c_dims, c_strides, c_box, CU_TENSOR_MAP_SWIZZLE_64B)) return false;
    }
    const int num_tiles = p.tiles_m * p.tiles_n;
    if constexpr (kSplitK) {
        const int num_kb = static_cast<int>((args.K + kBlockK - 1) / kBlockK);
        p.splits = effective_splits(args.K, args.splits < kPairMaxSplits ? args.splits : kPairMaxSplits);
        p.kb_per_split = (num_kb + p.splits - 1) / p.splits;
        p.partials = args.partials;
        p.counters = args.counters;
        p.band = p.tiles_m;   // one item per pair: no walk to order
        const int64_t items = static_cast<int64_t>(num_tiles) * p.splits;
        if (p.splits < 2) return false;
        // Up to four splits the tile's pairs form ONE cluster (at most eight CTAs, the portable limit) and exchange their partials
        // through distributed shared memory: no scratch, no tickets, and clusters need not all be resident at once.
        if (p.splits <= 4 && !cluster_reduce_off() && launch_clustered(kernel, 2 * p.splits, static_cast<unsigned>(2 * items), true, args.stream, map_a, map_b, map_c, p, 2 * margin_pairs)) {
            return true;
        }
        if (items > usable) return false;   // the caller falls back to the one-CTA split kernel
        return launch_clustered(kernel, 2, static_cast<unsigned>(2 * items), false, args.stream, map_a, map_b, map_c, p);
    }
    const int grid = 2 * (num_tiles < usable ? num_tiles : usable);
    return launch_clustered(kernel, 2, static_cast<unsigned>(grid), false, args.stream, map_a, map_b, map_c, p);
}

// `split`: the K-split variant (one (tile, split) item per pair); false when the items do not fit the resident pairs.
bool launch_pair(const LaunchArgs& args, bool split = false) {
    const bool operand_bf16 = args.a_bf16;
#define FEATHER_SMM_PAIR_CASE(E5, OB, OUT)                                 \
    if (args.e5m2 == E5 && operand_bf16 == OB && args.out_bf16 == OUT) {    \
        return split ? launch_pair_instance<E5, OB, OUT, true>(args) : launch_pair_instance<E5, OB, OUT, false>(args); \
    }
    FEATHER_SMM_PAIR_CASE(true, false, true)
    FEATHER_SMM_PAIR_CASE(true, false, false)
    FEATHER_SMM_PAIR_CASE(false, false, true)
    FEATHER_SMM_PAIR_CASE(false, false, false)
    FEATHER_SMM_PAIR_CASE(true, true, true)
    FEATHER_SMM_PAIR_CASE(true, true, false)
    FEATHER_SMM_PAIR_CASE(false, true, true)
    FEATHER_SMM_PAIR_CASE(false, true, false)
#undef FEATHER_SMM_PAIR_CASE
    return false;
}

// ---------------------------------------------------------------------------------------------------------
// Vector version for one or two rows (a decode token, a modulation vector): no tensor core. A 128-row UMMA tile would spend
// its floor of 96 clocks per 16-deep slice on one or two live rows, and the tensor-memory/barrier set-up costs as
// much as streaming the weight. Here a warp owns 32 consecutive output columns for one eighth of the contraction:
// per 16-deep slab it loads 32 prepack cells (512 contiguous bytes), decodes them exactly to fp32 and multiplies with
// the activations, which sit in shared memory as fp32 and are read as broadcasts. The eight warps of a CTA cover
// the contraction; their partial sums are added in warp order through shared memory (deterministic), then scale,
// round, bias, round as everywhere else. Products of a 16-bit activation and an fp8 weight are exact in fp32, so
// only the order of the fp32 additions differs from the tensor-core kernels.
// ---------------------------------------------------------------------------------------------------------
constexpr int kGemvMaxRows = 2;
constexpr int kGemvWarps = 8;
constexpr int kGemvUnroll = 8;   // cells in flight per lane
constexpr int kGemvSmemLimit = 64 * 1024;

template <bool kE5M2>
__device__ __forceinline__ void fp8x4_to_f32x4(uint32_t p, float (&f)[4]) {
    uint32_t lo, hi;
    fp8x4_to_f16x4<kE5M2>(p, lo, hi);
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&lo));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&hi));
    f[0] = a.x;
    f[1] = a.y;
    f[2] = b.x;
    f[3] = b.y;
}

template <int kRows, bool kE5M2, bool kActBf16, bool kOutBf16>
__global__ void __launch_bounds__(32 * kGemvWarps) scaled_mm_gemv_kernel(const uint16_t* __restrict__ a, const uint4* __restrict__ cells,
                                                                          const float* __restrict__ scale_ptr, const uint16_t* __restrict__ bias,
                                                                          uint16_t* __restrict__ c, int N, int K, int slabs) {
    extern __shared__ __align__(16) float gemv_smem[];
    float* const act = gemv_smem;                                  // [kRows][slabs * 16], zero past K
    float* const partial = gemv_smem + kRows * slabs * 16;         // [kGemvWarps][kRows][32]
    const int warp = static_cast<int>(threadIdx.x) / 32;
    const int lane = static_cast<int>(threadIdx.x) % 32;
    const int k_pad = slabs * 16;
    for (int i = static_cast<int>(threadIdx.x); i < kRows * k_pad; i += 32 * kGemvWarps) {
        const int r = i / k_pad;
        const int k = i - r * k_pad;
        float v = 0.0f;
        if (k < K) {
            const uint16_t bits = __ldg(a + static_cast<int64_t>(r) * K + k);
            v = kActBf16 ? __uint_as_float(static_cast<uint32_t>(bits) << 16) : __half2float(__ushort_as_half(bits));
        }
        act[i] = v;
    }
    __syncthreads();

    const int n = static_cast<int>(blockIdx.x) * 32 + lane;
    const bool live = n < N;
    const int per_warp = (slabs + kGemvWarps - 1) / kGemvWarps;
    const int s_begin = warp * per_warp;
    const int s_end = s_begin + per_warp < slabs ? s_begin + per_warp : slabs;
    float acc[kRows];
#pragma unroll
    for (int r = 0; r < kRows; ++r) acc[r] = 0.0f;
    const uint4* const column = cells + (live ? n : 0);
    for (int s0 = s_begin; s0 < s_end; s0 += kGemvUnroll) {
        uint4 cell[kGemvUnroll];
#pragma unroll
        for (int u = 0; u < kGemvUnroll; ++u) {
            cell[u] = (live && s0 + u < s_end) ? __ldg(column + static_cast<int64_t>(s0 + u) * N) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int u = 0; u < kGemvUnroll; ++u) {
            if (s0 + u >= s_end) break;
            const uint32_t w[4] = {cell[u].x, cell[u].y, cell[u].z, cell[u].w};
            float f[16];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                float g[4];
                fp8x4_to_f32x4<kE5M2>(w[q], g);
                f[4 * q] = g[0];
                f[4 * q + 1] = g[1];
                f[4 * q + 2] = g[2];
                f[4 * q + 3] = g[3];
            }
#pragma unroll
            for (int r = 0; r < kRows; ++r) {
                const float4* const av = reinterpret_cast<const float4*>(act + r * k_pad + (s0 + u) * 16);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float4 x = av[q];
                    acc[r] = fmaf(f[4 * q], x.x, acc[r]);
                    acc[r] = fmaf(f[4 * q + 1], x.y, acc[r]);
                    acc[r] = fmaf(f[4 * q + 2], x.z, acc[r]);
                    acc[r] = fmaf(f[4 * q + 3], x.w, acc[r]);
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < kRows; ++r) partial[(warp * kRows + r) * 32 + lane] = acc[r];
    __syncthreads();
    if (warp == 0 && live) {
        const float scale = scale_ptr != nullptr ? __ldg(scale_ptr) : 1.0f;
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            float sum = 0.0f;
#pragma unroll
            for (int w = 0; w < kGemvWarps; ++w) sum += partial[(w * kRows + r) * 32 + lane];
            uint32_t o = pack_out<kOutBf16>(sum * scale, 0.0f);
            if (bias != nullptr) {
                const float2 x = unpack_out<kOutBf16>(o);
                const float2 b = unpack_out<kOutBf16>(static_cast<uint32_t>(__ldg(bias + n)));
                o = pack_out<kOutBf16>(x.x + b.x, 0.0f);
            }
            c[static_cast<int64_t>(r) * N + n] = static_cast<uint16_t>(o & 0xffffu);
        }
    }
}

template <int kRows, bool kE5M2, bool kActBf16, bool kOutBf16>
bool launch_gemv_rows(const LaunchArgs& args, int slabs, size_t smem_bytes) {
    auto* kernel = &scaled_mm_gemv_kernel<kRows, kE5M2, kActBf16, kOutBf16>;
    static PerDeviceState configured;
    if (configured.get([&] { return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemvSmemLimit) == cudaSuccess ? 1 : 0; }) == 0) return false;
    const unsigned grid = static_cast<unsigned>((args.N + 31) / 32);
    kernel<<<grid, 32 * kGemvWarps, smem_bytes, args.stream>>>(args.a, reinterpret_cast<const uint4*>(args.b), args.scale, args.bias, args.c,
                                                                 static_cast<int>(args.N), static_cast<int>(args.K), slabs);
    return cudaGetLastError() == cudaSuccess;
}

// True when the vector kernel takes the problem. Measured at 12288 x 3072: one row 11 us against 22 for the skinny
// tensor-core kernel, four rows 25 against 22 (16 fused multiply-adds per weight and row), so it is used for one
// or two rows, when there are at least two CTAs of 32 columns per SM and the activations leave room for several
// CTAs per SM (3072 x 12288 with its 96 CTAs, or a 16384-deep contraction, are slower than the skinny kernel).
inline bool gemv_eligible(const LaunchArgs& args, int* slabs, size_t* smem_bytes) {
    if (args.M > 2) return false;
    *slabs = static_cast<int>((args.K + 15) / 16);
    *smem_bytes = (static_cast<size_t>(args.M) * *slabs * 16 + static_cast<size_t>(kGemvWarps) * args.M * 32) * sizeof(float);
    return *smem_bytes <= 64u * 1024u && args.N >= 64ll * device_info().sm_count && (reinterpret_cast<uintptr_t>(args.b) & 15u) == 0;
}

bool launch_gemv(const LaunchArgs& args, int slabs, size_t smem_bytes) {
#define FEATHER_SMM_GEMV_CASE(E5, AB, OUT)                                                                   \
    if (args.e5m2 == E5 && args.a_bf16 == AB && args.out_bf16 == OUT) {                                       \
        return args.M == 1 ? launch_gemv_rows<1, E5, AB, OUT>(args, slabs, smem_bytes)                        \
                           : launch_gemv_rows<2, E5, AB, OUT>(args, slabs, smem_bytes);                       \
    }
    FEATHER_SMM_GEMV_CASE(true, false, true)
    FEATHER_SMM_GEMV_CASE(true, false, false)
    FEATHER_SMM_GEMV_CASE(false, false, true)
    FEATHER_SMM_GEMV_CASE(false, false, false)
    FEATHER_SMM_GEMV_CASE(true, true, true)
    FEATHER_SMM_GEMV_CASE(true, true, false)
    FEATHER_SMM_GEMV_CASE(false, true, true)
    FEATHER_SMM_GEMV_CASE(false, true, false)
#undef FEATHER_SMM_GEMV_CASE
    return false;
}

// ---------------------------------------------------------------------------------------------------------
// Warp-MMA version for 3..16 rows and wide outputs. tcgen05 has no shape below 64 rows, and its set-up (tensor
// memory, barriers, a CTA per SM) costs more than streaming the weight once, so a problem this skinny is served by
// mma.sync m16n8k16: it is HBM bound, not tensor bound. Same decomposition as the vector kernel (a warp = 32 columns
// x one eighth of the contraction, partial sums added in warp order), and no shuffles or shared-memory staging:
// the contraction index inside a 16-deep slab is permuted the same way for both operands (fragment slots 2j, 2j+1,
// 2j+8, 2j+9 take k = 4j .. 4j+3), so a lane's B fragment is four consecutive bytes of one prepack cell (a warp
// reads eight cells = 128 contiguous bytes per 8-column block) and its A fragment four consecutive activations
// of a row (8 bytes), both straight from global memory.
// ---------------------------------------------------------------------------------------------------------
constexpr int kWmmaMaxRows = 16;   // rows of one CTA; two 16-row tiles per warp were measured too: 33-36 us at 12288 x 3072, slower than the tensor-memory kernel (23)
constexpr int kWmmaWarps = 8;
constexpr int kWmmaUnroll = 4;   // slabs in flight per warp with one 16-row tile (16 weight loads per lane), half as many with two

template <bool kBf16>
__device__ __forceinline__ void mma_m16n8k16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    if constexpr (kBf16) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    } else {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
}

template <int kRowTiles, bool kE5M2, bool kActBf16, bool kOutBf16>
__global__ void __launch_bounds__(32 * kWmmaWarps, kRowTiles == 1 ? 3 : 2) scaled_mm_wmma_kernel(const uint16_t* __restrict__ a, const uint8_t* __restrict__ cells,
                                                                          const float* __restrict__ scale_ptr, const uint16_t* __restrict__ bias,
                                                                          uint16_t* __restrict__ c, int M, int N, int K, int slabs) {
    __shared__ float partial[kWmmaWarps][kRowTiles][4][4][32];   // [warp][16-row tile][8-column block][fragment register][lane]
    const int warp = static_cast<int>(threadIdx.x) / 32;
    const int lane = static_cast<int>(threadIdx.x) % 32;
    const int g = lane >> 2;   // fragment row (and row + 8), B column inside an 8-column block
    const int j = lane & 3;    // which four k of the slab
    const int n0 = static_cast<int>(blockIdx.x) * 32;
    const int row0 = static_cast<int>(blockIdx.y) * 16 * kRowTiles;   // more rows than a warp's tiles: one grid row per block of them
    const int per_warp = (slabs + kWmmaWarps - 1) / kWmmaWarps;
    const int s_begin = warp * per_warp;
    const int s_end = s_begin + per_warp < slabs ? s_begin + per_warp : slabs;

    float acc[kRowTiles][4][4];
#pragma unroll
    for (int t = 0; t < kRowTiles; ++t) {
#pragma unroll
        for (int b = 0; b < 4; ++b) {
#pragma unroll
            for (int r = 0; r < 4; ++r) acc[t][b][r] = 0.0f;
        }
    }
    // rows of this lane's A fragments: 16 t + g and 16 t + g + 8
    bool row_live[kRowTiles][2];
    const uint16_t* a_row[kRowTiles][2];
#pragma unroll
    for (int t = 0; t < kRowTiles; ++t) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = row0 + 16 * t + g + 8 * h;
            row_live[t][h] = row < M;
            a_row[t][h] = a + static_cast<int64_t>(row_live[t][h] ? row : 0) * K + 4 * j;
        }
    }
    // byte address of this lane's four weights in slab 0, block 0; a block is 8 cells = 128 bytes further
    const uint8_t* const w_lane = cells + (static_cast<int64_t>(n0 + g) * 16 + 4 * j);
    const int64_t slab_stride = static_cast<int64_t>(N) * 16;
    bool col_live[4];
#pragma unroll
    for (int b = 0; b < 4; ++b) col_live[b] = n0 + 8 * b + g < N;

    constexpr int kUnroll = kWmmaUnroll / kRowTiles;
    for (int s0 = s_begin; s0 < s_end; s0 += kUnroll) {
        uint32_t w[kUnroll][4];
        uint2 x[kUnroll][kRowTiles][2];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const bool slab_live = s0 + u < s_end;
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                w[u][b] = (slab_live && col_live[b]) ? __ldg(reinterpret_cast<const uint32_t*>(w_lane + (s0 + u) * slab_stride + b * 128)) : 0u;
            }
#pragma unroll
            for (int t = 0; t < kRowTiles; ++t) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    x[u][t][h] = (slab_live && row_live[t][h]) ? __ldg(reinterpret_cast<const uint2*>(a_row[t][h] + (s0 + u) * 16)) : make_uint2(0u, 0u);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                uint32_t b0, b1;
                fp8x4_to_f16x4<kE5M2>(w[u][b], b0, b1);
                if constexpr (kActBf16) {
                    b0 = f16x2_to_bf16x2(b0);
                    b1 = f16x2_to_bf16x2(b1);
                }
#pragma unroll
                for (int t = 0; t < kRowTiles; ++t) {
                    // A fragment: {row g: k 4j, 4j+1}, {row g+8: same}, {row g: k 4j+2, 4j+3}, {row g+8: same}
                    const uint32_t af[4] = {x[u][t][0].x, x[u][t][1].x, x[u][t][0].y, x[u][t][1].y};
                    mma_m16n8k16<kActBf16>(acc[t][b], af, b0, b1);
                }
            }
        }
    }
#pragma unroll
    for (int t = 0; t < kRowTiles; ++t) {
#pragma unroll
        for (int b = 0; b < 4; ++b) {
#pragma unroll
            for (int r = 0; r < 4; ++r) partial[warp][t][b][r][lane] = acc[t][b][r];
        }
    }
    __syncthreads();
    // warp b adds the eight partial sums of block b in warp order and writes the block: accumulator registers 0, 1 are
    // row g, columns 2j and 2j+1 of the block; registers 2, 3 the same columns of row g + 8
    if (warp < 4) {
        const int b = warp;
        const float scale = scale_ptr != nullptr ? __ldg(scale_ptr) : 1.0f;
        const int col = n0 + 8 * b + 2 * j;
        if (col < N) {  // N is a multiple of 16 and col is even: col + 1 exists as well
            uint32_t bias_pair = 0u;
            if (bias != nullptr) bias_pair = static_cast<uint32_t>(__ldg(bias + col)) | (static_cast<uint32_t>(__ldg(bias + col + 1)) << 16);
#pragma unroll
            for (int t = 0; t < kRowTiles; ++t) {
                float sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                for (int w2 = 0; w2 < kWmmaWarps; ++w2) {
#pragma unroll
                    for (int r = 0; r < 4; ++r) sum[r] += partial[w2][t][b][r][lane];
                }
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int row = row0 + 16 * t + g + 8 * h;
                    if (row >= M) continue;
                    uint32_t o = pack_out<kOutBf16>(sum[2 * h] * scale, sum[2 * h + 1] * scale);
                    if (bias != nullptr) {
                        const float2 xo = unpack_out<kOutBf16>(o);
                        const float2 bb = unpack_out<kOutBf16>(bias_pair);
                        o = pack_out<kOutBf16>(xo.x + bb.x, xo.y + bb.y);
                    }
                    *reinterpret_cast<uint32_t*>(c + static_cast<int64_t>(row) * N + col) = o;
                }
            }
        }
    }
}

// True when the warp-MMA kernel takes the problem: at most 16 rows (one and two rows of a wide output go to the vector
// kernel first) and at least sixteen CTAs of 32 columns; the activation rows are read with 8-byte loads and the output
// with 4-byte stores. It was first limited to outputs of two CTAs per SM and more; measured against the skinny tcgen05
// kernel it also wins below that: 16 rows at 4096 x 4096 11.4 against 18.3 us, 3072 x 3072 9.0 against 14.9,
// 1280 x 1280 5.0 against 8.8, 8192 x 3072 12.1 against 18.0; level at N = 3072, K = 12288 (29 us).
constexpr int64_t kWmmaMinN = 512;
// 17..128 rows run as one grid row of CTAs per 16 rows (the weight comes from L2 again for every grid row) while all of
// them are resident at once and the contraction is at most 8192 long. Measured against the skinny tcgen05 kernel:
// 32 rows at 4096 x 4096 15.0 against 20.5 us, 64 rows at 3072 x 3072 14.7 against 16.2, 128 rows at 1280 x 1280 8.3
// against 12.2; at N = 3072, K = 12288 it loses below 48 rows (36-39 against 30-33), hence the limit on K.
constexpr int64_t kWmmaGridMaxK = 8192;
inline bool wmma_eligible(const LaunchArgs& args) {
    // more than 16 rows: one grid row per 16, as long as every CTA is resident at once (three per SM) and K is short
    const int64_t ctas = ((args.N + 31) / 32) * ((args.M + 15) / 16);
    const bool rows_ok = args.M <= kWmmaMaxRows || (args.M <= kBlockM && ctas <= 3ll * device_info().sm_count && args.K <= kWmmaGridMaxK);
    return rows_ok && args.N >= kWmmaMinN && args.K % 16 == 0 &&
           (reinterpret_cast<uintptr_t>(args.a) & 7u) == 0 && (reinterpret_cast<uintptr_t>(args.b) & 15u) == 0 &&
           (reinterpret_cast<uintptr_t>(args.c) & 3u) == 0;
}

bool launch_wmma(const LaunchArgs& args) {
    const int slabs = static_cast<int>(args.K / 16);
    const dim3 grid(static_cast<unsigned>((args.N + 31) / 32), static_cast<unsigned>((args.M + 15) / 16));
#define FEATHER_SMM_WMMA_CASE(E5, AB, OUT)                                                                              \
    if (args.e5m2 == E5 && args.a_bf16 == AB && args.out_bf16 == OUT) {                                                  \
        scaled_mm_wmma_kernel<1, E5, AB, OUT><<<grid, 32 * kWmmaWarps, 0, args.stream>>>(                                \
            args.a, args.b, args.scale, args.bias, args.c, static_cast<int>(args.M), static_cast<int>(args.N),           \
            static_cast<int>(args.K), slabs);                                                                            \
        return cudaGetLastError() == cudaSuccess;                                                                        \
    }
    FEATHER_SMM_WMMA_CASE(true, false, true)
    FEATHER_SMM_WMMA_CASE(true, false, false)
    FEATHER_SMM_WMMA_CASE(false, false, true)
    FEATHER_SMM_WMMA_CASE(false, false, false)
    FEATHER_SMM_WMMA_CASE(true, true, true)
    FEATHER_SMM_WMMA_CASE(true, true, false)
    FEATHER_SMM_WMMA_CASE(false, true, true)
    FEATHER_SMM_WMMA_CASE(false, true, false)
#undef FEATHER_SMM_WMMA_CASE
    return false;
}

template <bool kE5M2, bool kOperandBf16, bool kOutBf16>
bool launch_skinny_instance(const LaunchArgs& args, int splits, float* partials, uint32_t* counters) {
    auto* kernel = &scaled_mm_skinny_kernel<kE5M2, kOperandBf16, kOutBf16>;
    static PerDeviceState configured;
    if (configured.get([&] { return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSkinnySmemBudget) == cudaSuccess ? 1 : 0; }) == 0) return false;
    CUtensorMap map_a, map_b;
    const uint32_t a_rows = static_cast<uint32_t>((args.M + 7) / 8 * 8);
    const uint32_t a_slot_bytes = a_rows * kBlockK * 2;
    // ring depth: what fits in the budget after the operand slots, the barriers and the alignment slack
    const uint32_t fixed = kSkinnyOperandStages * kSkinnyOperandBytes + 1024 + 512;
    uint32_t stages = (kSkinnySmemBudget - fixed) / (a_slot_bytes + kSkinnyRawBytes);
    if (stages > kSkinnyMaxStages) stages = kSkinnyMaxStages;
    stages -= stages % kSkinnyTeams;  // see kSkinnyTeams
    if (stages < 2) return false;
    const uint32_t smem_bytes = fixed + stages * (a_slot_bytes + kSkinnyRawBytes);
    {
        const uint64_t dims[2] = {static_cast<uint64_t>(args.K), static_cast<uint64_t>(args.M)};
        const uint64_t strides[1] = {static_cast<uint64_t>(args.K) * 2};
        const uint32_t box[2] = {kBlockK, a_rows};
        if (!encode_map(&map_a, args.a_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, args.a, dims, strides, box,
                        CU_TENSOR_MAP_SWIZZLE_128B)) {
            return false;
        }
    }
    {
        const uint64_t k16_rows = static_cast<uint64_t>((args.K + 127) / 128) * 8;
        const uint64_t dims[2] = {static_cast<uint64_t>(args.N) * 2, k16_rows};
        const uint64_t strides[1] = {static_cast<uint64_t>(args.N) * 16};
        const uint32_t box[2] = {kSkinnyN * 2, kSlabsPerBlock};
        if (!encode_map(&map_b, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, args.b, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE)) return false;
    }
    SkinnyParams sp{};
    sp.base.scale = args.scale;
    sp.base.bias = args.bias;
    sp.base.c = args.c;
    sp.base.M = static_cast<int>(args.M);
    sp.base.N = static_cast<int>(args.N);
    sp.base.K = static_cast<int>(args.K);
    sp.base.tiles_m = 1;
    sp.base.tiles_n = static_cast<int>((args.N + kSkinnyN - 1) / kSkinnyN);
    sp.base.idesc = make_idesc(kAccF32, args.a_bf16 ? kFmtBF16 : kFmtF16, kOperandBf16 ? kFmtBF16 : kFmtF16, kBlockM, kSkinnyN);
    sp.base.bias_vec = 0;
    const int num_kb = static_cast<int>((args.K + kBlockK - 1) / kBlockK);
    if (splits < 1) splits = 1;
    if (splits > num_kb) splits = num_kb;
    sp.kb_per_split = (num_kb + splits - 1) / splits;
    sp.splits = (num_kb + sp.kb_per_split - 1) / sp.kb_per_split;  // no empty split
    sp.partials = partials;
    sp.counters = counters;
    sp.a_slot_bytes = a_slot_bytes;
    sp.load_stages = stages;
    const int64_t grid = static_cast<int64_t>(sp.base.tiles_n) * sp.splits;
    if (grid > (1 << 30)) return false;
    kernel<<<static_cast<unsigned>(grid), kSkinnyThreads, smem_bytes, args.stream>>>(map_a, map_b, sp);
    return cudaGetLastError() == cudaSuccess;
}

// A caller that asks for a K split (more than one effective split, with scratch) gets the tcgen05 kernel that
// splits K: the scratch and the tickets are then really used, whatever the shape. Without a split the fastest
// kernel for the shape runs: the vector kernel for one or two rows of a wide output, the warp-MMA kernel for few
// rows, else the tcgen05 kernel with 64-wide tiles.
bool launch_skinny(const LaunchArgs& args, int splits, float* partials, uint32_t* counters) {
    const bool operand_bf16 = args.a_bf16;
    const bool split_requested = effective_splits(args.K, splits) > 1 && partials != nullptr && counters != nullptr;
    if (!split_requested) {
        int slabs = 0;
        size_t smem_bytes = 0;
        if (gemv_eligible(args, &slabs, &smem_bytes)) return launch_gemv(args, slabs, smem_bytes);
        if (wmma_eligible(args) && !skinny_wmma_off()) return launch_wmma(args);
        splits = 1;
    }
#define FEATHER_SMM_SKINNY_CASE(E5, OB, OUT)                               \
    if (args.e5m2 == E5 && operand_bf16 == OB && args.out_bf16 == OUT) {    \
        return launch_skinny_instance<E5, OB, OUT>(args, splits, partials, counters); \
    }
    FEATHER_SMM_SKINNY_CASE(true, false, true)
    FEATHER_SMM_SKINNY_CASE(true, false, false)
    FEATHER_SMM_SKINNY_CASE(false, false, true)
    FEATHER_SMM_SKINNY_CASE(false, false, false)
    FEATHER_SMM_SKINNY_CASE(true, true, true)
    FEATHER_SMM_SKINNY_CASE(true, true, false)
    FEATHER_SMM_SKINNY_CASE(false, true, true)
    FEATHER_SMM_SKINNY_CASE(false, true, false)
#undef FEATHER_SMM_SKINNY_CASE
    return false;
}

// Number of K splits that `launch_skinny` will actually use for a request of `splits`.
inline int effective_splits(int64_t K, int splits) {
    const int num_kb = static_cast<int>((K + kBlockK - 1) / kBlockK);
    if (splits < 1) splits = 1;
    if (splits > num_kb) splits = num_kb;
    const int per = (num_kb + splits - 1) / splits;
    return (num_kb + per - 1) / per;
}

template <int BN>
bool launch_for_block_n(const LaunchArgs& args) {
    const bool operand_bf16 = args.a_bf16;  // the weights are decoded to the activation's format
#define FEATHER_SMM_CASE(E5, OB, OUT)                                      \
    if (args.e5m2 == E5 && operand_bf16 == OB && args.out_bf16 == OUT) {    \
        return launch_instance<BN, E5, OB, OUT>(args);                      \
    }
    FEATHER_SMM_CASE(true, false, true)
    FEATHER_SMM_CASE(true, false, false)
    FEATHER_SMM_CASE(false, false, true)
    FEATHER_SMM_CASE(false, false, false)
    FEATHER_SMM_CASE(true, true, true)
    FEATHER_SMM_CASE(true, true, false)
    FEATHER_SMM_CASE(false, true, true)
    FEATHER_SMM_CASE(false, true, false)
#undef FEATHER_SMM_CASE
    return false;
}

}  // namespace smm
}  // namespace feather

// C ABI, same signature as the reference's `launch_scaled_mm` (csrc/hip_kernel.cu:687-713) with a CUDA
// stream. The six tile integers are the reference's `(warps_m, warps_n, unroll_k, repeat_m, repeat_n,
// prefetch)` tuple: it must be a row of the tile table, and its `16 * warps_n * repeat_n` width picks the
// UMMA tile width. Returns false for an unknown tuple or unsupported shape; never synchronizes.
extern "C" bool launch_scaled_mm(const uint16_t* a, const uint8_t* b_prepacked, const float* scale, const uint16_t* bias, uint16_t* c,
                                 int64_t M, int64_t N, int64_t K, int has_scale, int has_bias, bool use_fp8_e5m2, bool a_bf16,
                                 bool output_bf16, int block_warps_m, int block_warps_n, int unroll_k, int repeat_m, int repeat_n,
                                 bool prefetch, cudaStream_t stream) {
    using namespace feather;
    const int block_n = scaled_mm_tile_block_n(block_warps_m, block_warps_n, unroll_k, repeat_m, repeat_n, prefetch ? 1 : 0);
    if (block_n == 0) return false;
    if (M < 0 || N <= 0 || K <= 0 || N % 16 != 0 || K % 16 != 0) return false;
    if (M > (1 << 30) || N > (1 << 30) || K > (1 << 30)) return false;
    if (M == 0) return true;
    const smm::LaunchArgs args{a, b_prepacked, has_scale ? scale : nullptr, has_bias ? bias : nullptr, c, M, N, K,
                               use_fp8_e5m2, a_bf16, output_bf16, stream};
    if (block_n >= 256) {
        // a pair tile is 256 rows tall: worth it as soon as there is more than one 128-row tile
        if (M > smm::kBlockM && smm::pair_kernel_enabled()) return smm::launch_pair(args);
        return smm::launch_for_block_n<256>(args);
    }
    if (block_n >= 128) return smm::launch_for_block_n<128>(args);
    // narrow tiles with at most one row tile: one CTA per 64-column tile, two CTAs per SM
    if (M <= smm::kBlockM) return smm::launch_skinny(args, 1, nullptr, nullptr);
    return smm::launch_for_block_n<64>(args);
}

// Split-K variant for skinny problems (M <= 128), no counterpart in the reference's C ABI (its README calls
// split-K "no notable speedup" on gfx11; on B200 a 1..16-row product is bound by how many CTAs stream the
// weight). `partials` is scratch for `feather_scaled_mm_splitk_partial_floats(M, N, K, splits)` floats,
// `counters` holds ceil(N / 64) uint32 that must be zero before the first launch and are left zero by every
// launch. Launches that share the scratch must not overlap on the device. The result is deterministic:
// partial sums are added in split order.
extern "C" bool launch_scaled_mm_splitk(const uint16_t* a, const uint8_t* b_prepacked, const float* scale, const uint16_t* bias, uint16_t* c,
                                        int64_t M, int64_t N, int64_t K, int has_scale, int has_bias, bool use_fp8_e5m2, bool a_bf16,
                                        bool output_bf16, int splits, float* partials, uint32_t* counters, cudaStream_t stream) {
    using namespace feather;
    if (M < 0 || M > smm::kBlockM || N <= 0 || K <= 0 || N % 16 != 0 || K % 16 != 0) return false;
    if (N > (1 << 30) || K > (1 << 30)) return false;
    if (M == 0) return true;
    if (smm::effective_splits(K, splits) > 1 && (partials == nullptr || counters == nullptr)) return false;
    const smm::LaunchArgs args{a, b_prepacked, has_scale ? scale : nullptr, has_bias ? bias : nullptr, c, M, N, K,
                               use_fp8_e5m2, a_bf16, output_bf16, stream};
    return smm::launch_skinny(args, splits, partials, counters);
}

// launch_scaled_mm_splitk for taller problems, on the one-CTA kernel with 128 x `block_n` tiles (`block_n` 128 or 256):
// a work item is (tile, K split), so a product with too few tiles for the SMs (a few hundred rows) still occupies
// them all. `partials` holds feather_scaled_mm_splitk_wide_partial_floats(M, N, K, block_n, splits) floats; `counters` holds ceil(M / 128) * ceil(N / block_n) zeroed uint32, left zero again.
// Any M. Returns false for another `block_n` or an unsupported shape.
extern "C" bool launch_scaled_mm_splitk_wide(const uint16_t* a, const uint8_t* b_prepacked, const float* scale, const uint16_t* bias, uint16_t* c,
                                             int64_t M, int64_t N, int64_t K, int has_scale, int has_bias, bool use_fp8_e5m2, bool a_bf16,
                                             bool output_bf16, int block_n, int splits, float* partials, uint32_t* counters, cudaStream_t stream) {
    using namespace feather;
    if (block_n != 128 && block_n != 256) return false;
    if (M < 0 || N <= 0 || K <= 0 || N % 16 != 0 || K % 16 != 0) return false;
    if (M > (1 << 30) || N > (1 << 30) || K > (1 << 30)) return false;
    if (M == 0) return true;
    if (smm::effective_splits(K, splits) > 1 && (partials == nullptr || counters == nullptr)) return false;
    smm::LaunchArgs args{a, b_prepacked, has_scale ? scale : nullptr, has_bias ? bias : nullptr, c, M, N, K,
                         use_fp8_e5m2, a_bf16, output_bf16, stream};
    args.splits = splits;
    args.partials = partials;
    args.counters = counters;
    if (block_n == 256 && M > smm::kBlockM && smm::pair_kernel_enabled() && smm::effective_splits(K, splits) > 1) {
        // more than one row tile: CTA pairs, one (256 x 256 tile, split) item per pair, when all items fit the device at once
        if (smm::launch_pair(args, true)) return true;
        (void)cudaGetLastError();
    }
    return block_n == 256 ? smm::launch_for_block_n<256>(args) : smm::launch_for_block_n<128>(args);
}

// Number of uint32 tickets `launch_scaled_mm_splitk_wide` needs in `counters` (zero before the first launch).
extern "C" int64_t feather_scaled_mm_splitk_wide_counters(int64_t M, int64_t N, int block_n) {
    if (M <= 0 || N <= 0 || (block_n != 128 && block_n != 256)) return 0;
    // the one-CTA kernel: an "in" and a "done" counter per 128 x block_n tile; the CTA-pair kernel: two "in" counters (one per row half) and a "done" counter per 256 x 256 tile
    const int64_t one_cta = 2 * ((M + feather::smm::kBlockM - 1) / feather::smm::kBlockM) * ((N + block_n - 1) / block_n);
    const int64_t pair = (block_n == 256 && M > feather::smm::kBlockM) ? 3 * feather::smm::pair_tiles(M, N) : 0;
    return one_cta > pair ? one_cta : pair;
}

// Floats of `partials` scratch that `launch_scaled_mm_splitk_wide` needs: whole 128 x block_n tiles per split
// (0 when the request collapses to one split or `block_n` is not 128 or 256).
extern "C" int64_t feather_scaled_mm_splitk_wide_partial_floats(int64_t M, int64_t N, int64_t K, int block_n, int splits) {
    if (M <= 0 || N <= 0 || K <= 0 || (block_n != 128 && block_n != 256)) return 0;
    const int effective = feather::smm::effective_splits(K, splits);
    int64_t tiles = ((M + feather::smm::kBlockM - 1) / feather::smm::kBlockM) * ((N + block_n - 1) / block_n);
    // the CTA-pair kernel (block_n 256, more than one row tile) keeps whole 256 x 256 tiles: two 128-row halves per pair tile
    if (block_n == 256 && M > feather::smm::kBlockM && 2 * feather::smm::pair_tiles(M, N) > tiles) tiles = 2 * feather::smm::pair_tiles(M, N);
    return effective > 1 ? static_cast<int64_t>(effective) * tiles * feather::smm::kBlockM * block_n : 0;
}

// Floats of `partials` scratch that `launch_scaled_mm_splitk` needs (0 when the request collapses to one split).
extern "C" int64_t feather_scaled_mm_splitk_partial_floats(int64_t M, int64_t N, int64_t K, int splits) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    const int effective = feather::smm::effective_splits(K, splits);
    return effective > 1 ? static_cast<int64_t>(effective) * M * N : 0;
}

// ---------------------------------------------------------------------------------------------------------
// Split-K scaled_mm without any allocation: the scratch lives in this library's own device memory.
//
// Who needs this: hosts that bind the C ABI directly and have nothing to allocate device memory with once
// they are running. Examples are a serving loop that has handed all free device memory to its own arena at
// start-up (so a later cudaMalloc fails or, worse, stalls the device while the driver reshuffles), a
// foreign-language plugin (C, Go, Rust through FFI) that owns its input and output buffers but has no
// device allocator of its own, and code running inside a callback where the runtime forbids allocation
// calls. They still pass inputs and outputs; only the fp32 partials and the per-tile tickets come from here.
//
// The scratch is one file-scope __device__ array (4 MiB of partials + 1 KiB of tickets, held by every GPU
// that loads the library, from load until exit). That bounds the problems this entry point accepts:
// M <= 16, N <= 16384 and at most 4 splits; anything larger is refused with an error code and message.
// On the host the array's name is only a handle, not a device address: the address is looked up once per
// device with cudaGetSymbolAddress (with that device current), by the first call made on that device. That
// first call therefore does a little extra runtime work and should be made before any stream capture begins.
// Every call uses the same array and finds the previous call's partials in it; the tickets, which must start
// at zero, are cleared on the caller's stream before each launch. Two calls that run on the device at the
// same time (different streams, different host threads) would race on the scratch: serialize them.
// ---------------------------------------------------------------------------------------------------------
namespace feather {
namespace smm {

constexpr int64_t kStaticMaxM = 16;
constexpr int64_t kStaticMaxN = 16384;
constexpr int kStaticMaxSplits = 4;
constexpr size_t kStaticPartialBytes = static_cast<size_t>(kStaticMaxSplits) * kStaticMaxM * kStaticMaxN * sizeof(float);  // 4 MiB
constexpr size_t kStaticCounterBytes = (kStaticMaxN / kSkinnyN) * sizeof(uint32_t);                                         // 1 KiB

static __device__ __align__(256) unsigned char g_static_scratch[kStaticPartialBytes + kStaticCounterBytes];

// Device address of the scratch on the current device, looked up on first use. Returns nullptr on failure.
static unsigned char* static_scratch_address(cudaError_t* error) {
    static std::mutex lock;
    static unsigned char* address[64] = {};
    int dev = 0;
    *error = cudaGetDevice(&dev);
    if (*error != cudaSuccess || dev < 0 || dev >= 64) {
        if (*error == cudaSuccess) *error = cudaErrorInvalidDevice;
        return nullptr;
    }
    std::lock_guard<std::mutex> hold(lock);
    if (address[dev] == nullptr) {
        void* found = nullptr;
        *error = cudaGetSymbolAddress(&found, g_static_scratch);
        if (*error != cudaSuccess) return nullptr;
        address[dev] = static_cast<unsigned char*>(found);
    }
    return address[dev];
}

static void write_message(char* out, size_t capacity, const char* text) {
    if (out != nullptr && capacity > 0) snprintf(out, capacity, "%s", text);
}

}  // namespace smm
}  // namespace feather

// Same computation and arguments as launch_scaled_mm_splitk, minus the two scratch pointers. Returns 0 when
// the kernel was enqueued; 1 for arguments launch_scaled_mm_splitk would refuse too; 2 when the problem is
// larger than the built-in scratch (M > 16, N > 16384 or more than 4 effective splits); 3 when a CUDA call
// failed. `error_message` (may be NULL) receives a description for every nonzero return. Calls no
// allocating routine. Calls that overlap on the device race on the shared scratch.
extern "C" int launch_scaled_mm_splitk_static(const uint16_t* a, const uint8_t* b_prepacked, const float* scale, const uint16_t* bias,
                                              uint16_t* c, int64_t M, int64_t N, int64_t K, int has_scale, int has_bias, bool use_fp8_e5m2,
                                              bool a_bf16, bool output_bf16, int splits, cudaStream_t stream, char* error_message,
                                              size_t error_capacity) {
    using namespace feather;
    if (M < 0 || N <= 0 || K <= 0 || N % 16 != 0 || K % 16 != 0 || K > (1 << 30)) {
        smm::write_message(error_message, error_capacity, "scaled_mm_splitk_static: M must be >= 0, N and K positive multiples of 16");
        return 1;
    }
    const int effective = smm::effective_splits(K, splits);
    if (M > smm::kStaticMaxM || N > smm::kStaticMaxN || effective > smm::kStaticMaxSplits) {
        char text[200];
        snprintf(text, sizeof(text),
                 "scaled_mm_splitk_static: M=%lld N=%lld splits=%d exceeds the built-in scratch (M <= %lld, N <= %lld, splits <= %d); "
                 "use launch_scaled_mm_splitk with caller scratch",
                 static_cast<long long>(M), static_cast<long long>(N), effective, static_cast<long long>(smm::kStaticMaxM),
                 static_cast<long long>(smm::kStaticMaxN), smm::kStaticMaxSplits);
        smm::write_message(error_message, error_capacity, text);
        return 2;
    }
    if (M == 0) return 0;
    cudaError_t error = cudaSuccess;
    unsigned char* const scratch = smm::static_scratch_address(&error);
    if (scratch == nullptr) {
        smm::write_message(error_message, error_capacity, cudaGetErrorString(error));
        return 3;
    }
    float* const partials = reinterpret_cast<float*>(scratch);
    uint32_t* const counters = reinterpret_cast<uint32_t*>(scratch + smm::kStaticPartialBytes);
    // the tickets must start at zero whatever an earlier (possibly interrupted) call left behind
    error = cudaMemsetAsync(counters, 0, smm::kStaticCounterBytes, stream);
    if (error != cudaSuccess) {
        smm::write_message(error_message, error_capacity, cudaGetErrorString(error));
        return 3;
    }
    const smm::LaunchArgs args{a, b_prepacked, has_scale ? scale : nullptr, has_bias ? bias : nullptr, c, M, N, K,
                               use_fp8_e5m2, a_bf16, output_bf16, stream};
    if (!smm::launch_skinny(args, splits, partials, counters)) {
        smm::write_message(error_message, error_capacity, "scaled_mm_splitk_static: the kernel launch failed");
        return 3;
    }
    return 0;
}

// Leaves `sms` SMs free in every later launch of the persistent scaled_mm kernels (the CTA-pair kernel and the one-CTA
// kernel size their grids by the SM count); 0 restores full grids. For a caller that overlaps the product with other
// kernels that need SMs of their own, e.g. an NCCL collective on another stream. Returns the previous value.
// Process-wide; takes effect at the next launch. No counterpart in the reference.
extern "C" int feather_scaled_mm_set_sm_margin(int sms) {
    if (sms < 0) sms = 0;
    return feather::smm::g_sm_margin.exchange(sms, std::memory_order_relaxed);
}

// out[r][g][:] = slabs[g][r][:] for g < world, r < rows, rows of `width_bytes` bytes (a multiple of 16, pointers 16-byte
// aligned): turns the [world][rows][width] result of an all-gather of column slabs into the row-major [rows][world * width]
// matrix. A plain HBM-bound copy kernel with 16-byte accesses. Returns false for bad arguments. No counterpart in the
// reference (it has no multi-GPU path).
namespace feather {
namespace smm {
__global__ void __launch_bounds__(256) interleave_slabs_kernel(const uint4* __restrict__ slabs, uint4* __restrict__ out, int64_t world, int64_t rows,
                                                                int64_t width16) {
    const int64_t total = world * rows * width16;
    const int64_t row16 = world * width16;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        // i indexes the output: row r, slab g, 16-byte unit w
        const int64_t r = i / row16;
        const int64_t rem = i - r * row16;
        const int64_t g = rem / width16;
        const int64_t w = rem - g * width16;
        out[i] = __ldcs(slabs + (g * rows + r) * width16 + w);
    }
}
}  // namespace smm
}  // namespace feather

extern "C" bool launch_interleave_slabs(const void* slabs, void* out, int64_t world, int64_t rows, int64_t width_bytes, cudaStream_t stream) {
    if (world <= 0 || rows < 0 || width_bytes <= 0 || width_bytes % 16 != 0) return false;
    if (((reinterpret_cast<uintptr_t>(slabs) | reinterpret_cast<uintptr_t>(out)) & 15u) != 0) return false;
    if (rows == 0) return true;
    const int64_t total = world * rows * (width_bytes / 16);
    int64_t blocks = (total + 255) / 256;
    const int64_t cap = static_cast<int64_t>(feather::device_info().sm_count) * 16;
    if (blocks > cap) blocks = cap;
    feather::smm::interleave_slabs_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(static_cast<const uint4*>(slabs), static_cast<uint4*>(out), world, rows,
                                                                                             width_bytes / 16);
    return cudaGetLastError() == cudaSuccess;
}

// Output columns per tile that the CTA-pair kernel (256-wide tile tuples, more than 128 rows, no K split) uses for `M` rows and `N` columns
// when `pairs` CTA pairs are resident (74 on a B200). For tests and logs.
extern "C" int feather_scaled_mm_pair_tile_width(int64_t M, int64_t N, int pairs) { return feather::smm::pair_tile_width(M, N, pairs); }

// Reads (and clears) the status record the kernel's bounded waits report into: out[0] = wait site
// (0 = every wait completed) | tag << 8, out[1] = block index. Synchronizes the device.
extern "C" int feather_scaled_mm_status(uint32_t* out) {
    uint32_t zero[2] = {0u, 0u};
    if (cudaDeviceSynchronize() != cudaSuccess) return 1;
    if (cudaMemcpyFromSymbol(out, feather::smm::g_status, sizeof(zero)) != cudaSuccess) return 1;
    if (cudaMemcpyToSymbol(feather::smm::g_status, zero, sizeof(zero)) != cudaSuccess) return 1;
    return 0;
}
