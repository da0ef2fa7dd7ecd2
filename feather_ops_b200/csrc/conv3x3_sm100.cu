// 3x3, stride 1, padding 1, NCHW conv2d (fp16 / bf16) for sm_100a as an implicit GEMM on tcgen05.
//
// GEMM view, as in the reference (csrc/hip_conv2d_3x3.cu:1-26): M = C_out, N = pixels, K = 9 * C_in with
// the contraction ordered (16-channel group, tap, channel % 16). The weight is the reference's prepack
// [ceil(C_in / 16) * 18][C_out][8]: row g * 18 + tap * 2 + half holds, per output channel, eight
// consecutive input channels, i.e. one 16-byte K-major core-matrix row. B200 counterpart of
// `conv3x3_kernel` / `feather_conv3x3_launch` (kernel :100-476, C ABI :561-575).
//
// One persistent CTA per SM walks tiles of 128 output channels x (rows x BN) pixels, one launch for the
// whole batch. Per 16-channel group (one pipeline slot):
//   * warp 0 (TMA): the group's 18 weight rows x 128 channels (2 KB contiguous each) land as [18][128][16 B], which already is
//     the no-swizzle K-major UMMA layout (8-channel core matrices 128 B apart, K-adjacent ones 2 KB apart).
//     Output channels past C_out are zero filled by the TMA unit.
//   * sixteen gather warps in two alternating teams: read the (rows + 2) x (BN + 2) halo tile of the
//     group's 16 input channels straight from global memory, interleave eight channels per pixel and
//     store [plane][halo row][halo col][8 channels]. A pixel is one 16-byte record, so eight consecutive
//     pixels are a core matrix and tap (kh, kw) of output row r is nothing but a start-address offset of
//     ((r + kh) * (BN + 2) + kw) records. Out-of-image pixels and channels past C_in are written as zeros,
//     which is the padding.
//   * warp 1: one thread issues 9 x rows tcgen05.mma kind::f16 (M = 128, N = BN, K = 16) per group into
//     one of two fp32 TMEM accumulators (k order: groups ascending, taps 0..8 inside, as the reference).
//   * four epilogue warps: TMEM lane = output channel, columns = consecutive pixels of one output row;
//     add the bias in fp32, round once, 64-byte contiguous NCHW stores.
// With more than 128 output channels and the two-row tile, CTA pairs take over: two SMs share the pixels of a
// 256-channel tile. Four kernels in this file: the one above and its CTA-pair form (halo tiles gathered from global
// memory, any width), and the staged forms of both for W % 8 == 0 (halo tiles by TMA, two tiles per weight slot,
// output through bulk tensor stores), which serve every benchmark shape.
#include "feather_host.h"
#include "feather_tiles_gen.h"
#include "sm100_ptx.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdlib>

namespace feather {
namespace conv {

constexpr int kBlockM = 128;
constexpr int kStages = 3;
constexpr int kGatherWarps = 16;
constexpr int kTeams = 2;   // one-CTA kernel (four teams over four slots measured half as fast: eight items per thread)
constexpr int kTeamWarps = kGatherWarps / kTeams;
constexpr int kEpilogueWarps = 4;
constexpr int kFirstEpilogueWarp = 2;
constexpr int kFirstGatherWarp = kFirstEpilogueWarp + kEpilogueWarps;
constexpr int kThreads = 32 * (kFirstGatherWarp + kTeams * kTeamWarps);
constexpr int kWeightRows = 18;                                  // 9 taps x 2 eight-channel halves
constexpr int kWeightStageBytes = kWeightRows * kBlockM * 16;    // 36864
constexpr int kMaxItems = 4;                                     // pixel-pair gather items per thread per slot
constexpr int kAccColumns = 256;                                 // TMEM columns per accumulator buffer

__device__ uint32_t g_status[2];

struct Params {
    const uint16_t* x;
    const uint16_t* bias;
    uint16_t* y;
    int B, C_in, C_out, H, W;
    int groups;       // ceil(C_in / 16)
    int bn;           // pixels per output row segment (UMMA N): 64, 128 or 256
    int rows;         // output rows per tile: 1 or 2
    int tiles_m, tiles_w, tiles_h;
    int act_stage_bytes;
    uint32_t idesc;
    int pairs;        // W is even: gather two pixels per 4-byte load
    int staging_bytes;   // staged kernels: bytes of one slot's raw halo tile [16 channels][rows + 2][bn + 16] as TMA delivers it
    int weight_slots, raw_slots, rec_slots;   // staged one-CTA kernel: ring depths
};

template <bool kBf16>
__device__ __forceinline__ uint32_t pack_out(float a, float b) {
    if constexpr (kBf16) {
        const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<const uint32_t*>(&v);
    } else {
        const __half2 v = __floats2half2_rn(a, b);
        return *reinterpret_cast<const uint32_t*>(&v);
    }
}

template <bool kBf16>
__device__ __forceinline__ float bits_to_float(uint16_t bits) {
    if constexpr (kBf16) {
        return __uint_as_float(static_cast<uint32_t>(bits) << 16);
    } else {
        return __half2float(__ushort_as_half(bits));
    }
}

struct TileCoord {
    int b, m0, h0, w0;
};

__device__ __forceinline__ TileCoord tile_coord(const Params& p, int tile) {
    TileCoord t;
    t.m0 = (tile % p.tiles_m) * kBlockM;
    tile /= p.tiles_m;
    t.w0 = (tile % p.tiles_w) * p.bn;
    tile /= p.tiles_w;
    t.h0 = (tile % p.tiles_h) * p.rows;
    t.b = tile / p.tiles_h;
    return t;
}

// one chunk of 32 consecutive pixels of an output row: bias in fp32, one rounding, 16-byte stores where rows allow
template <bool kBf16>
__device__ __forceinline__ void store_pixels(const uint32_t (&v)[32], float bias, uint16_t* y_row, int w_first, int W, bool vector_rows) {
    if (vector_rows) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            if (w_first + g * 8 < W) {
                uint32_t o[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    o[i] = pack_out<kBf16>(__uint_as_float(v[g * 8 + 2 * i]) + bias, __uint_as_float(v[g * 8 + 2 * i + 1]) + bias);
                }
                *reinterpret_cast<uint4*>(y_row + w_first + g * 8) = make_uint4(o[0], o[1], o[2], o[3]);
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            if (w_first + i < W) {
                const uint32_t o = pack_out<kBf16>(__uint_as_float(v[i]) + bias, 0.0f);
                y_row[w_first + i] = static_cast<uint16_t>(o & 0xffffu);
            }
        }
    }
}

// The kernel for every shape the staged kernels below do not take (widths that are not multiples of 8, row segments of
// 256 pixels, unaligned inputs): the gather warps load the halo tile from global memory into registers, one group per
// team in flight.
template <bool kBf16>
__global__ void __launch_bounds__(kThreads, 1) conv3x3_kernel(const __grid_constant__ CUtensorMap map_w, const Params p) {
    extern __shared__ uint8_t smem_dyn[];
    uint8_t* const smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t* const weight_smem = smem;
    uint8_t* const act_smem = smem + kStages * kWeightStageBytes;
    uint64_t* const bars = reinterpret_cast<uint64_t*>(act_smem + kStages * p.act_stage_bytes);
    uint64_t* const weight_full = bars;
    uint64_t* const act_full = weight_full + kStages;
    uint64_t* const stage_empty = act_full + kStages;
    uint64_t* const tmem_full = stage_empty + kStages;
    uint64_t* const tmem_empty = tmem_full + 2;
    uint32_t* const tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
    volatile uint32_t* const abort_flag = tmem_slot + 1;

    const int warp = static_cast<int>(threadIdx.x) / 32;
    const int lane = static_cast<int>(threadIdx.x) % 32;
    const WaitGuard guard{abort_flag, g_status};
    // Two teams over three slots: a team skips every other use of a slot. Its parity waits stay sound because the
    // barriers it waits on are MMA commits, which arrive in issue order (a team that has passed its wait for one group
    // knows that every earlier group's commit has arrived, so it is never a whole ring ahead of a barrier's phase).

    if (threadIdx.x == 0) {
        *abort_flag = 0u;
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&weight_full[s], 1);
            mbar_init(&act_full[s], kTeamWarps);
            mbar_init(&stage_empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&tmem_full[s], 1);
            mbar_init(&tmem_empty[s], kEpilogueWarps);
        }
        mbar_init_fence();
        tma_prefetch_desc(&map_w);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 2 * kAccColumns);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    const int num_tiles = p.B * p.tiles_m * p.tiles_h * p.tiles_w;
    const int halo_cols = p.bn + 2;
    const int halo_rows = p.rows + 2;
    const int plane_bytes = halo_rows * halo_cols * 16;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (weights)
        if (elect_one()) {
            uint32_t it = 0;
            bool ok = true;
            for (int tile = static_cast<int>(blockIdx.x); ok && tile < num_tiles; tile += static_cast<int>(gridDim.x)) {
                const TileCoord tc = tile_coord(p, tile);
                for (int g = 0; g < p.groups; ++g, ++it) {
                    const uint32_t s = it % kStages;
                    const uint32_t phase = (it / kStages) & 1u;
                    ok = guard.wait(&stage_empty[s], phase ^ 1u, kSiteLoadEmpty);
                    if (!ok) break;
                    mbar_arrive_expect_tx(&weight_full[s], kWeightStageBytes);
                    tma_load_2d(weight_smem + s * kWeightStageBytes, &map_w, &weight_full[s], tc.m0 * 2, g * kWeightRows);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (elect_one()) {
            uint32_t it = 0;
            uint32_t acc_it = 0;
            bool ok = true;
            for (int tile = static_cast<int>(blockIdx.x); ok && tile < num_tiles; tile += static_cast<int>(gridDim.x), ++acc_it) {
                const uint32_t acc = acc_it & 1u;
                ok = guard.wait(&tmem_empty[acc], ((acc_it >> 1) & 1u) ^ 1u, kSiteTmemEmpty);
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t tmem_d = tmem_base + acc * kAccColumns;
                for (int g = 0; g < p.groups; ++g, ++it) {
                    const uint32_t s = it % kStages;
                    const uint32_t phase = (it / kStages) & 1u;
                    ok = guard.wait(&weight_full[s], phase, kSiteLoadFull) && guard.wait(&act_full[s], phase, kSiteOperandFull);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint32_t w_addr = smem_u32(weight_smem + s * kWeightStageBytes);
                    const uint32_t x_addr = smem_u32(act_smem + s * p.act_stage_bytes);
                    // the start address sits in the low bits of a descriptor in 16-byte units: a tap is an addition
                    const uint64_t desc_w0 = make_smem_desc(w_addr, kBlockM * 16, 128, kSwizzleNone);
                    const uint64_t desc_x0 = make_smem_desc(x_addr, plane_bytes, 128, kSwizzleNone);
#pragma unroll
                    for (int tap = 0; tap < 9; ++tap) {
                        const int kh = tap / 3;
                        const int kw = tap % 3;
                        const uint64_t desc_w = desc_w0 + static_cast<uint64_t>(tap * 2 * kBlockM);
                        for (int r = 0; r < p.rows; ++r) {
                            const uint64_t desc_x = desc_x0 + static_cast<uint64_t>((r + kh) * halo_cols + kw);
                            umma_f16(tmem_d + r * p.bn, desc_w, desc_x, p.idesc, (g | tap) != 0 ? 1u : 0u);
                        }
                    }
                    umma_commit(&stage_empty[s]);
                }
                if (!ok) break;
                umma_commit(&tmem_full[acc]);
            }
        }
    } else if (warp < kFirstGatherWarp) {
        // ------------------------------------------------------------------ epilogue
        const int quarter = warp % 4;
        const bool vector_rows = (p.W % 8) == 0;
        uint32_t acc_it = 0;
        bool ok = true;
        for (int tile = static_cast<int>(blockIdx.x); ok && tile < num_tiles; tile += static_cast<int>(gridDim.x), ++acc_it) {
            const TileCoord tc = tile_coord(p, tile);
            const uint32_t acc = acc_it & 1u;
            ok = guard.wait(&tmem_full[acc], (acc_it >> 1) & 1u, kSiteTmemFull);
            if (!ok) break;
            tc_fence_after_sync();
            const int co = tc.m0 + quarter * 32 + lane;
            const bool co_live = co < p.C_out;
            const float bias = (p.bias != nullptr && co_live) ? bits_to_float<kBf16>(__ldg(p.bias + co)) : 0.0f;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * kAccColumns;
            const int chunks = p.bn / 32;
            for (int r = 0; r < p.rows; ++r) {
                const int h = tc.h0 + r;
                uint16_t* const y_row = p.y + ((static_cast<int64_t>(tc.b) * p.C_out + (co_live ? co : 0)) * p.H + (h < p.H ? h : 0)) * p.W;
#pragma unroll 1
                for (int c = 0; c < chunks; ++c) {
                    uint32_t v[32];
                    tmem_ld_32x32(taddr + r * p.bn + c * 32, v);
                    tmem_wait_ld();
                    if (r == p.rows - 1 && c == chunks - 1) {
                        tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&tmem_empty[acc]);
                    }
                    if (!co_live || h >= p.H) continue;
                    store_pixels<kBf16>(v, bias, y_row, tc.w0 + c * 32, p.W, vector_rows);
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ activation gather warps
        const int team = (warp - kFirstGatherWarp) / kTeamWarps;
        const int t = static_cast<int>(threadIdx.x) - (kFirstGatherWarp + team * kTeamWarps) * 32;
        constexpr int kTeamThreads = kTeamWarps * 32;
        const int64_t hw = static_cast<int64_t>(p.H) * p.W;
        // Work items of one slot. With `pairs`: per (plane, halo row) the halo columns 1..BN as BN / 2 aligned
        // pixel pairs, then the two edge columns 0 and BN + 1 as single pixels. Without: every column alone.
        const int per_row = p.pairs ? p.bn / 2 + 2 : halo_cols;
        const int items = 2 * halo_rows * per_row;
        uint32_t it = 0;
        bool ok = true;
        for (int tile = static_cast<int>(blockIdx.x); ok && tile < num_tiles; tile += static_cast<int>(gridDim.x)) {
            const TileCoord tc = tile_coord(p, tile);
            const uint16_t* const x_img = p.x + static_cast<int64_t>(tc.b) * p.C_in * hw;
            // The item geometry depends on the tile only: decode it once, so that the per-group work is loads,
            // byte permutes and stores. `kind`: 0 = nothing (past the item list or outside the image, where the
            // zeros are stored without loading), 1 = single pixel, 2 = pixel pair.
            int64_t src_off[kMaxItems];   // element offset of channel (plane * 8) of group 0 at the item's first pixel
            int dst_off[kMaxItems];       // byte offset inside the stage; < 0: no item
            uint32_t kinds = 0;            // 4 bits per item: kind | in_image << 2 | plane << 3
#pragma unroll
            for (int j = 0; j < kMaxItems; ++j) {
                const int item = t + j * kTeamThreads;
                src_off[j] = 0;
                dst_off[j] = -1;
                if (item < items) {
                    const int plane = item / (halo_rows * per_row);
                    const int rem = item % (halo_rows * per_row);
                    const int hr = rem / per_row;
                    const int e = rem % per_row;
                    int hc;       // first halo column of the item
                    bool pair;
                    if (p.pairs) {
                        pair = e < p.bn / 2;
                        hc = pair ? 1 + 2 * e : (e == p.bn / 2 ? 0 : p.bn + 1);
                    } else {
                        pair = false;
                        hc = e;
                    }
                    const int h = tc.h0 - 1 + hr;
                    const int w = tc.w0 - 1 + hc;
                    const bool in_image = h >= 0 && h < p.H && w >= 0 && w < p.W;
                    src_off[j] = static_cast<int64_t>(plane) * 8 * hw + static_cast<int64_t>(in_image ? h : 0) * p.W + (in_image ? w : 0);
                    dst_off[j] = plane * plane_bytes + (hr * halo_cols + hc) * 16;
                    kinds |= ((pair ? 2u : 1u) | (in_image ? 4u : 0u) | (plane ? 8u : 0u)) << (4 * j);
                }
            }
            for (int g = 0; g < p.groups; ++g, ++it) {
                if (static_cast<int>(it % kTeams) != team) continue;
                const uint32_t s = it % kStages;
                const uint32_t phase = (it / kStages) & 1u;
                const uint16_t* const x_group = x_img + static_cast<int64_t>(g) * 16 * hw;
                const bool second_plane_live = g * 16 + 8 < p.C_in;  // C_in is a multiple of 8: a plane is whole or absent
                // issue every load of this thread's items first, so they are all in flight together
                uint32_t v[kMaxItems][8];
#pragma unroll
                for (int j = 0; j < kMaxItems; ++j) {
                    const uint32_t k = (kinds >> (4 * j)) & 15u;
                    const bool live = (k & 4u) != 0 && ((k & 8u) == 0 || second_plane_live);
                    const uint16_t* const src = x_group + src_off[j];
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        if ((k & 2u) != 0) {
                            v[j][c] = live ? __ldg(reinterpret_cast<const uint32_t*>(src + c * hw)) : 0u;
                        } else {
                            v[j][c] = live ? static_cast<uint32_t>(__ldg(src + c * hw)) : 0u;
                        }
                    }
                }
                ok = guard.wait(&stage_empty[s], phase ^ 1u, kSiteOperandEmpty);
                if (!ok) break;
                uint8_t* const dst = act_smem + s * p.act_stage_bytes;
#pragma unroll
                for (int j = 0; j < kMaxItems; ++j) {
                    if (dst_off[j] < 0) continue;
                    // low halves = this pixel (the only one of a single), high halves = the pair's second pixel
                    const uint4 first = make_uint4(__byte_perm(v[j][0], v[j][1], 0x5410u), __byte_perm(v[j][2], v[j][3], 0x5410u),
                                                   __byte_perm(v[j][4], v[j][5], 0x5410u), __byte_perm(v[j][6], v[j][7], 0x5410u));
                    *reinterpret_cast<uint4*>(dst + dst_off[j]) = first;
                    if (((kinds >> (4 * j)) & 2u) != 0) {
                        const uint4 second = make_uint4(__byte_perm(v[j][0], v[j][1], 0x7632u), __byte_perm(v[j][2], v[j][3], 0x7632u),
                                                        __byte_perm(v[j][4], v[j][5], 0x7632u), __byte_perm(v[j][6], v[j][7], 0x7632u));
                        *reinterpret_cast<uint4*>(dst + dst_off[j] + 16) = second;
                    }
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(&act_full[s]);
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
        tmem_dealloc(tmem_base, 2 * kAccColumns);
    }
}

// ---------------------------------------------------------------------------------------------------------
// Staged kernels (W % 8 == 0): the halo tile of a 16-channel group comes by TMA as a 4-D box over the NCHW input,
// channel-planar, zero filled outside the image and past C_in (that is the padding), into a raw buffer, and the
// re-layout warps only re-lay it shared -> shared into the pixel records. A TMA box starts on a 16-byte boundary, so the
// box begins eight pixels left of the tile (w0 - 8, the halo's first column is w0 - 1) and is sixteen pixels wider; a
// box side is at most 256 elements, so a 256-pixel segment takes two boxes of 136 pixels side by side.
//
// Two tiles per weight slot. Weights, raw halo tiles and pixel records travel in rings of their own: a weight slot
// serves the same group of TWO consecutive tiles of the CTA (one accumulator each, i.e. all of tensor memory), the
// halo rings advance twice per weight step, and a raw slot is free again as soon as it has been re-laid (not when the
// UMMAs have read the records), so the copies run further ahead. A CTA owns a contiguous range of the tile list, which
// is ordered with the output-channel tile slowest, so that neighbours share their weights; the last tile of an odd
// range, or of an output-channel tile, runs alone. Per tile the accumulation order is unchanged (groups ascending,
// taps 0..8), so the results are bit-identical to the other kernels.
//
// Output: a lane holds one output channel, so storing straight to NCHW makes every warp store 32 requests of 16 bytes.
// Every epilogue warp instead lays its 32 channels x 32 pixels into a swizzled shared-memory image of its own that its first
// lane hands to the copy engine (a 4-D bulk tensor store, which also clips at the image edge and at C_out).
//
// The re-layout is ONE team that visits every use of every slot: it waits on barriers that the copy engine
// completes, in any order across slots, and a parity wait cannot tell "my phase has completed" from "the phase before
// mine has not" for a waiter that skipped a use of the slot.
//
// What each part costs was measured by leaving it out (128 channels @ 512 x 512, 95 us whole): no output stores 73 us,
// no re-layout 86, no halo copies 86, no UMMAs 78, weights and UMMAs alone 59, weights and hand-offs alone 32. The
// parts do not hide behind one another: UMMA operand reads (108 KB per group and 256 pixels), copies landing (45 KB),
// the re-layout (50 KB) and the output image (16 KB) all go through the SM's shared memory, 219 KB per 1458 clocks of
// UMMAs against 128 B per clock, and the same 45 KB come through the SM's L2 port at about 35 B per clock.
// ---------------------------------------------------------------------------------------------------------
constexpr int kMaxSlots = 4;       // ring depths are chosen by the launcher to fill the shared memory, at most this
constexpr int kStagedItems = 2;   // re-layout items per thread per halo slot
// Both accumulators of a step finish together, so their drain is exposed unless it is short: eight epilogue warps, two
// per lane quarter of tensor memory, each taking half of a tile's 32-pixel chunks.
constexpr int kStagedEpilogueWarps = 8;
constexpr int kStagedFirstGatherWarp = kFirstEpilogueWarp + kStagedEpilogueWarps;
constexpr int kStagedThreads = 32 * (kStagedFirstGatherWarp + kGatherWarps);
constexpr int kOutImageBytes = 128 * 64;   // 128 output channels x 32 pixels of 16 bits: what one bulk tensor store writes
constexpr int kOutImages = 2;              // per half of the epilogue warps: a warp writes its slice of one while the copy engine reads that of the other

struct TileRange {
    int begin, end;
};

// the contiguous share of `worker` (of `workers`) of a list of `num_tiles` tiles
__device__ __forceinline__ TileRange tile_range(int num_tiles, int worker, int workers) {
    TileRange r;
    r.begin = static_cast<int>(static_cast<int64_t>(num_tiles) * worker / workers);
    r.end = static_cast<int>(static_cast<int64_t>(num_tiles) * (worker + 1) / workers);
    return r;
}

// tiles that share the weight slots of one step: `tile` and, when it is in the range and in the same output-channel
// tile (`per_m` consecutive list entries), its successor
__device__ __forceinline__ int tiles_of_step(int tile, int end, int per_m) {
    return (tile + 1 < end && (tile + 1) % per_m != 0) ? 2 : 1;
}

// tile list of the staged kernels: pixel segments fastest, then rows, images, and the output-channel tile slowest
__device__ __forceinline__ TileCoord staged_tile_coord(const Params& p, int tile, int per_m) {
    TileCoord t;
    t.m0 = (tile / per_m) * kBlockM;
    tile %= per_m;
    t.w0 = (tile % p.tiles_w) * p.bn;
    tile /= p.tiles_w;
    t.h0 = (tile % p.tiles_h) * p.rows;
    t.b = tile / p.tiles_h;
    return t;
}

// Eight channels of a pixel pair (4-byte loads, channel-planar source) or of one edge pixel into 16-byte pixel records.
// Consecutive lanes hold consecutive pairs, so their record pairs are 32 bytes apart: a 16-byte store of "every lane's
// first record" would put lanes L and L + 4 of a quarter warp on the same banks. Lanes with bit 2 set therefore store their
// second record first (`swap`): each quarter warp then covers all 32 banks once per store.
__device__ __forceinline__ void relayout_item(const uint8_t* src, uint8_t* dst, int channel_pitch, bool pair, bool swap) {
    uint32_t v[8];
    if (pair) {
#pragma unroll
        for (int c = 0; c < 8; ++c) v[c] = *reinterpret_cast<const uint32_t*>(src + c * channel_pitch);
        const uint32_t sel_a = swap ? 0x7632u : 0x5410u;   // low halves = the pair's first pixel, high halves = its second
        const uint32_t sel_b = swap ? 0x5410u : 0x7632u;
        const int off = swap ? 16 : 0;
        *reinterpret_cast<uint4*>(dst + off) = make_uint4(__byte_perm(v[0], v[1], sel_a), __byte_perm(v[2], v[3], sel_a),
                                                          __byte_perm(v[4], v[5], sel_a), __byte_perm(v[6], v[7], sel_a));
        *reinterpret_cast<uint4*>(dst + (off ^ 16)) = make_uint4(__byte_perm(v[0], v[1], sel_b), __byte_perm(v[2], v[3], sel_b),
                                                                 __byte_perm(v[4], v[5], sel_b), __byte_perm(v[6], v[7], sel_b));
    } else {
#pragma unroll
        for (int c = 0; c < 8; ++c) v[c] = *reinterpret_cast<const uint16_t*>(src + c * channel_pitch);
        *reinterpret_cast<uint4*>(dst) = make_uint4(__byte_perm(v[0], v[1], 0x5410u), __byte_perm(v[2], v[3], 0x5410u),
                                                    __byte_perm(v[4], v[5], 0x5410u), __byte_perm(v[6], v[7], 0x5410u));
    }
}

template <bool kBf16>
__global__ void __launch_bounds__(kStagedThreads, 1) conv3x3_staged_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_y, const Params p) {
    extern __shared__ uint8_t smem_dyn[];
    uint8_t* const smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t* const weight_smem = smem;
    uint8_t* const out_smem = smem + p.weight_slots * kWeightStageBytes;   // images of 128 channels x 32 pixels, kOutImages per half of the epilogue warps
    uint8_t* const act_smem = out_smem + 2 * kOutImages * kOutImageBytes;
    uint8_t* const staging_smem = act_smem + p.rec_slots * p.act_stage_bytes;
    uint64_t* const bars = reinterpret_cast<uint64_t*>(staging_smem + p.raw_slots * p.staging_bytes);
    uint64_t* const weight_full = bars;                        // TMA: a group's weights have landed
    uint64_t* const weight_empty = weight_full + kMaxSlots;    // MMA commit: every tile of the step has used them
    uint64_t* const raw_full = weight_empty + kMaxSlots;       // TMA: a raw halo tile has landed
    uint64_t* const raw_empty = raw_full + kMaxSlots;          // re-layout warps: it has been read
    uint64_t* const rec_full = raw_empty + kMaxSlots;          // re-layout warps: the pixel records are written
    uint64_t* const rec_empty = rec_full + kMaxSlots;          // MMA commit: the records have been read
    uint64_t* const tmem_full = rec_empty + kMaxSlots;
    uint64_t* const tmem_empty = tmem_full + 2;
    uint32_t* const tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
    volatile uint32_t* const abort_flag = tmem_slot + 1;

    const int warp = static_cast<int>(threadIdx.x) / 32;
    const int lane = static_cast<int>(threadIdx.x) % 32;
    const WaitGuard guard{abort_flag, g_status};
    const uint32_t weight_slots = static_cast<uint32_t>(p.weight_slots);
    const uint32_t raw_slots = static_cast<uint32_t>(p.raw_slots);
    const uint32_t rec_slots = static_cast<uint32_t>(p.rec_slots);

    if (threadIdx.x == 0) {
        *abort_flag = 0u;
        for (int s = 0; s < kMaxSlots; ++s) {
            mbar_init(&weight_full[s], 1);
            mbar_init(&weight_empty[s], 1);
            mbar_init(&raw_full[s], 1);
            mbar_init(&raw_empty[s], kGatherWarps);
            mbar_init(&rec_full[s], kGatherWarps);
            mbar_init(&rec_empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&tmem_full[s], 1);
            mbar_init(&tmem_empty[s], kStagedEpilogueWarps);
        }
        mbar_init_fence();
        tma_prefetch_desc(&map_w);
        tma_prefetch_desc(&map_x);
        tma_prefetch_desc(&map_y);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 2 * kAccColumns);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    const int per_m = p.B * p.tiles_h * p.tiles_w;
    const TileRange range = tile_range(p.tiles_m * per_m, static_cast<int>(blockIdx.x), static_cast<int>(gridDim.x));
    const int halo_cols = p.bn + 2;
    const int halo_rows = p.rows + 2;
    const int plane_bytes = halo_rows * halo_cols * 16;
    // the raw tile of a slot is one box of bn + 16 pixels per row, or for 256-pixel segments two boxes of 136 side by side
    const int boxes = p.bn > 128 ? 2 : 1;
    const int box_w = (p.bn + 16) / boxes;
    const int box_bytes = 16 * halo_rows * box_w * 2;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (weights and raw halo tiles)
        if (elect_one()) {
            uint32_t w_it = 0, a_it = 0;
            bool ok = true;
            for (int tile = range.begin; ok && tile < range.end;) {
                const int n = tiles_of_step(tile, range.end, per_m);
                const TileCoord tc[2] = {staged_tile_coord(p, tile, per_m), staged_tile_coord(p, tile + n - 1, per_m)};
                for (int g = 0; ok && g < p.groups; ++g, ++w_it) {
                    const uint32_t ws = w_it % weight_slots;
                    ok = guard.wait(&weight_empty[ws], ((w_it / weight_slots) & 1u) ^ 1u, kSiteLoadEmpty);
                    if (!ok) break;
                    mbar_arrive_expect_tx(&weight_full[ws], kWeightStageBytes);
                    tma_load_2d(weight_smem + ws * kWeightStageBytes, &map_w, &weight_full[ws], tc[0].m0 * 2, g * kWeightRows);
                    for (int s = 0; s < n; ++s, ++a_it) {
                        const uint32_t rs = a_it % raw_slots;
                        ok = guard.wait(&raw_empty[rs], ((a_it / raw_slots) & 1u) ^ 1u, kSiteLoadEmpty, 1);
                        if (!ok) break;
                        mbar_arrive_expect_tx(&raw_full[rs], boxes * box_bytes);
                        for (int b = 0; b < boxes; ++b) {
                            tma_load_4d(staging_smem + rs * p.staging_bytes + b * box_bytes, &map_x, &raw_full[rs], tc[s].w0 - 8 + b * box_w, tc[s].h0 - 1, g * 16, tc[s].b);
                        }
                    }
                }
                tile += n;
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (elect_one()) {
            uint32_t w_it = 0, a_it = 0;
            uint32_t q = 0;   // tiles this CTA has started: tile q accumulates in buffer q & 1, the buffer's use number is q >> 1
            bool ok = true;
            for (int tile = range.begin; ok && tile < range.end;) {
                const int n = tiles_of_step(tile, range.end, per_m);
                for (int g = 0; ok && g < p.groups; ++g, ++w_it) {
                    const uint32_t ws = w_it % weight_slots;
                    ok = guard.wait(&weight_full[ws], (w_it / weight_slots) & 1u, kSiteLoadFull);
                    if (!ok) break;
                    const uint64_t desc_w0 = make_smem_desc(smem_u32(weight_smem + ws * kWeightStageBytes), kBlockM * 16, 128, kSwizzleNone);
                    for (int s = 0; s < n; ++s, ++a_it) {
                        const uint32_t acc = (q + s) & 1u;
                        if (g == 0) {
                            ok = guard.wait(&tmem_empty[acc], (((q + s) >> 1) & 1u) ^ 1u, kSiteTmemEmpty);
                            if (!ok) break;
                        }
                        const uint32_t cs = a_it % rec_slots;
                        ok = guard.wait(&rec_full[cs], (a_it / rec_slots) & 1u, kSiteOperandFull);
                        if (!ok) break;
                        tc_fence_after_sync();
                        const uint32_t tmem_d = tmem_base + acc * kAccColumns;
                        // the start address sits in the low bits of a descriptor in 16-byte units: a tap is an addition
                        const uint64_t desc_x0 = make_smem_desc(smem_u32(act_smem + cs * p.act_stage_bytes), plane_bytes, 128, kSwizzleNone);
#pragma unroll
                        for (int tap = 0; tap < 9; ++tap) {
                            const int kh = tap / 3;
                            const int kw = tap % 3;
                            const uint64_t desc_w = desc_w0 + static_cast<uint64_t>(tap * 2 * kBlockM);
                            for (int r = 0; r < p.rows; ++r) {
                                const uint64_t desc_x = desc_x0 + static_cast<uint64_t>((r + kh) * halo_cols + kw);
                                umma_f16(tmem_d + r * p.bn, desc_w, desc_x, p.idesc, (g | tap) != 0 ? 1u : 0u);
                            }
                        }
                        umma_commit(&rec_empty[cs]);
                        // the first tile of a step finishes one tile's worth of UMMAs before the second: its epilogue runs meanwhile
                        if (g == p.groups - 1) umma_commit(&tmem_full[acc]);
                    }
                    if (!ok) break;
                    umma_commit(&weight_empty[ws]);
                }
                q += static_cast<uint32_t>(n);
                tile += n;
            }
        }
    } else if (warp < kStagedFirstGatherWarp) {
        // ------------------------------------------------------------------ epilogue
        const int quarter = warp % 4;                            // the lane quarter of tensor memory this warp may read
        const int half = (warp - kFirstEpilogueWarp) / 4;        // which half of a tile's chunks it takes
        uint32_t stores = 0;                                     // bulk stores of this warp so far
        uint32_t q = 0;
        bool ok = true;
        for (int tile = range.begin; ok && tile < range.end; ++tile, ++q) {
            const TileCoord tc = staged_tile_coord(p, tile, per_m);
            const uint32_t acc = q & 1u;
            ok = guard.wait(&tmem_full[acc], (q >> 1) & 1u, kSiteTmemFull);
            if (!ok) break;
            tc_fence_after_sync();
            const int co = tc.m0 + quarter * 32 + lane;
            const bool co_live = co < p.C_out;
            const float bias = (p.bias != nullptr && co_live) ? bits_to_float<kBf16>(__ldg(p.bias + co)) : 0.0f;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * kAccColumns;
            const int chunks = p.bn / 32;                       // per output row; rows * chunks is even
            const int mine = p.rows * chunks / 2;
            uint8_t* const images = out_smem + half * kOutImages * kOutImageBytes;
            const int twist = (lane >> 1) & 3;                   // the 64-byte swizzle of the tensor map: 16-byte chunk ^= bits 7..8 of the offset
#pragma unroll 1
            for (int i = half * mine; i < (half + 1) * mine; ++i) {
                const int r = i / chunks;
                const int c = i % chunks;
                const int h = tc.h0 + r;
                uint32_t v[32];
                tmem_ld_32x32(taddr + r * p.bn + c * 32, v);
                tmem_wait_ld();
                if (i == (half + 1) * mine - 1) {
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&tmem_empty[acc]);
                }
                if (h >= p.H || tc.w0 + c * 32 >= p.W) continue;   // uniform over the four warps of this half
                // A lane storing its channel's pixels straight to global memory makes every warp store 32 requests of 16
                // bytes. Instead a warp lays its 32 channels x 32 pixels into a shared-memory image (64-byte rows, swizzled
                // so that a quarter warp covers all banks) and its first lane hands it to the copy engine, which also clips
                // at the image edge and at C_out. One image per warp (of two used alternately): the warps of a half never
                // wait for one another, only a lane for the copy engine's read of its own store before last.
                const uint32_t img = stores % kOutImages;       // this store's image
                if (stores >= kOutImages) {
                    if (lane == 0) tma_store_wait_read<kOutImages - 1>();   // all but this lane's newest stores have been read: this image's last one too
                    __syncwarp();
                }
                uint8_t* const image = images + img * kOutImageBytes + quarter * (32 * 64);   // this warp's 32 channels
                uint8_t* const image_row = image + lane * 64;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    uint32_t o[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        o[e] = pack_out<kBf16>(__uint_as_float(v[j * 8 + 2 * e]) + bias, __uint_as_float(v[j * 8 + 2 * e + 1]) + bias);
                    }
                    *reinterpret_cast<uint4*>(image_row + ((j ^ twist) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    tma_store_4d(&map_y, image, tc.w0 + c * 32, h, tc.m0 + quarter * 32, tc.b);
                    tma_store_commit();
                }
                ++stores;
            }
        }
        if (lane == 0) tma_store_wait<0>();   // the image must outlive the copy engine's reads, and the stores the kernel
    } else {
        // ------------------------------------------------------------------ re-layout warps
        // A raw box is [16 channels][halo_rows][box_w pixels]; halo column hc is staged pixel hc + 7 (pixel i of the tile's
        // staged row sits in box i / box_w). An item is a pixel pair (halo columns 1 + 2 e and 2 + 2 e: a 4-byte aligned
        // load per channel, never across two boxes) or one of the two edge pixels, for one 8-channel plane: eight loads, a
        // byte permute, one or two 16-byte record stores. The geometry does not depend on the tile (the TMA unit has
        // done the clipping and the zero fill), so it is decoded once.
        const int t = static_cast<int>(threadIdx.x) - kStagedFirstGatherWarp * 32;
        constexpr int kGatherThreads = kGatherWarps * 32;
        const int per_row = p.bn / 2 + 2;
        const int items = 2 * halo_rows * per_row;
        const int channel_pitch = halo_rows * box_w * 2;   // bytes between the same pixel of consecutive channels
        int src_off[kStagedItems];
        int dst_off[kStagedItems];
        uint32_t pair_mask = 0;
#pragma unroll
        for (int j = 0; j < kStagedItems; ++j) {
            const int item = t + j * kGatherThreads;
            src_off[j] = 0;
            dst_off[j] = -1;
            if (item < items) {
                const int plane = item / (halo_rows * per_row);
                const int rem = item % (halo_rows * per_row);
                const int hr = rem / per_row;
                const int e = rem % per_row;
                const bool pair = e < p.bn / 2;
                const int hc = pair ? 1 + 2 * e : (e == p.bn / 2 ? 0 : p.bn + 1);
                const int staged = hc + 7;
                src_off[j] = (staged / box_w) * box_bytes + plane * 8 * channel_pitch + (hr * box_w + staged % box_w) * 2;
                dst_off[j] = plane * plane_bytes + (hr * halo_cols + hc) * 16;
                if (pair) pair_mask |= 1u << j;
            }
        }
        // one raw tile per (tile, group), in the producer's order: the ring positions are all the re-layout needs
        const uint32_t steps = static_cast<uint32_t>(range.end - range.begin) * static_cast<uint32_t>(p.groups);
        for (uint32_t a_it = 0; a_it < steps; ++a_it) {
            const uint32_t rs = a_it % raw_slots;
            const uint32_t cs = a_it % rec_slots;
            if (!guard.wait(&raw_full[rs], (a_it / raw_slots) & 1u, kSiteLoadFull, 3)) break;
            if (!guard.wait(&rec_empty[cs], ((a_it / rec_slots) & 1u) ^ 1u, kSiteOperandEmpty)) break;
            const uint8_t* const src = staging_smem + rs * p.staging_bytes;
            uint8_t* const dst = act_smem + cs * p.act_stage_bytes;
#pragma unroll
            for (int j = 0; j < kStagedItems; ++j) {
                if (dst_off[j] >= 0) relayout_item(src + src_off[j], dst + dst_off[j], channel_pitch, ((pair_mask >> j) & 1u) != 0, (lane & 4) != 0);
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&rec_full[cs]);
                mbar_arrive(&raw_empty[rs]);   // every lane's loads have returned: their values went into the stores above
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
        tmem_dealloc(tmem_base, 2 * kAccColumns);
    }
}

// The prepacked weight as a 2-D array of 8-byte words: x = 2 words per output channel (its eight input
// channels of one row), y = prepack row. A box of 256 words x 18 rows is the group's tile for 128 output
// channels, every box row one contiguous 2 KB run. (Described as [8 elements][C_out][rows] with 16-byte box
// rows, the copy engine fetched a 32-byte sector and spent one row slot per output channel: twice the L2
// traffic and most of the time of a group.)
inline bool encode_weight_map(CUtensorMap* map, const void* wp, int C_out, int groups) {
    const uint64_t dims[2] = {static_cast<uint64_t>(C_out) * 2, static_cast<uint64_t>(groups) * kWeightRows};
    const uint64_t strides[1] = {static_cast<uint64_t>(C_out) * 16};
    const uint32_t box[2] = {2 * kBlockM, kWeightRows};
    return encode_map(map, CU_TENSOR_MAP_DATA_TYPE_INT64, 2, wp, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE);
}

// The NCHW input as a 4-D tensor [W][H][C_in][B] with a box of `box_w` pixels x `box_h` rows x 16 channels of one image:
// what the staged kernels fetch per 16-channel group. Coordinates outside the image (the padding ring, the rounded-up
// box, channels past C_in) read as zero. Needs W % 8 == 0 (strides are multiples of 16 bytes).
// The NCHW output as a 4-D tensor [W][H][C_out][B] with a box of 32 pixels x 32 channels (one epilogue warp's) of one row and image, 64-byte
// swizzle (the image rows in shared memory are 64 bytes): what the staged kernels' epilogues store. The copy engine
// clips the box at W and at C_out. Needs W % 8 == 0.
inline bool encode_output_map(CUtensorMap* map, void* y, int B, int C_out, int H, int W, bool bf16) {
    const uint64_t dims[4] = {static_cast<uint64_t>(W), static_cast<uint64_t>(H), static_cast<uint64_t>(C_out), static_cast<uint64_t>(B)};
    const uint64_t strides[3] = {static_cast<uint64_t>(W) * 2, static_cast<uint64_t>(H) * W * 2, static_cast<uint64_t>(C_out) * H * W * 2};
    const uint32_t box[4] = {32u, 1u, 32u, 1u};   // one epilogue warp's 32 channels
    return encode_map(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, y, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B);
}

inline bool encode_input_map(CUtensorMap* map, const void* x, int B, int C_in, int H, int W, int box_w, int box_h, bool bf16) {
    const uint64_t dims[4] = {static_cast<uint64_t>(W), static_cast<uint64_t>(H), static_cast<uint64_t>(C_in), static_cast<uint64_t>(B)};
    const uint64_t strides[3] = {static_cast<uint64_t>(W) * 2, static_cast<uint64_t>(H) * W * 2, static_cast<uint64_t>(C_in) * H * W * 2};
    const uint32_t box[4] = {static_cast<uint32_t>(box_w), static_cast<uint32_t>(box_h), 16u, 1u};
    return encode_map(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, x, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE);
}

// FEATHER_CONV_STAGING_OFF=1 keeps the gather from global memory for every shape (A/B measurements). Read once per process.
inline bool staging_off() {
    static const bool off = env_switch("FEATHER_CONV_STAGING_OFF");
    return off;
}

// ---------------------------------------------------------------------------------------------------------
// CTA-pair version (tcgen05 cta_group::2) for C_out > 128: a cluster of two CTAs owns 256 output channels x
// two output rows x 128 pixels. CTA r loads the weights of output channels [128 r, +128) and gathers the
// halo tile (3 rows x 130 columns) of output row h0 + r; the UMMA (M = 256, N = 256, K = 16) is issued by
// CTA 0, takes the 128 pixels of each CTA as one half of its N extent and leaves 128 channels x 256 pixels in
// each CTA's tensor memory (columns 0..127: row h0, 128..255: row h0 + 1). Against the one-CTA kernel with the
// same tile, every SM gathers 3 halo rows instead of 4 per 256 pixels, the UMMA reads half as much shared
// memory per flop (the measured limiter of the one-CTA kernel), and the 256-wide UMMA spends a smaller share
// of its time loading the weight operand (162 clocks per 128 x 256 x 16 against 2 x 98 for two 128-wide ones).
// ---------------------------------------------------------------------------------------------------------
constexpr int kPairBN = 128;                       // pixels per CTA (one output row segment)
constexpr int kPairHaloCols = kPairBN + 2;
constexpr int kPairHaloRows = 3;
constexpr int kPairPlaneBytes = kPairHaloRows * kPairHaloCols * 16;
constexpr int kPairActStageBytes = (2 * kPairPlaneBytes + 127) / 128 * 128;
constexpr int kPairStagedCols = kPairBN + 16;      // staged halo rows start eight pixels left of the tile (16-byte rule) and are sixteen wider
constexpr int kPairStagingBytes = 16 * kPairHaloRows * kPairStagedCols * 2;
static_assert(kPairStagingBytes % 128 == 0, "staging slots must keep the 128-byte alignment of TMA destinations");

// Gathering from global memory: four slots, four teams of gather warps taking the 16-channel groups in turn, so that
// four groups' loads are in flight (2 teams: 1.19, 4: 1.24 PFLOP/s). Ring depth = team count: a team always meets the
// same slot and sees every phase of its barriers.
constexpr int kPairStages = 4;
constexpr int kPairTeams = 4;
constexpr int kPairTeamWarps = kGatherWarps / kPairTeams;
constexpr int kPairItems = (2 * kPairHaloRows * (kPairBN / 2 + 2) + kPairTeamWarps * 32 - 1) / (kPairTeamWarps * 32);   // gather items per thread per slot
constexpr int kPairSmemBytes = kPairStages * (kWeightStageBytes + kPairActStageBytes) + (3 * kPairStages + 4) * 8 + 16 + 1024;
static_assert(kPairStages % kPairTeams == 0, "ring depth must be a multiple of the team count");
static_assert(kPairSmemBytes <= 227 * 1024, "a CTA's shared memory");

template <bool kBf16>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
conv3x3_pair_kernel(const __grid_constant__ CUtensorMap map_w, const Params p) {
    extern __shared__ uint8_t smem_dyn[];
    uint8_t* const smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t* const weight_smem = smem;
    uint8_t* const act_smem = smem + kPairStages * kWeightStageBytes;
    uint64_t* const bars = reinterpret_cast<uint64_t*>(act_smem + kPairStages * kPairActStageBytes);
    uint64_t* const weight_full = bars;                        // local: this CTA's weight rows have landed
    uint64_t* const act_full = weight_full + kPairStages;      // CTA 0 only: both CTAs' gather warps arrive here
    uint64_t* const stage_empty = act_full + kPairStages;      // signalled in both CTAs by CTA 0's commits
    uint64_t* const tmem_full = stage_empty + kPairStages;
    uint64_t* const tmem_empty = tmem_full + 2;                // CTA 0 only
    uint32_t* const tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
    volatile uint32_t* const abort_flag = tmem_slot + 1;

    const int warp = static_cast<int>(threadIdx.x) / 32;
    const int lane = static_cast<int>(threadIdx.x) % 32;
    const uint32_t cta = cluster_cta_rank();
    const WaitGuard guard{abort_flag, g_status};

    if (threadIdx.x == 0) {
        *abort_flag = 0u;
        for (int s = 0; s < kPairStages; ++s) {
            mbar_init(&weight_full[s], 1);
            // a gather warp arrives only after its own CTA's weights have landed, so this one barrier tells the
            // MMA thread that both CTAs' operands of the slot are complete
            mbar_init(&act_full[s], 2 * kPairTeamWarps);
            mbar_init(&stage_empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&tmem_full[s], 1);
            mbar_init(&tmem_empty[s], 2 * kEpilogueWarps);
        }
        mbar_init_fence();
        tma_prefetch_desc(&map_w);
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, 2 * kAccColumns);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    // tiles: output-channel pairs fastest, then pixel segments, then row pairs, then images
    const int tiles_m = (p.C_out + 2 * kBlockM - 1) / (2 * kBlockM);
    const int tiles_w = (p.W + kPairBN - 1) / kPairBN;
    const int tiles_h = (p.H + 1) / 2;
    const int num_tiles = p.B * tiles_m * tiles_h * tiles_w;
    const int first_tile = static_cast<int>(blockIdx.x) / 2;
    const int tile_step = static_cast<int>(gridDim.x) / 2;
    auto coord = [&](int tile) {
        TileCoord t;
        t.m0 = (tile % tiles_m) * 2 * kBlockM + static_cast<int>(cta) * kBlockM;
        tile /= tiles_m;
        t.w0 = (tile % tiles_w) * kPairBN;
        tile /= tiles_w;
        t.h0 = (tile % tiles_h) * 2;
        t.b = tile / tiles_h;
        return t;
    };

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (this CTA's weight rows)
        if (elect_one()) {
            uint32_t it = 0;
            bool ok = true;
            for (int tile = first_tile; ok && tile < num_tiles; tile += tile_step) {
                const TileCoord tc = coord(tile);
                for (int g = 0; g < p.groups; ++g, ++it) {
                    const uint32_t s = it % kPairStages;
                    const uint32_t phase = (it / kPairStages) & 1u;
                    ok = guard.wait(&stage_empty[s], phase ^ 1u, kSiteLoadEmpty);
                    if (!ok) break;
                    mbar_arrive_expect_tx(&weight_full[s], kWeightStageBytes);
                    tma_load_2d(weight_smem + s * kWeightStageBytes, &map_w, &weight_full[s], tc.m0 * 2, g * kWeightRows);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (CTA 0 of the pair)
        if (cta == 0 && elect_one()) {
            uint32_t it = 0;
            uint32_t acc_it = 0;
            bool ok = true;
            for (int tile = first_tile; ok && tile < num_tiles; tile += tile_step, ++acc_it) {
                const uint32_t acc = acc_it & 1u;
                ok = guard.wait(&tmem_empty[acc], ((acc_it >> 1) & 1u) ^ 1u, kSiteTmemEmpty);
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t tmem_d = tmem_base + acc * kAccColumns;
                for (int g = 0; g < p.groups; ++g, ++it) {
                    const uint32_t s = it % kPairStages;
                    const uint32_t phase = (it / kPairStages) & 1u;
                    ok = guard.wait(&act_full[s], phase, kSiteOperandFull);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint64_t desc_w0 = make_smem_desc(smem_u32(weight_smem + s * kWeightStageBytes), kBlockM * 16, 128, kSwizzleNone);
                    const uint64_t desc_x0 = make_smem_desc(smem_u32(act_smem + s * kPairActStageBytes), kPairPlaneBytes, 128, kSwizzleNone);
#pragma unroll
                    for (int tap = 0; tap < 9; ++tap) {
                        const int kh = tap / 3;
                        const int kw = tap % 3;
                        umma_f16_pair(tmem_d, desc_w0 + static_cast<uint64_t>(tap * 2 * kBlockM),
                                      desc_x0 + static_cast<uint64_t>(kh * kPairHaloCols + kw), p.idesc, (g | tap) != 0 ? 1u : 0u);
                    }
#pragma unroll
                    for (uint32_t dst = 0; dst < 2; ++dst) umma_commit_pair(map_to_cta(smem_u32(&stage_empty[s]), dst));
                }
                if (!ok) break;
#pragma unroll
                for (uint32_t dst = 0; dst < 2; ++dst) umma_commit_pair(map_to_cta(smem_u32(&tmem_full[acc]), dst));
            }
        }
    } else if (warp < kFirstGatherWarp) {
        // ------------------------------------------------------------------ epilogue (this CTA's 128 channels, both rows)
        const int quarter = warp % 4;
        const bool vector_rows = (p.W % 8) == 0;
        uint32_t acc_it = 0;
        bool ok = true;
        for (int tile = first_tile; ok && tile < num_tiles; tile += tile_step, ++acc_it) {
            const TileCoord tc = coord(tile);
            const uint32_t acc = acc_it & 1u;
            ok = guard.wait(&tmem_full[acc], (acc_it >> 1) & 1u, kSiteTmemFull);
            if (!ok) break;
            tc_fence_after_sync();
            const int co = tc.m0 + quarter * 32 + lane;
            const bool co_live = co < p.C_out;
            const float bias = (p.bias != nullptr && co_live) ? bits_to_float<kBf16>(__ldg(p.bias + co)) : 0.0f;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * kAccColumns;
            constexpr int kChunks = kPairBN / 32;
#pragma unroll 1
            for (int r = 0; r < 2; ++r) {
                const int h = tc.h0 + r;
                uint16_t* const y_row = p.y + ((static_cast<int64_t>(tc.b) * p.C_out + (co_live ? co : 0)) * p.H + (h < p.H ? h : 0)) * p.W;
#pragma unroll 1
                for (int c = 0; c < kChunks; ++c) {
                    uint32_t v[32];
                    tmem_ld_32x32(taddr + r * kPairBN + c * 32, v);
                    tmem_wait_ld();
                    if (r == 1 && c == kChunks - 1) {
                        tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tmem_empty[acc]), 0));
                    }
                    if (!co_live || h >= p.H) continue;
                    store_pixels<kBf16>(v, bias, y_row, tc.w0 + c * 32, p.W, vector_rows);
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ activation gather warps (output row h0 + cta)
        // W is even here (the launcher checks): per (plane, halo row) the halo columns 1..128 as 64 aligned pixel
        // pairs, then the edge columns 0 and 129 as single pixels.
        const int team = (warp - kFirstGatherWarp) / kPairTeamWarps;
        const int t = static_cast<int>(threadIdx.x) - (kFirstGatherWarp + team * kPairTeamWarps) * 32;
        constexpr int kTeamThreads = kPairTeamWarps * 32;
        constexpr int kPerRow = kPairBN / 2 + 2;
        constexpr int kItems = 2 * kPairHaloRows * kPerRow;
        static_assert(kItems <= kPairItems * kTeamThreads, "the halo tile must fit the per-thread item count");
        const int64_t hw = static_cast<int64_t>(p.H) * p.W;
        uint32_t it = 0;
        bool ok = true;
        for (int tile = first_tile; ok && tile < num_tiles; tile += tile_step) {
            const TileCoord tc = coord(tile);
            const uint16_t* const x_img = p.x + static_cast<int64_t>(tc.b) * p.C_in * hw;
            int64_t src_off[kPairItems];
            int dst_off[kPairItems];
            uint32_t kinds = 0;  // 4 bits per item: kind (1 single, 2 pair) | in_image << 2 | plane << 3
#pragma unroll
            for (int j = 0; j < kPairItems; ++j) {
                const int item = t + j * kTeamThreads;
                src_off[j] = 0;
                dst_off[j] = -1;
                if (item < kItems) {
                    const int plane = item / (kPairHaloRows * kPerRow);
                    const int rem = item % (kPairHaloRows * kPerRow);
                    const int hr = rem / kPerRow;
                    const int e = rem % kPerRow;
                    const bool pair = e < kPairBN / 2;
                    const int hc = pair ? 1 + 2 * e : (e == kPairBN / 2 ? 0 : kPairBN + 1);
                    const int h = tc.h0 + static_cast<int>(cta) - 1 + hr;
                    const int w = tc.w0 - 1 + hc;
                    const bool in_image = h >= 0 && h < p.H && w >= 0 && w < p.W;
                    src_off[j] = static_cast<int64_t>(plane) * 8 * hw + static_cast<int64_t>(in_image ? h : 0) * p.W + (in_image ? w : 0);
                    dst_off[j] = plane * kPairPlaneBytes + (hr * kPairHaloCols + hc) * 16;
                    kinds |= ((pair ? 2u : 1u) | (in_image ? 4u : 0u) | (plane ? 8u : 0u)) << (4 * j);
                }
            }
            for (int g = 0; g < p.groups; ++g, ++it) {
                if (static_cast<int>(it % kPairTeams) != team) continue;
                const uint32_t s = it % kPairStages;
                const uint32_t phase = (it / kPairStages) & 1u;
                const uint16_t* const x_group = x_img + static_cast<int64_t>(g) * 16 * hw;
                const bool second_plane_live = g * 16 + 8 < p.C_in;
                uint32_t v[kPairItems][8];
#pragma unroll
                for (int j = 0; j < kPairItems; ++j) {
                    const uint32_t k = (kinds >> (4 * j)) & 15u;
                    const bool live = (k & 4u) != 0 && ((k & 8u) == 0 || second_plane_live);
                    const uint16_t* const src = x_group + src_off[j];
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        if ((k & 2u) != 0) {
                            v[j][c] = live ? __ldg(reinterpret_cast<const uint32_t*>(src + c * hw)) : 0u;
                        } else {
                            v[j][c] = live ? static_cast<uint32_t>(__ldg(src + c * hw)) : 0u;
                        }
                    }
                }
                ok = guard.wait(&stage_empty[s], phase ^ 1u, kSiteOperandEmpty);
                if (!ok) break;
                uint8_t* const dst = act_smem + s * kPairActStageBytes;
#pragma unroll
                for (int j = 0; j < kPairItems; ++j) {
                    if (dst_off[j] < 0) continue;
                    const uint4 first = make_uint4(__byte_perm(v[j][0], v[j][1], 0x5410u), __byte_perm(v[j][2], v[j][3], 0x5410u),
                                                   __byte_perm(v[j][4], v[j][5], 0x5410u), __byte_perm(v[j][6], v[j][7], 0x5410u));
                    *reinterpret_cast<uint4*>(dst + dst_off[j]) = first;
                    if (((kinds >> (4 * j)) & 2u) != 0) {
                        const uint4 second = make_uint4(__byte_perm(v[j][0], v[j][1], 0x7632u), __byte_perm(v[j][2], v[j][3], 0x7632u),
                                                        __byte_perm(v[j][4], v[j][5], 0x7632u), __byte_perm(v[j][6], v[j][7], 0x7632u));
                        *reinterpret_cast<uint4*>(dst + dst_off[j] + 16) = second;
                    }
                }
                fence_proxy_async_smem();
                // this CTA's weight rows of the slot must have landed before the slot is published to the MMA thread
                ok = guard.wait(&weight_full[s], phase, kSiteLoadFull, 2);
                if (!ok) break;
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&act_full[s]), 0));
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
        tmem_dealloc_pair(tmem_base, 2 * kAccColumns);
    }
}

// Staged CTA-pair kernel: the pair kernel's tile (256 output channels x 2 rows x 128 pixels, `cta_group::2` UMMAs of
// 256 x 256 x 16) with the halo tiles by TMA and two tiles per weight slot, as in conv3x3_staged_kernel. CTA r loads
// the weight rows of its 128 channels and the raw halo tile of its output row h0 + r. The MMA thread (CTA 0) waits on
// one barrier per halo slot: a re-layout warp of either CTA arrives there only after its own CTA's weights of the step
// have landed too, so the barrier tells that both CTAs' operands are complete.
constexpr int kPairWeightSlots = 3;
constexpr int kPairActSlots = 3;
constexpr int kPairStagedItems = (2 * kPairHaloRows * (kPairBN / 2 + 2) + kGatherWarps * 32 - 1) / (kGatherWarps * 32);
constexpr int kPairStagedSmemBytes = kPairWeightSlots * kWeightStageBytes + 2 * kOutImages * kOutImageBytes + kPairActSlots * (kPairActStageBytes + kPairStagingBytes) +
                                     (2 * kPairWeightSlots + 3 * kPairActSlots + 4) * 8 + 16 + 1024;
static_assert(kPairStagedSmemBytes <= 227 * 1024, "a CTA's shared memory");

template <bool kBf16>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kStagedThreads, 1)
conv3x3_pair_staged_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_y, const Params p) {
    extern __shared__ uint8_t smem_dyn[];
    uint8_t* const smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t* const weight_smem = smem;
    uint8_t* const out_smem = smem + kPairWeightSlots * kWeightStageBytes;   // images of 128 channels x 32 pixels, kOutImages per output row
    uint8_t* const act_smem = out_smem + 2 * kOutImages * kOutImageBytes;
    uint8_t* const staging_smem = act_smem + kPairActSlots * kPairActStageBytes;
    uint64_t* const bars = reinterpret_cast<uint64_t*>(staging_smem + kPairActSlots * kPairStagingBytes);
    uint64_t* const weight_full = bars;                             // local: this CTA's weight rows have landed
    uint64_t* const weight_empty = weight_full + kPairWeightSlots;  // signalled in both CTAs by CTA 0's commits
    uint64_t* const raw_full = weight_empty + kPairWeightSlots;     // local: this CTA's raw halo tile has landed
    uint64_t* const act_full = raw_full + kPairActSlots;            // CTA 0 only: both CTAs' re-layout warps arrive here
    uint64_t* const act_empty = act_full + kPairActSlots;           // signalled in both CTAs by CTA 0's commits
    uint64_t* const tmem_full = act_empty + kPairActSlots;
    uint64_t* const tmem_empty = tmem_full + 2;                     // CTA 0 only
    uint32_t* const tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
    volatile uint32_t* const abort_flag = tmem_slot + 1;

    const int warp = static_cast<int>(threadIdx.x) / 32;
    const int lane = static_cast<int>(threadIdx.x) % 32;
    const uint32_t cta = cluster_cta_rank();
    const WaitGuard guard{abort_flag, g_status};

    if (threadIdx.x == 0) {
        *abort_flag = 0u;
        for (int s = 0; s < kPairWeightSlots; ++s) {
            mbar_init(&weight_full[s], 1);
            mbar_init(&weight_empty[s], 1);
        }
        for (int s = 0; s < kPairActSlots; ++s) {
            mbar_init(&raw_full[s], 1);
            mbar_init(&act_full[s], 2 * kGatherWarps);
            mbar_init(&act_empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&tmem_full[s], 1);
            mbar_init(&tmem_empty[s], 2 * kStagedEpilogueWarps);
        }
        mbar_init_fence();
        tma_prefetch_desc(&map_w);
        tma_prefetch_desc(&map_x);
        tma_prefetch_desc(&map_y);
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, 2 * kAccColumns);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    // tile list: pixel segments fastest, then row pairs, images, and the 256-channel tile slowest
    const int tiles_w = (p.W + kPairBN - 1) / kPairBN;
    const int tiles_h = (p.H + 1) / 2;
    const int per_m = p.B * tiles_h * tiles_w;
    const int tiles_m = (p.C_out + 2 * kBlockM - 1) / (2 * kBlockM);
    const TileRange range = tile_range(tiles_m * per_m, static_cast<int>(blockIdx.x) / 2, static_cast<int>(gridDim.x) / 2);
    auto coord = [&](int tile) {
        TileCoord t;
        t.m0 = (tile / per_m) * 2 * kBlockM + static_cast<int>(cta) * kBlockM;
        tile %= per_m;
        t.w0 = (tile % tiles_w) * kPairBN;
        tile /= tiles_w;
        t.h0 = (tile % tiles_h) * 2;
        t.b = tile / tiles_h;
        return t;
    };

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (this CTA's weight rows and raw halo tiles)
        if (elect_one()) {
            uint32_t w_it = 0, a_it = 0;
            bool ok = true;
            for (int tile = range.begin; ok && tile < range.end;) {
                const int n = tiles_of_step(tile, range.end, per_m);
                const TileCoord tc[2] = {coord(tile), coord(tile + n - 1)};
                for (int g = 0; ok && g < p.groups; ++g, ++w_it) {
                    const uint32_t ws = w_it % kPairWeightSlots;
                    ok = guard.wait(&weight_empty[ws], ((w_it / kPairWeightSlots) & 1u) ^ 1u, kSiteLoadEmpty);
                    if (!ok) break;
                    mbar_arrive_expect_tx(&weight_full[ws], kWeightStageBytes);
                    tma_load_2d(weight_smem + ws * kWeightStageBytes, &map_w, &weight_full[ws], tc[0].m0 * 2, g * kWeightRows);
                    for (int s = 0; s < n; ++s, ++a_it) {
                        const uint32_t as = a_it % kPairActSlots;
                        ok = guard.wait(&act_empty[as], ((a_it / kPairActSlots) & 1u) ^ 1u, kSiteLoadEmpty, 1);
                        if (!ok) break;
                        mbar_arrive_expect_tx(&raw_full[as], kPairStagingBytes);
                        // the three halo rows of this CTA's output row h0 + cta, eight pixels to the left for the 16-byte rule
                        tma_load_4d(staging_smem + as * kPairStagingBytes, &map_x, &raw_full[as], tc[s].w0 - 8, tc[s].h0 + static_cast<int>(cta) - 1, g * 16, tc[s].b);
                    }
                }
                tile += n;
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (CTA 0 of the pair)
        if (cta == 0 && elect_one()) {
            uint32_t w_it = 0, a_it = 0;
            uint32_t q = 0;   // tiles this pair has started: tile q accumulates in buffer q & 1, the buffer's use number is q >> 1
            bool ok = true;
            for (int tile = range.begin; ok && tile < range.end;) {
                const int n = tiles_of_step(tile, range.end, per_m);
                for (int g = 0; ok && g < p.groups; ++g, ++w_it) {
                    const uint32_t ws = w_it % kPairWeightSlots;
                    const uint64_t desc_w0 = make_smem_desc(smem_u32(weight_smem + ws * kWeightStageBytes), kBlockM * 16, 128, kSwizzleNone);
                    for (int s = 0; s < n; ++s, ++a_it) {
                        const uint32_t acc = (q + s) & 1u;
                        if (g == 0) {
                            ok = guard.wait(&tmem_empty[acc], (((q + s) >> 1) & 1u) ^ 1u, kSiteTmemEmpty);
                            if (!ok) break;
                        }
                        const uint32_t as = a_it % kPairActSlots;
                        ok = guard.wait(&act_full[as], (a_it / kPairActSlots) & 1u, kSiteOperandFull);
                        if (!ok) break;
                        tc_fence_after_sync();
                        const uint32_t tmem_d = tmem_base + acc * kAccColumns;
                        const uint64_t desc_x0 = make_smem_desc(smem_u32(act_smem + as * kPairActStageBytes), kPairPlaneBytes, 128, kSwizzleNone);
#pragma unroll
                        for (int tap = 0; tap < 9; ++tap) {
                            const int kh = tap / 3;
                            const int kw = tap % 3;
                            umma_f16_pair(tmem_d, desc_w0 + static_cast<uint64_t>(tap * 2 * kBlockM),
                                          desc_x0 + static_cast<uint64_t>(kh * kPairHaloCols + kw), p.idesc, (g | tap) != 0 ? 1u : 0u);
                        }
#pragma unroll
                        for (uint32_t dst = 0; dst < 2; ++dst) umma_commit_pair(map_to_cta(smem_u32(&act_empty[as]), dst));
                        if (g == p.groups - 1) {
#pragma unroll
                            for (uint32_t dst = 0; dst < 2; ++dst) umma_commit_pair(map_to_cta(smem_u32(&tmem_full[acc]), dst));
                        }
                    }
                    if (!ok) break;
#pragma unroll
                    for (uint32_t dst = 0; dst < 2; ++dst) umma_commit_pair(map_to_cta(smem_u32(&weight_empty[ws]), dst));
                }
                q += static_cast<uint32_t>(n);
                tile += n;
            }
        }
    } else if (warp < kStagedFirstGatherWarp) {
        // ------------------------------------------------------------------ epilogue (this CTA's 128 channels; two warps per lane quarter, one output row each)
        const int quarter = warp % 4;
        const int r = (warp - kFirstEpilogueWarp) / 4;
        uint8_t* const images = out_smem + r * kOutImages * kOutImageBytes;
        const int twist = (lane >> 1) & 3;                       // the 64-byte swizzle of the tensor map
        uint32_t stores = 0;                                     // bulk stores of this warp so far
        uint32_t q = 0;
        bool ok = true;
        for (int tile = range.begin; ok && tile < range.end; ++tile, ++q) {
            const TileCoord tc = coord(tile);
            const uint32_t acc = q & 1u;
            ok = guard.wait(&tmem_full[acc], (q >> 1) & 1u, kSiteTmemFull);
            if (!ok) break;
            tc_fence_after_sync();
            const int co = tc.m0 + quarter * 32 + lane;
            const bool co_live = co < p.C_out;
            const float bias = (p.bias != nullptr && co_live) ? bits_to_float<kBf16>(__ldg(p.bias + co)) : 0.0f;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * kAccColumns;
            constexpr int kChunks = kPairBN / 32;
            const int h = tc.h0 + r;
#pragma unroll 1
            for (int c = 0; c < kChunks; ++c) {
                uint32_t v[32];
                tmem_ld_32x32(taddr + r * kPairBN + c * 32, v);
                tmem_wait_ld();
                if (c == kChunks - 1) {
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tmem_empty[acc]), 0));
                }
                if (h >= p.H || tc.w0 + c * 32 >= p.W) continue;   // uniform over the four warps of this row
                // the output goes through a shared-memory image and a bulk tensor store, as in conv3x3_staged_kernel
                const uint32_t img = stores % kOutImages;
                if (stores >= kOutImages) {
                    if (lane == 0) tma_store_wait_read<kOutImages - 1>();
                    __syncwarp();
                }
                uint8_t* const image = images + img * kOutImageBytes + quarter * (32 * 64);   // this warp's 32 channels
                uint8_t* const image_row = image + lane * 64;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    uint32_t o[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        o[e] = pack_out<kBf16>(__uint_as_float(v[j * 8 + 2 * e]) + bias, __uint_as_float(v[j * 8 + 2 * e + 1]) + bias);
                    }
                    *reinterpret_cast<uint4*>(image_row + ((j ^ twist) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    tma_store_4d(&map_y, image, tc.w0 + c * 32, h, tc.m0 + quarter * 32, tc.b);
                    tma_store_commit();
                }
                ++stores;
            }
        }
        if (lane == 0) tma_store_wait<0>();   // the image must outlive the copy engine's reads, and the stores the kernel
    } else {
        // ------------------------------------------------------------------ re-layout warps (output row h0 + cta)
        // From the slot's staging buffer [16 channels][3 halo rows][144 pixels] (halo column hc is staged pixel hc + 7) into
        // the pixel records: per (plane, halo row) the halo columns 1..128 as 64 aligned pixel pairs, then the edge columns
        // 0 and 129 as single pixels. The geometry does not depend on the tile, the TMA unit has done the clipping.
        const int t = static_cast<int>(threadIdx.x) - kStagedFirstGatherWarp * 32;
        constexpr int kGatherThreads = kGatherWarps * 32;
        constexpr int kPerRow = kPairBN / 2 + 2;
        constexpr int kItems = 2 * kPairHaloRows * kPerRow;
        constexpr int kChannelPitch = kPairHaloRows * kPairStagedCols * 2;
        int src_off[kPairStagedItems];
        int dst_off[kPairStagedItems];
        uint32_t pair_mask = 0;
#pragma unroll
        for (int j = 0; j < kPairStagedItems; ++j) {
            const int item = t + j * kGatherThreads;
            src_off[j] = 0;
            dst_off[j] = -1;
            if (item < kItems) {
                const int plane = item / (kPairHaloRows * kPerRow);
                const int rem = item % (kPairHaloRows * kPerRow);
                const int hr = rem / kPerRow;
                const int e = rem % kPerRow;
                const bool pair = e < kPairBN / 2;
                const int hc = pair ? 1 + 2 * e : (e == kPairBN / 2 ? 0 : kPairBN + 1);
                src_off[j] = plane * 8 * kChannelPitch + (hr * kPairStagedCols + hc + 7) * 2;
                dst_off[j] = plane * kPairPlaneBytes + (hr * kPairHaloCols + hc) * 16;
                if (pair) pair_mask |= 1u << j;
            }
        }
        uint32_t w_it = 0, a_it = 0;
        bool ok = true;
        for (int tile = range.begin; ok && tile < range.end;) {
            const int n = tiles_of_step(tile, range.end, per_m);
            for (int g = 0; ok && g < p.groups; ++g, ++w_it) {
                for (int s = 0; s < n; ++s, ++a_it) {
                    const uint32_t as = a_it % kPairActSlots;
                    // this CTA's raw halo tile has landed (the slot's records were last read by UMMAs that completed before the
                    // copy engine was allowed to refill the slot)
                    ok = guard.wait(&raw_full[as], (a_it / kPairActSlots) & 1u, kSiteLoadFull, 3);
                    if (!ok) break;
                    const uint8_t* const src = staging_smem + as * kPairStagingBytes;
                    uint8_t* const dst = act_smem + as * kPairActStageBytes;
#pragma unroll
                    for (int j = 0; j < kPairStagedItems; ++j) {
                        if (dst_off[j] >= 0) relayout_item(src + src_off[j], dst + dst_off[j], kChannelPitch, ((pair_mask >> j) & 1u) != 0, (lane & 4) != 0);
                    }
                    fence_proxy_async_smem();
                    if (s == 0) {
                        // this CTA's weight rows of the step must have landed before its first halo slot is published to the MMA thread
                        ok = guard.wait(&weight_full[w_it % kPairWeightSlots], (w_it / kPairWeightSlots) & 1u, kSiteLoadFull, 2);
                        if (!ok) break;
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&act_full[as]), 0));
                }
            }
            tile += n;
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
        tmem_dealloc_pair(tmem_base, 2 * kAccColumns);
    }
}

// How many CTA pairs of `kernel` fit on the device at once (a persistent grid must be resident as a whole, and a pair needs
// both SMs of a TPC); also raises the kernel's shared-memory limit. 0 on failure.
template <typename Kernel>
int resident_pairs_of(Kernel* kernel, int threads, int smem_bytes) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes) != cudaSuccess) return 0;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(static_cast<unsigned>(device_info().sm_count / 2 * 2));
    config.blockDim = dim3(static_cast<unsigned>(threads));
    config.dynamicSmemBytes = smem_bytes;
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
}

template <bool kBf16>
int launch_pair(const void* x, const void* wp, const void* bias, void* y, int B, int C_in, int C_out, int H, int W, cudaStream_t stream) {
    const bool staged = (W % 8) == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15u) == 0 && !staging_off();
    Params p{};
    p.x = static_cast<const uint16_t*>(x);
    p.bias = static_cast<const uint16_t*>(bias);
    p.y = static_cast<uint16_t*>(y);
    p.B = B;
    p.C_in = C_in;
    p.C_out = C_out;
    p.H = H;
    p.W = W;
    p.groups = (C_in + 15) / 16;
    p.bn = kPairBN;
    p.rows = 2;
    p.idesc = make_idesc(kAccF32, kBf16 ? kFmtBF16 : kFmtF16, kBf16 ? kFmtBF16 : kFmtF16, 2 * kBlockM, 2 * kPairBN);
    p.pairs = 1;

    static PerDeviceState resident_pairs[2];   // once per device and kernel
    const int pairs = staged ? resident_pairs[1].get([&] { return resident_pairs_of(&conv3x3_pair_staged_kernel<kBf16>, kStagedThreads, kPairStagedSmemBytes); })
                             : resident_pairs[0].get([&] { return resident_pairs_of(&conv3x3_pair_kernel<kBf16>, kThreads, kPairSmemBytes); });
    if (pairs <= 0) return 1;

    CUtensorMap map_w;
    if (!encode_weight_map(&map_w, wp, C_out, p.groups)) return 1;
    const int64_t tiles_m = (C_out + 2 * kBlockM - 1) / (2 * kBlockM);
    const int64_t num_tiles = static_cast<int64_t>(B) * tiles_m * ((H + 1) / 2) * ((W + kPairBN - 1) / kPairBN);
    if (num_tiles > (1ll << 30)) return 1;
    const int grid = 2 * static_cast<int>(num_tiles < pairs ? num_tiles : pairs);
    if (staged) {
        CUtensorMap map_x, map_y;
        if (!encode_input_map(&map_x, x, B, C_in, H, W, kPairStagedCols, kPairHaloRows, kBf16)) return 1;
        if (!encode_output_map(&map_y, y, B, C_out, H, W, kBf16)) return 1;
        conv3x3_pair_staged_kernel<kBf16><<<grid, kStagedThreads, kPairStagedSmemBytes, stream>>>(map_w, map_x, map_y, p);
    } else {
        conv3x3_pair_kernel<kBf16><<<grid, kThreads, kPairSmemBytes, stream>>>(map_w, p);
    }
    return cudaGetLastError() == cudaSuccess ? 0 : 1;
}

template <bool kBf16>
int launch(const void* x, const void* wp, const void* bias, void* y, int B, int C_in, int C_out, int H, int W, int bn, int rows,
           cudaStream_t stream) {
    // staged halo tiles need a 16-byte row pitch and a 16-byte aligned input
    const bool staged = (W % 8) == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15u) == 0 && !staging_off();
    Params p{};
    p.x = static_cast<const uint16_t*>(x);
    p.bias = static_cast<const uint16_t*>(bias);
    p.y = static_cast<uint16_t*>(y);
    p.B = B;
    p.C_in = C_in;
    p.C_out = C_out;
    p.H = H;
    p.W = W;
    p.groups = (C_in + 15) / 16;
    p.bn = bn;
    p.rows = rows;
    p.tiles_m = (C_out + kBlockM - 1) / kBlockM;
    p.tiles_w = (W + bn - 1) / bn;
    p.tiles_h = (H + rows - 1) / rows;
    p.act_stage_bytes = ((2 * (rows + 2) * (bn + 2) * 16) + 127) / 128 * 128;
    p.idesc = make_idesc(kAccF32, kBf16 ? kFmtBF16 : kFmtF16, kBf16 ? kFmtBF16 : kFmtF16, kBlockM, bn);
    p.pairs = (W % 2 == 0) ? 1 : 0;
    const int per_row = p.pairs ? bn / 2 + 2 : bn + 2;
    const int items = 2 * (rows + 2) * per_row;
    if (items > (staged ? kStagedItems * kGatherWarps * 32 : kMaxItems * kTeamWarps * 32)) return 1;

    CUtensorMap map_w;
    if (!encode_weight_map(&map_w, wp, C_out, p.groups)) return 1;
    const int64_t num_tiles = static_cast<int64_t>(B) * p.tiles_m * p.tiles_h * p.tiles_w;
    if (num_tiles > (1ll << 30)) return 1;
    const int sms = device_info().sm_count;
    const int grid = num_tiles < sms ? static_cast<int>(num_tiles) : sms;
    static PerDeviceState smem_limit[2];
    if (staged) {
        // a box side is at most 256 elements: a 256-pixel segment takes two boxes of 136 pixels side by side
        const int boxes = bn > 128 ? 2 : 1;
        const int box_w = (bn + 16) / boxes;
        p.staging_bytes = boxes * 16 * (rows + 2) * box_w * 2;   // a multiple of 256 bytes
        // Ring depths: two weight slots, three raw halo tiles in flight and two record slots at least; what is left of the
        // shared memory goes to a third weight slot (a step of one tile holds a slot only half as long), then a fourth raw tile.
        const int fixed_bytes = 2 * kOutImages * kOutImageBytes + (6 * kMaxSlots + 4) * 8 + 16 + 1024;
        const int budget = 227 * 1024 - fixed_bytes;
        p.weight_slots = 2;
        p.raw_slots = 2;
        p.rec_slots = 2;
        auto ring_bytes = [&] { return p.weight_slots * kWeightStageBytes + p.raw_slots * p.staging_bytes + p.rec_slots * p.act_stage_bytes; };
        if (ring_bytes() > budget) return 1;
        if (ring_bytes() + p.staging_bytes <= budget) p.raw_slots = 3;
        if (ring_bytes() + kWeightStageBytes <= budget) p.weight_slots = 3;
        if (ring_bytes() + p.staging_bytes <= budget) p.raw_slots = 4;
        if (ring_bytes() + p.act_stage_bytes <= budget) p.rec_slots = 3;
        const int smem_bytes = ring_bytes() + fixed_bytes;
            auto* kernel = &conv3x3_staged_kernel<kBf16>;
        if (!smem_limit[1].at_least(smem_bytes, [&](int need) { return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, need) == cudaSuccess; })) {
            return 1;
        }
        CUtensorMap map_x;
        if (!encode_input_map(&map_x, x, B, C_in, H, W, box_w, rows + 2, kBf16)) return 1;
        CUtensorMap map_y;
        if (!encode_output_map(&map_y, y, B, C_out, H, W, kBf16)) return 1;
        kernel<<<grid, kStagedThreads, smem_bytes, stream>>>(map_w, map_x, map_y, p);
    } else {
        const int smem_bytes = kStages * (kWeightStageBytes + p.act_stage_bytes) + (3 * kStages + 4) * 8 + 16 + 1024;
        auto* kernel = &conv3x3_kernel<kBf16>;
        if (!smem_limit[0].at_least(smem_bytes, [&](int need) { return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, need) == cudaSuccess; })) {
            return 1;
        }
        kernel<<<grid, kThreads, smem_bytes, stream>>>(map_w, p);
    }
    return cudaGetLastError() == cudaSuccess ? 0 : 1;
}

// FEATHER_CONV_PAIR_OFF=1 keeps every shape on the one-CTA kernel (A/B measurements). Read once per process.
inline bool pair_off() {
    static const bool off = env_switch("FEATHER_CONV_PAIR_OFF");
    return off;
}

}  // namespace conv
}  // namespace feather

// C ABI, same signature as the reference's `feather_conv3x3_launch` (csrc/hip_conv2d_3x3.cu:561-575).
// x: [B, C_in, H, W]; wp: prepacked weight [ceil(C_in / 16) * 18, C_out, 8]; bias: [C_out] or NULL;
// y: [B, C_out, H, W]; all in one 16-bit dtype (is_bf16), contiguous, 16-byte aligned; C_in % 8 == 0.
// `(warps_m, warps_n, repeat_m, repeat_n, rows)` must be a row of the conv tile table: its
// `16 * warps_n * repeat_n` picks the pixel-segment width and `rows` the rows per tile. `prefetch` is
// accepted and ignored (the pipeline always runs ahead). Returns 0 on success, 1 for an unknown tile, a
// two-row tile with an odd W, or an unsupported shape.
extern "C" int feather_conv3x3_launch(const void* x, const void* wp, const void* bias, void* y, int B, int C_in, int C_out, int H, int W,
                                      int has_bias, int warps_m, int warps_n, int repeat_m, int repeat_n, int rows, int is_bf16,
                                      int prefetch, void* stream_ptr) {
    using namespace feather;
    (void)prefetch;
    if (!conv_tile_known(warps_m, warps_n, repeat_m, repeat_n, rows)) return 1;
    if (rows == 2 && (W & 1) != 0) return 1;
    if (B < 0 || C_in <= 0 || C_out <= 0 || H <= 0 || W <= 0 || C_in % 8 != 0) return 1;
    if (B == 0) return 0;
    const int block_n = 16 * warps_n * repeat_n;
    int bn = block_n <= 64 ? 64 : block_n <= 128 ? 128 : 256;
    if (rows == 2 && bn == 256) bn = 128;  // two rows of 256 pixels do not fit one accumulator buffer
    if ((W & 1) != 0 && bn == 256) bn = 128;  // odd widths gather pixel by pixel: keep the item count per thread bounded
    const cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_ptr);
    const void* const bias_ptr = has_bias ? bias : nullptr;
    // two rows of 128 pixels and more than one 128-channel tile: the CTA-pair kernel computes the same tile
    // shape (same accumulation order) with two SMs sharing the pixels
    if (rows == 2 && bn == 128 && C_out > conv::kBlockM && !conv::pair_off()) {
        return is_bf16 != 0 ? conv::launch_pair<true>(x, wp, bias_ptr, y, B, C_in, C_out, H, W, stream)
                            : conv::launch_pair<false>(x, wp, bias_ptr, y, B, C_in, C_out, H, W, stream);
    }
    return is_bf16 != 0 ? conv::launch<true>(x, wp, bias_ptr, y, B, C_in, C_out, H, W, bn, rows, stream)
                        : conv::launch<false>(x, wp, bias_ptr, y, B, C_in, C_out, H, W, bn, rows, stream);
}

// Reads and clears the conv kernel's wait-status record (see feather_scaled_mm_status).
extern "C" int feather_conv3x3_status(uint32_t* out) {
    uint32_t zero[2] = {0u, 0u};
    if (cudaDeviceSynchronize() != cudaSuccess) return 1;
    if (cudaMemcpyFromSymbol(out, feather::conv::g_status, sizeof(zero)) != cudaSuccess) return 1;
    if (cudaMemcpyToSymbol(feather::conv::g_status, zero, sizeof(zero)) != cudaSuccess) return 1;
    return 0;
}
