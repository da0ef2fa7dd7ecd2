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
// With more than 128 output channels and the two-row tile, CTA pairs take over (second kernel in this file): two
// SMs share the pixels of a 256-channel tile.
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

// kStaged: the halo tile of a slot comes by TMA (a 4-D box over the NCHW input, channel-planar, zero filled outside the
// image and past C_in) into a staging buffer of the slot, and the gather warps only re-lay it shared -> shared into
// the pixel records. The copies then run slots ahead of the gather without holding registers; with loads from global
// memory into registers the gather has one group per team in flight and runs at the pace of the memory latency.
// A TMA box starts on a 16-byte boundary, so the box begins eight pixels left of the tile (w0 - 8, the halo's first
// column is w0 - 1) and is sixteen pixels wider; it needs W % 8 == 0 (16-byte row pitch) and at most 128 pixels per row
// segment (a box side is at most 256 elements).
template <bool kBf16, bool kStaged>
__global__ void __launch_bounds__(kThreads, 1) conv3x3_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const Params p) {
    extern __shared__ uint8_t smem_dyn[];
    uint8_t* const smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t* const weight_smem = smem;
    uint8_t* const act_smem = smem + kStages * kWeightStageBytes;
    uint8_t* const staging_smem = act_smem + kStages * p.act_stage_bytes;   // kStaged only (staging_bytes is 0 otherwise)
    uint64_t* const bars = reinterpret_cast<uint64_t*>(staging_smem + kStages * p.staging_bytes);
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
    // A parity wait tells "the phase I need has completed" from "the phase before it has not" only for a waiter that
    // visits every use of a slot, or whose barriers complete in the order of the uses. The staged gather waits on the
    // copy engine's barriers, which complete in any order across slots: a team that skipped a use of a slot (two teams
    // over three slots) could run a whole ring ahead of a late copy and take the slot's previous phase for its own. So
    // the staged gather is one team that visits every use. The gather from global memory waits on the MMA commits, which
    // arrive in issue order, and keeps two teams.
    constexpr int kMyTeams = kStaged ? 1 : kTeams;
    constexpr int kMyTeamWarps = kGatherWarps / kMyTeams;

    if (threadIdx.x == 0) {
        *abort_flag = 0u;
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&weight_full[s], 1);
            mbar_init(&act_full[s], kMyTeamWarps);
            mbar_init(&stage_empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&tmem_full[s], 1);
            mbar_init(&tmem_empty[s], kEpilogueWarps);
        }
        mbar_init_fence();
        tma_prefetch_desc(&map_w);
        if constexpr (kStaged) tma_prefetch_desc(&map_x);
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
                    mbar_arrive_expect_tx(&weight_full[s], kWeightStageBytes + (kStaged ? p.staging_bytes : 0));
                    tma_load_2d(weight_smem + s * kWeightStageBytes, &map_w, &weight_full[s], tc.m0 * 2, g * kWeightRows);
                    if constexpr (kStaged) {
                        tma_load_4d(staging_smem + s * p.staging_bytes, &map_x, &weight_full[s], tc.w0 - 8, tc.h0 - 1, g * 16, tc.b);
                    }
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
                    const int w_first = tc.w0 + c * 32;
                    if (vector_rows) {
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            if (w_first + g * 8 < p.W) {
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
                            if (w_first + i < p.W) {
                                const uint32_t o = pack_out<kBf16>(__uint_as_float(v[i]) + bias, 0.0f);
                                y_row[w_first + i] = static_cast<uint16_t>(o & 0xffffu);
                            }
                        }
                    }
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ activation gather warps
        const int team = (warp - kFirstGatherWarp) / kMyTeamWarps;
        const int t = static_cast<int>(threadIdx.x) - (kFirstGatherWarp + team * kMyTeamWarps) * 32;
        constexpr int kTeamThreads = kMyTeamWarps * 32;
        const int64_t hw = static_cast<int64_t>(p.H) * p.W;
        // Work items of one slot. With `pairs`: per (plane, halo row) the halo columns 1..BN as BN / 2 aligned
        // pixel pairs, then the two edge columns 0 and BN + 1 as single pixels. Without: every column alone.
        const int per_row = p.pairs ? p.bn / 2 + 2 : halo_cols;
        const int items = 2 * halo_rows * per_row;
        uint32_t it = 0;
        bool ok = true;
        if constexpr (kStaged) {
            // The staging buffer is [16 channels][halo_rows][bn + 16 pixels]; halo column hc is staged pixel hc + 7. An item is
            // a pixel pair (halo columns 1 + 2 e and 2 + 2 e: a 4-byte aligned load per channel) or one of the two edge
            // pixels, for one 8-channel plane: eight loads, a byte permute, one or two 16-byte record stores. The geometry
            // does not depend on the tile (the TMA unit has done the clipping and the zero fill), so it is decoded once.
            const int staged_cols = p.bn + 16;
            const int channel_pitch = halo_rows * staged_cols * 2;   // bytes between the same pixel of consecutive channels
            int src_off[kMaxItems];
            int dst_off[kMaxItems];
            uint32_t pair_mask = 0;
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
                    const bool pair = e < p.bn / 2;
                    const int hc = pair ? 1 + 2 * e : (e == p.bn / 2 ? 0 : p.bn + 1);
                    src_off[j] = plane * 8 * channel_pitch + (hr * staged_cols + hc + 7) * 2;
                    dst_off[j] = plane * plane_bytes + (hr * halo_cols + hc) * 16;
                    if (pair) pair_mask |= 1u << j;
                }
            }
            for (int tile = static_cast<int>(blockIdx.x); ok && tile < num_tiles; tile += static_cast<int>(gridDim.x)) {
                for (int g = 0; g < p.groups; ++g, ++it) {
                    static_assert(kMyTeams == 1, "the staged gather visits every use of a slot");
                    const uint32_t s = it % kStages;
                    const uint32_t phase = (it / kStages) & 1u;
                    // the slot's raw tile (and its weights) have landed; the records of the slot's previous use were read by
                    // UMMAs that completed before the copy engine was allowed to refill the slot
                    ok = guard.wait(&weight_full[s], phase, kSiteLoadFull, 3);
                    if (!ok) break;
                    const uint8_t* const src = staging_smem + s * p.staging_bytes;
                    uint8_t* const dst = act_smem + s * p.act_stage_bytes;
#pragma unroll
                    for (int j = 0; j < kMaxItems; ++j) {
                        if (dst_off[j] < 0) continue;
                        uint32_t v[8];
                        if ((pair_mask >> j) & 1u) {
#pragma unroll
                            for (int c = 0; c < 8; ++c) v[c] = *reinterpret_cast<const uint32_t*>(src + src_off[j] + c * channel_pitch);
                            *reinterpret_cast<uint4*>(dst + dst_off[j]) = make_uint4(__byte_perm(v[0], v[1], 0x5410u), __byte_perm(v[2], v[3], 0x5410u),
                                                                                      __byte_perm(v[4], v[5], 0x5410u), __byte_perm(v[6], v[7], 0x5410u));
                            *reinterpret_cast<uint4*>(dst + dst_off[j] + 16) = make_uint4(__byte_perm(v[0], v[1], 0x7632u), __byte_perm(v[2], v[3], 0x7632u),
                                                                                           __byte_perm(v[4], v[5], 0x7632u), __byte_perm(v[6], v[7], 0x7632u));
                        } else {
#pragma unroll
                            for (int c = 0; c < 8; ++c) v[c] = *reinterpret_cast<const uint16_t*>(src + src_off[j] + c * channel_pitch);
                            *reinterpret_cast<uint4*>(dst + dst_off[j]) = make_uint4(__byte_perm(v[0], v[1], 0x5410u), __byte_perm(v[2], v[3], 0x5410u),
                                                                                      __byte_perm(v[4], v[5], 0x5410u), __byte_perm(v[6], v[7], 0x5410u));
                        }
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&act_full[s]);
                }
            }
        }
        for (int tile = static_cast<int>(blockIdx.x); !kStaged && ok && tile < num_tiles; tile += static_cast<int>(gridDim.x)) {
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

// Pipeline shape of the two variants. Gathering from global memory: four slots, four teams of gather warps taking the
// 16-channel groups in turn, so that four groups' loads are in flight (2 teams: 1.19, 4: 1.24 PFLOP/s). Staged by TMA:
// three slots (a slot also holds the raw halo tile), one team: the re-layout reads shared memory and takes a fraction
// of a group's UMMA time, and the copies run ahead by themselves.
template <bool kStaged>
struct PairShape {
    static constexpr int kStages = kStaged ? 3 : 4;
    static constexpr int kTeams = kStaged ? 1 : 4;
    static constexpr int kTeamWarps = kGatherWarps / kTeams;
    static constexpr int kItems = (2 * kPairHaloRows * (kPairBN / 2 + 2) + kTeamWarps * 32 - 1) / (kTeamWarps * 32);   // gather items per thread per slot
    static constexpr int kStagingBytes = kStaged ? kPairStagingBytes : 0;
    static constexpr int kSmemBytes = kStages * (kWeightStageBytes + kPairActStageBytes + kStagingBytes) + (3 * kStages + 4) * 8 + 16 + 1024;
    static_assert(kStages % kTeams == 0, "ring depth must be a multiple of the team count");
    static_assert(kSmemBytes <= 227 * 1024, "a CTA's shared memory");
};

template <bool kBf16, bool kStaged>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
conv3x3_pair_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const Params p) {
    using S = PairShape<kStaged>;
    constexpr int kPairStages = S::kStages;
    constexpr int kPairTeams = S::kTeams;
    constexpr int kPairTeamWarps = S::kTeamWarps;
    constexpr int kPairItems = S::kItems;
    extern __shared__ uint8_t smem_dyn[];
    uint8_t* const smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t* const weight_smem = smem;
    uint8_t* const act_smem = smem + kPairStages * kWeightStageBytes;
    uint8_t* const staging_smem = act_smem + kPairStages * kPairActStageBytes;   // kStaged only
    uint64_t* const bars = reinterpret_cast<uint64_t*>(staging_smem + kPairStages * S::kStagingBytes);
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
        if constexpr (kStaged) tma_prefetch_desc(&map_x);
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
                    mbar_arrive_expect_tx(&weight_full[s], kWeightStageBytes + S::kStagingBytes);
                    tma_load_2d(weight_smem + s * kWeightStageBytes, &map_w, &weight_full[s], tc.m0 * 2, g * kWeightRows);
                    if constexpr (kStaged) {
                        // the three halo rows of this CTA's output row h0 + cta, eight pixels to the left for the 16-byte rule
                        tma_load_4d(staging_smem + s * kPairStagingBytes, &map_x, &weight_full[s], tc.w0 - 8, tc.h0 + static_cast<int>(cta) - 1, g * 16, tc.b);
                    }
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
                    const int w_first = tc.w0 + c * 32;
                    if (vector_rows) {
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            if (w_first + g * 8 < p.W) {
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
                            if (w_first + i < p.W) {
                                const uint32_t o = pack_out<kBf16>(__uint_as_float(v[i]) + bias, 0.0f);
                                y_row[w_first + i] = static_cast<uint16_t>(o & 0xffffu);
                            }
                        }
                    }
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
        if constexpr (kStaged) {
            // Re-layout from the slot's staging buffer [16 channels][3 halo rows][144 pixels] (halo column hc is staged pixel
            // hc + 7) into the pixel records; the geometry does not depend on the tile, the TMA unit has done the clipping.
            constexpr int kChannelPitch = kPairHaloRows * kPairStagedCols * 2;
            int src_off[kPairItems];
            int dst_off[kPairItems];
            uint32_t pair_mask = 0;
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
                    src_off[j] = plane * 8 * kChannelPitch + (hr * kPairStagedCols + hc + 7) * 2;
                    dst_off[j] = plane * kPairPlaneBytes + (hr * kPairHaloCols + hc) * 16;
                    if (pair) pair_mask |= 1u << j;
                }
            }
            for (int tile = first_tile; ok && tile < num_tiles; tile += tile_step) {
                for (int g = 0; g < p.groups; ++g, ++it) {
                    if (static_cast<int>(it % kPairTeams) != team) continue;
                    const uint32_t s = it % kPairStages;
                    const uint32_t phase = (it / kPairStages) & 1u;
                    // this CTA's raw halo tile and weight rows of the slot have landed (the slot's records were last read by
                    // UMMAs that completed before the copy engine was allowed to refill the slot)
                    ok = guard.wait(&weight_full[s], phase, kSiteLoadFull, 3);
                    if (!ok) break;
                    const uint8_t* const src = staging_smem + s * kPairStagingBytes;
                    uint8_t* const dst = act_smem + s * kPairActStageBytes;
#pragma unroll
                    for (int j = 0; j < kPairItems; ++j) {
                        if (dst_off[j] < 0) continue;
                        uint32_t v[8];
                        if ((pair_mask >> j) & 1u) {
#pragma unroll
                            for (int c = 0; c < 8; ++c) v[c] = *reinterpret_cast<const uint32_t*>(src + src_off[j] + c * kChannelPitch);
                            *reinterpret_cast<uint4*>(dst + dst_off[j]) = make_uint4(__byte_perm(v[0], v[1], 0x5410u), __byte_perm(v[2], v[3], 0x5410u),
                                                                                      __byte_perm(v[4], v[5], 0x5410u), __byte_perm(v[6], v[7], 0x5410u));
                            *reinterpret_cast<uint4*>(dst + dst_off[j] + 16) = make_uint4(__byte_perm(v[0], v[1], 0x7632u), __byte_perm(v[2], v[3], 0x7632u),
                                                                                           __byte_perm(v[4], v[5], 0x7632u), __byte_perm(v[6], v[7], 0x7632u));
                        } else {
#pragma unroll
                            for (int c = 0; c < 8; ++c) v[c] = *reinterpret_cast<const uint16_t*>(src + src_off[j] + c * kChannelPitch);
                            *reinterpret_cast<uint4*>(dst + dst_off[j]) = make_uint4(__byte_perm(v[0], v[1], 0x5410u), __byte_perm(v[2], v[3], 0x5410u),
                                                                                      __byte_perm(v[4], v[5], 0x5410u), __byte_perm(v[6], v[7], 0x5410u));
                        }
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&act_full[s]), 0));
                }
            }
        }
        for (int tile = first_tile; !kStaged && ok && tile < num_tiles; tile += tile_step) {
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

template <bool kBf16>
int launch_pair(const void* x, const void* wp, const void* bias, void* y, int B, int C_in, int C_out, int H, int W, cudaStream_t stream) {
    const bool staged = (W % 8) == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0 && !staging_off();
    auto* kernel = staged ? &conv3x3_pair_kernel<kBf16, true> : &conv3x3_pair_kernel<kBf16, false>;
    const int kPairSmemBytes = staged ? PairShape<true>::kSmemBytes : PairShape<false>::kSmemBytes;
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

    // once per device: the shared-memory limit and how many CTA pairs fit at once (a persistent grid must be resident as a
    // whole, and a pair needs both SMs of a TPC)
    static PerDeviceState resident_pairs_of[2];
    PerDeviceState& resident_pairs = resident_pairs_of[staged ? 1 : 0];
    const int pairs = resident_pairs.get([&] {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmemBytes) != cudaSuccess) return 0;
        cudaLaunchConfig_t config = {};
        config.gridDim = dim3(static_cast<unsigned>(device_info().sm_count / 2 * 2));
        config.blockDim = dim3(kThreads);
        config.dynamicSmemBytes = kPairSmemBytes;
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
    if (pairs <= 0) return 1;

    CUtensorMap map_w;
    if (!encode_weight_map(&map_w, wp, C_out, p.groups)) return 1;
    CUtensorMap map_x = map_w;   // unused by the kernel that gathers from global memory
    if (staged && !encode_input_map(&map_x, x, B, C_in, H, W, kPairStagedCols, kPairHaloRows, kBf16)) return 1;
    const int64_t tiles_m = (C_out + 2 * kBlockM - 1) / (2 * kBlockM);
    const int64_t num_tiles = static_cast<int64_t>(B) * tiles_m * ((H + 1) / 2) * ((W + kPairBN - 1) / kPairBN);
    if (num_tiles > (1ll << 30)) return 1;
    const int grid = 2 * static_cast<int>(num_tiles < pairs ? num_tiles : pairs);
    kernel<<<grid, kThreads, kPairSmemBytes, stream>>>(map_w, map_x, p);
    return cudaGetLastError() == cudaSuccess ? 0 : 1;
}

template <bool kBf16>
int launch(const void* x, const void* wp, const void* bias, void* y, int B, int C_in, int C_out, int H, int W, int bn, int rows,
           cudaStream_t stream) {
    // staged halo tiles need a 16-byte row pitch, at most 128 pixels per segment (a TMA box side is at most 256 elements)
    // and a 16-byte aligned input
    const bool staged = (W % 8) == 0 && bn <= 128 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0 && !staging_off();
    auto* kernel = staged ? &conv3x3_kernel<kBf16, true> : &conv3x3_kernel<kBf16, false>;
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
    if (2 * (rows + 2) * per_row > kMaxItems * kTeamWarps * 32) return 1;

    p.staging_bytes = staged ? (16 * (rows + 2) * (bn + 16) * 2 + 127) / 128 * 128 : 0;
    const int smem_bytes = kStages * (kWeightStageBytes + p.act_stage_bytes + p.staging_bytes) + (3 * kStages + 4) * 8 + 16 + 1024;
    static PerDeviceState smem_limit[2];
    if (!smem_limit[staged ? 1 : 0].at_least(smem_bytes, [&](int need) { return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, need) == cudaSuccess; })) {
        return 1;
    }

    CUtensorMap map_w;
    if (!encode_weight_map(&map_w, wp, C_out, p.groups)) return 1;
    CUtensorMap map_x = map_w;   // unused by the kernel that gathers from global memory
    if (staged && !encode_input_map(&map_x, x, B, C_in, H, W, bn + 16, rows + 2, kBf16)) return 1;
    const int64_t num_tiles = static_cast<int64_t>(B) * p.tiles_m * p.tiles_h * p.tiles_w;
    if (num_tiles > (1ll << 30)) return 1;
    const int sms = device_info().sm_count;
    const int grid = num_tiles < sms ? static_cast<int>(num_tiles) : sms;
    kernel<<<grid, kThreads, smem_bytes, stream>>>(map_w, map_x, p);
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
