// Generated from feather_ops_b200/tiles.py by feather_ops_b200/_build.py. Do not edit.
#pragma once

namespace feather {

constexpr int kScaledMmTilesArity = 6;
constexpr int kScaledMmTilesCount = 35;
constexpr int kScaledMmTiles[35][6] = {
    {1, 1, 2, 1, 2, 0},
    {1, 1, 4, 1, 2, 0},
    {1, 2, 2, 1, 2, 0},
    {1, 2, 4, 1, 2, 0},
    {1, 2, 4, 1, 2, 1},
    {1, 4, 2, 1, 2, 0},
    {1, 4, 4, 1, 2, 0},
    {1, 8, 2, 1, 2, 0},
    {1, 8, 4, 1, 2, 0},
    {1, 1, 2, 2, 2, 0},
    {1, 1, 4, 2, 2, 0},
    {1, 1, 2, 4, 4, 0},
    {1, 1, 4, 4, 4, 0},
    {1, 2, 2, 2, 2, 0},
    {1, 2, 2, 2, 2, 1},
    {1, 2, 4, 2, 2, 0},
    {2, 1, 2, 2, 2, 0},
    {2, 2, 2, 2, 2, 0},
    {2, 2, 2, 2, 2, 1},
    {2, 1, 4, 2, 2, 0},
    {1, 4, 2, 4, 2, 0},
    {1, 4, 2, 4, 2, 1},
    {1, 4, 4, 4, 2, 0},
    {1, 8, 2, 8, 2, 0},
    {1, 8, 4, 8, 2, 0},
    {2, 2, 2, 4, 4, 0},
    {2, 2, 4, 4, 4, 0},
    {2, 4, 2, 4, 2, 0},
    {2, 4, 4, 4, 2, 0},
    {2, 4, 2, 4, 4, 0},
    {2, 4, 4, 4, 4, 0},
    {4, 2, 2, 2, 4, 0},
    {4, 2, 4, 2, 4, 0},
    {4, 4, 2, 4, 2, 0},
    {4, 4, 2, 4, 4, 0},
};

constexpr int kInt8TilesArity = 5;
constexpr int kInt8TilesCount = 22;
constexpr int kInt8Tiles[22][5] = {
    {1, 1, 2, 1, 2},
    {1, 2, 2, 1, 2},
    {1, 4, 2, 1, 2},
    {1, 8, 2, 1, 2},
    {1, 1, 4, 1, 2},
    {1, 2, 4, 1, 2},
    {1, 4, 4, 1, 2},
    {1, 8, 4, 1, 2},
    {1, 2, 2, 2, 2},
    {1, 4, 2, 2, 2},
    {2, 2, 2, 2, 2},
    {2, 4, 2, 2, 2},
    {1, 4, 2, 4, 2},
    {1, 8, 2, 4, 2},
    {2, 2, 2, 4, 4},
    {2, 4, 2, 4, 4},
    {4, 2, 2, 4, 4},
    {2, 4, 4, 4, 4},
    {2, 2, 4, 4, 2},
    {2, 4, 2, 4, 2},
    {2, 8, 2, 4, 2},
    {4, 4, 2, 4, 4},
};

constexpr int kConvTilesArity = 5;
constexpr int kConvTilesCount = 38;
constexpr int kConvTiles[38][5] = {
    {4, 4, 2, 4, 1},
    {4, 4, 2, 3, 1},
    {4, 4, 2, 2, 1},
    {4, 2, 2, 3, 1},
    {8, 2, 1, 2, 1},
    {8, 1, 1, 2, 1},
    {3, 8, 2, 2, 1},
    {3, 4, 2, 3, 1},
    {3, 4, 2, 2, 1},
    {3, 3, 2, 2, 1},
    {3, 2, 2, 2, 1},
    {3, 1, 2, 2, 1},
    {2, 8, 2, 2, 1},
    {2, 4, 2, 3, 1},
    {2, 4, 2, 2, 1},
    {2, 2, 2, 3, 1},
    {2, 2, 2, 2, 1},
    {4, 1, 1, 2, 1},
    {1, 8, 3, 2, 1},
    {1, 4, 3, 3, 1},
    {1, 4, 3, 2, 1},
    {1, 2, 3, 3, 1},
    {1, 2, 3, 2, 1},
    {1, 1, 3, 2, 1},
    {2, 8, 1, 2, 1},
    {2, 4, 1, 3, 1},
    {2, 4, 1, 2, 1},
    {2, 3, 1, 2, 1},
    {2, 2, 1, 2, 1},
    {2, 1, 1, 2, 1},
    {1, 8, 1, 2, 1},
    {1, 4, 1, 3, 1},
    {1, 4, 1, 2, 1},
    {1, 3, 1, 2, 1},
    {1, 2, 1, 2, 1},
    {1, 1, 1, 2, 1},
    {4, 4, 2, 2, 2},
    {2, 8, 2, 2, 2},
};

template <int kCount, int kArity>
inline bool tile_in_table(const int (&table)[kCount][kArity], const int (&query)[kArity]) {
    for (int i = 0; i < kCount; ++i) {
        bool same = true;
        for (int j = 0; j < kArity; ++j) same = same && table[i][j] == query[j];
        if (same) return true;
    }
    return false;
}

// `16 * warps_n * repeat_n` of a known scaled_mm tile tuple, 0 for an unknown one.
inline int scaled_mm_tile_block_n(int wm, int wn, int uk, int rm, int rn, int pipeline) {
    const int query[6] = {wm, wn, uk, rm, rn, pipeline};
    return tile_in_table(kScaledMmTiles, query) ? 16 * wn * rn : 0;
}

// `16 * warps_n * repeat_n` of a known int8 tile tuple, 0 for an unknown one.
inline int int8_tile_block_n(int wm, int wn, int uk, int rm, int rn) {
    const int query[5] = {wm, wn, uk, rm, rn};
    return tile_in_table(kInt8Tiles, query) ? 16 * wn * rn : 0;
}

// Whether `(warps_m, warps_n, repeat_m, repeat_n, rows)` is a known conv tile tuple.
inline bool conv_tile_known(int wm, int wn, int rm, int rn, int rows) {
    const int query[5] = {wm, wn, rm, rn, rows};
    return tile_in_table(kConvTiles, query);
}

}  // namespace feather
