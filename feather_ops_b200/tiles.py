"""Blackwell tile table: which UMMA tile each tile tuple of the public API runs on.

The public API keeps the reference's tile vocabulary (`feather_ops/tiles.py:17-119` in the reference): a
GEMM tile is `(warps_m, warps_n, unroll_k, repeat_m, repeat_n[, pipeline])` and a conv tile is
`(warps_m, warps_n, repeat_m, repeat_n, rows)`, with `block = 16 * warps * repeat`. On gfx11 those
numbers instantiate one kernel each. On sm_100a a tile tuple is only a key: the kernels are built
around one `tcgen05.mma` shape family (M = 128 rows per CTA, N in {64, 128, 256} columns, TMEM
accumulators), and a tuple selects the member of that family whose width matches the tuple's
`block_n`. Tuples that are not in these tables are rejected by the launchers ("Unsupported config").

This module must not import torch: the build step reads it to generate `csrc/feather_tiles_gen.h`.
"""

from typing import NamedTuple


class UmmaTile(NamedTuple):
    """The sm_100a tile a public tuple maps to."""

    block_m: int  # rows of the accumulator one CTA owns (the UMMA M)
    block_n: int  # UMMA N
    block_k: int  # contraction elements staged per pipeline slot


def gemm_block_sizes(tile: tuple[int, ...]) -> tuple[int, int, int]:
    """`(block_m, block_n, chunk_k)` a GEMM tile tuple names in the public vocabulary."""
    return 16 * tile[0] * tile[3], 16 * tile[1] * tile[4], 16 * tile[2]


def conv_block_sizes(tile: tuple[int, ...]) -> tuple[int, int, int]:
    """`(block_m, block_n, rows)` a conv tile tuple names in the public vocabulary."""
    return 16 * tile[0] * tile[2], 16 * tile[1] * tile[3], tile[4]


def _umma_width(block_n: int) -> int:
    if block_n >= 256:
        return 256
    return 128 if block_n >= 128 else 64


def _expand(rows: str, arity: int) -> list[tuple[int, ...]]:
    """Tuples from a whitespace separated string of `arity`-digit words (every field is < 10)."""
    tiles = [tuple(int(ch) for ch in word) for word in rows.split()]
    assert all(len(tile) == arity for tile in tiles)
    return tiles


# fp8 weights x fp16/bf16 activations: `(warps_m, warps_n, unroll_k, repeat_m, repeat_n, pipeline)`.
SCALED_MM_TILES = _expand(
    """
    112120 114120 122120 124120 124121 142120 144120 182120 184120
    112220 114220 112440 114440 122220 122221 124220 212220 222220
    222221 214220 142420 142421 144420 182820 184820 222440 224440
    242420 244420 242440 244440 422240 424240 442420 442440
    """,
    6,
)

# int8 ConvRot GEMM: `(warps_m, warps_n, unroll_k, repeat_m, repeat_n)`.
INT8_TILES = _expand(
    """
    11212 12212 14212 18212 11412 12412 14412 18412 12222 14222 22222
    24222 14242 18242 22244 24244 42244 24444 22442 24242 28242 44244
    """,
    5,
)

# conv2d 3x3: `(warps_m, warps_n, repeat_m, repeat_n, rows)`.
CONV_TILES = _expand(
    """
    44241 44231 44221 42231 82121 81121 38221 34231 34221 33221 32221 31221
    28221 24231 24221 22231 22221 41121 18321 14331 14321 12331 12321 11321
    28121 24131 24121 23121 22121 21121 18121 14131 14121 13121 12121 11121
    44222 28222
    """,
    5,
)

SCALED_MM_UMMA = {tile: UmmaTile(128, _umma_width(gemm_block_sizes(tile)[1]), 64) for tile in SCALED_MM_TILES}
INT8_UMMA = {tile: UmmaTile(128, _umma_width(gemm_block_sizes(tile)[1]), 128) for tile in INT8_TILES}
# The conv kernel's accumulator is `block_m` output channels x `block_n * rows` pixels.
CONV_UMMA = {tile: UmmaTile(128 if conv_block_sizes(tile)[0] >= 128 else 64, conv_block_sizes(tile)[1] * tile[4], 16) for tile in CONV_TILES}

# Kept for API compatibility with the reference's policy constants (`feather_ops/tiles.py:134-142`). On
# B200 neither dtype is delegated for a shape the kernel tiles, so the fp16 threshold is zero.
MIOPEN_FP16_MAX_INPUT_ELEMS = 0
MIOPEN_BF16_FALLBACK_MAX_INPUT_ELEMS = 1 << 30
CONV_PREFETCH_MIN_C_IN = 128


def render_header() -> str:
    """C++ lookup tables generated from the lists above (written to `csrc/feather_tiles_gen.h`)."""
    out = [
        "// Generated from feather_ops_b200/tiles.py by feather_ops_b200/_build.py. Do not edit.",
        "#pragma once",
        "",
        "namespace feather {",
        "",
    ]

    def table(name: str, tiles: list[tuple[int, ...]], arity: int) -> None:
        out.append(f"constexpr int k{name}Arity = {arity};")
        out.append(f"constexpr int k{name}Count = {len(tiles)};")
        out.append(f"constexpr int k{name}[{len(tiles)}][{arity}] = {{")
        for tile in tiles:
            out.append("    {" + ", ".join(str(v) for v in tile) + "},")
        out.append("};")
        out.append("")

    table("ScaledMmTiles", SCALED_MM_TILES, 6)
    table("Int8Tiles", INT8_TILES, 5)
    table("ConvTiles", CONV_TILES, 5)
    out += [
        "template <int kCount, int kArity>",
        "inline bool tile_in_table(const int (&table)[kCount][kArity], const int (&query)[kArity]) {",
        "    for (int i = 0; i < kCount; ++i) {",
        "        bool same = true;",
        "        for (int j = 0; j < kArity; ++j) same = same && table[i][j] == query[j];",
        "        if (same) return true;",
        "    }",
        "    return false;",
        "}",
        "",
        "// `16 * warps_n * repeat_n` of a known scaled_mm tile tuple, 0 for an unknown one.",
        "inline int scaled_mm_tile_block_n(int wm, int wn, int uk, int rm, int rn, int pipeline) {",
        "    const int query[6] = {wm, wn, uk, rm, rn, pipeline};",
        "    return tile_in_table(kScaledMmTiles, query) ? 16 * wn * rn : 0;",
        "}",
        "",
        "// `16 * warps_n * repeat_n` of a known int8 tile tuple, 0 for an unknown one.",
        "inline int int8_tile_block_n(int wm, int wn, int uk, int rm, int rn) {",
        "    const int query[5] = {wm, wn, uk, rm, rn};",
        "    return tile_in_table(kInt8Tiles, query) ? 16 * wn * rn : 0;",
        "}",
        "",
        "// Whether `(warps_m, warps_n, repeat_m, repeat_n, rows)` is a known conv tile tuple.",
        "inline bool conv_tile_known(int wm, int wn, int rm, int rn, int rows) {",
        "    const int query[5] = {wm, wn, rm, rn, rows};",
        "    return tile_in_table(kConvTiles, query);",
        "}",
        "",
        "}  // namespace feather",
        "",
    ]
    return "\n".join(out)
