"""`Y = (X @ W) * scale + bias` with fp16/bf16 activations and a prepacked fp8 weight.

Python side of the `scaled_mm` operator: output allocation, tile choice, and the weight prepack. The API
is the reference's (`feather_ops/scaled_mm.py` there): `scaled_mm_hip(a, b_prepacked, scale, bias,
out_dtype, tile=None)` keeps its name so callers switch by changing the import.
`X` is `[M, K]`, the weight is `[K_pad/16, N, 16]` fp8 (e5m2 or e4m3fn), `scale` a one-element float32
tensor or None, `bias` `[N]` in the output dtype or None. Any `M >= 1`; `N` and `K` multiples of 16.
"""

import torch
from torch.library import custom_op

from .tiles import SCALED_MM_UMMA, gemm_block_sizes

# One public tuple per UMMA width (all rows of the tile table).
_TILE_N256 = (1, 8, 4, 8, 2, 0)
_TILE_N128 = (2, 2, 2, 4, 4, 0)
_TILE_N64 = (1, 2, 4, 1, 2, 1)

_DEFAULT_SM_COUNT = 148   # a B200; used only when no CUDA device is visible (the heuristics are also exercised on CPU)
_SM_COUNTS: dict = {}


def sm_count() -> int:
    """Streaming multiprocessors of the current CUDA device (the number the launchers size their grids by)."""
    if not torch.cuda.is_available():
        return _DEFAULT_SM_COUNT
    index = torch.cuda.current_device()
    if index not in _SM_COUNTS:
        _SM_COUNTS[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return _SM_COUNTS[index]


# Measured time of one wave of tiles per 64-deep k block, in microseconds (M > 128, N = 12288, K = 3072 sweeps):
# 256-wide tiles run as 256 x 256 tiles on CTA pairs, the narrower ones as 128-row tiles on single CTAs.
_WAVE_COST_US = {256: 0.40, 128: 0.42, 64: 0.35}
# launch, pipeline fill and the last tile's epilogue: what a launch costs before its k blocks count
_FIXED_COST_US = {256: 8.0, 128: 6.0, 64: 6.0}
_TILE_OF_WIDTH = {256: _TILE_N256, 128: _TILE_N128, 64: _TILE_N64}


def select_scaled_mm_config(M: int, N: int, K: int, a_dtype=torch.float16, b_dtype=torch.float8_e5m2, out_dtype=torch.bfloat16):
    """Tile tuple for one shape (same signature as the reference's `select_scaled_mm_config`,
    `feather_ops/scaled_mm.py:35-90`; the dtypes do not matter).

    The kernels are persistent, so the cost of a width is `fixed + waves * k blocks * cost of a wave per k block`: 256-wide tiles go to CTA
    pairs (256 x 256 tiles, 74 pairs) as soon as there is more than one 128-row tile, the narrower widths to
    one CTA per 128-row tile (148 CTAs). A shape with few tiles trades the wide tile for a narrower one to fill
    more SMs.
    """
    del a_dtype, b_dtype, out_dtype
    sms = sm_count()
    k_blocks = -(-K // 64)
    best = None
    for width in (256, 128, 64):
        if width == 256 and M > 128:
            waves = -(-(-(-M // 256) * -(-N // 256)) // (sms // 2))
            fixed = _FIXED_COST_US[256]
        else:
            waves = -(-(-(-M // 128) * -(-N // width)) // sms)
            fixed = _FIXED_COST_US[width if width != 256 else 128]
        cost = fixed + waves * k_blocks * _WAVE_COST_US[width] * (1.4 if width == 256 and M <= 128 else 1.0)
        if best is None or cost < best[0] - 1e-9:
            best = (cost, width)
    return _TILE_OF_WIDTH[best[1]]


_WARP_MMA_MAX_M = 16     # the launcher's vector (1-2 rows, wide outputs) and warp-MMA kernels take these rows
_WARP_MMA_MIN_N = 512
_WARP_MMA_GRID_MAX_K = 8192
_SKINNY_MAX_M = 128      # one row tile: the weight stream is the cost, a 64-wide tile per CTA, two CTAs per SM
_SKINNY_WIDE_M = 64      # above this the activation re-reads of 64-wide tiles cost more than 128-wide tiles save
_SPLIT_MAX_M = 32        # below this the fp32 partials are small against the weight and K is split as well


def select_scaled_mm_splits(M: int, N: int, K: int) -> int:
    """How many K splits the skinny path uses (1 = none). A split costs a round trip of fp32 partials and more
    CTA start-ups, so K is only split when the 64-wide column tiles alone cannot fill the resident CTAs (two per
    SM), at most four ways and never below sixteen 64-wide k blocks per split (measured: 32 x 3840 x 2560 loses a
    third with ten blocks per split, 16 x 4096 x 4096 gains 7 % with sixteen)."""
    if M > _SPLIT_MAX_M:
        return 1
    tiles = -(-N // 64)
    k_blocks = -(-K // 64)
    return max(1, min(4, 2 * sm_count() // tiles, k_blocks // 16))


_WIDE_SPLIT_MIN_K_BLOCKS = 128   # 64-deep k blocks: below this the fp32 partials cost more than the idle SMs


def warp_mma_takes(M: int, N: int, K: int) -> bool:
    """Whether the launcher runs a 64-wide tile of this shape on the vector / warp-MMA kernels (the same rule as
    `wmma_eligible` in `csrc/scaled_mm_sm100.cu`): at most 16 rows, or at most 128 rows as one grid row of CTAs per
    16 rows while all of them fit on the device at once and K is at most 8192."""
    if N < _WARP_MMA_MIN_N:
        return False
    if M <= _WARP_MMA_MAX_M:
        return True
    return M <= _SKINNY_MAX_M and -(-N // 32) * -(-M // 16) <= 3 * sm_count() and K <= _WARP_MMA_GRID_MAX_K


def select_wide_splits(M: int, N: int, K: int) -> int:
    """K splits of the one-CTA kernel with 128 x 128 tiles (1 = none): for shapes whose tiles leave at least half of
    the SMs idle. The splits are chosen so that every (tile, split) item is resident at once; then the whole CTA that
    draws a tile's last ticket adds the partials (twenty warps; with more items than SMs only the four epilogue warps
    can, and that costs more than the split wins).

    One row tile (33..128 rows that the warp-MMA kernel does not take): up to four splits, six with K >= 8192, at least
    eight 64-deep k blocks each; up to 64 rows only with three splits or more (below that the skinny kernel is level).
    Measured at 65 and 128 rows against the skinny kernel: N = 3072, K = 12288 85-90 -> 22-24 us (six splits),
    4096 x 4096 31-33 -> 16-17 (four), 3072 x 3072 25-26 -> 15-16, 5120 x 5120 38-40 -> 19-20 (three), 8192 x 3072
    25-26 -> 18 (two); one split too many and the items need a second wave (5120 x 5120 with four: 34-35 us).
    More row tiles: up to three splits of at least sixteen k blocks, from K = 3072 on: 256 x 4096 x 4096 21.8 -> 19.6 us,
    256 x 3072 x 3072 18.7 -> 16.9, 256 x 3072 x 8192 41 -> 25, 384 x 3072 x 12288 58 -> 42."""
    tiles = -(-M // 128) * -(-N // 128)
    k_blocks = -(-K // 64)
    sms = sm_count()
    if M <= 32 or tiles > sms // 2:
        return 1
    if M > _SKINNY_MAX_M:
        if k_blocks < 48:
            return 1
        return max(1, min(3, sms // tiles, k_blocks // 16))
    splits = max(1, min(6 if k_blocks >= _WIDE_SPLIT_MIN_K_BLOCKS else 4, sms // tiles, k_blocks // 8))
    if M <= 64 and splits < 3:
        return 1
    return splits


_PAIR_SPLIT_MAX = 8          # a split owns at least one 32-column chunk of a 256-wide tile's reduction
_PAIR_SPLIT_MIN_K_BLOCKS = 64   # 64-deep k blocks (K >= 4096); from 48 (K >= 3072) with more than 256 rows


def select_pair_splits(M: int, N: int, K: int) -> int:
    """K splits of the CTA-pair kernel (1 = none), for more than 128 rows and so few 256 x 256 tiles that at least half of
    the CTA pairs would idle. Every (tile, split) item gets a pair of its own, all resident at once, and every CTA of a tile
    adds its share of the columns, so the reduction is spread over the SMs that worked on the tile. A pair tile pulls half
    as many bytes per flop through an SM's L2 port as a 128 x 128 tile, which is what bounds these shapes; the price is
    a fixed cost of about 14 us per launch, so short contractions stay on the one-CTA kernels. Measured against the
    choice before (us): 256 x 4096 x 4096 23.3 -> 20.1, 512 x 4096 x 4096 29.8 -> 24.8, 256 x 5120 x 5120 37.1 -> 24.0,
    1024 x 1536 x 6144 42.2 -> 25.6, 512 x 3072 x 12288 69.6 -> 38.5, 768 x 2048 x 8192 46.7 -> 30.4; level at K = 3072
    with at most 256 rows (18.3 / 18.5) and slower below K = 3072 (256 x 2560 x 2560 16.4 -> 17.0, 512 x 1280 x 1280 9.5 -> 16.1)."""
    if M <= 128:
        return 1
    pairs = sm_count() // 2
    tiles = -(-M // 256) * -(-N // 256)
    k_blocks = -(-K // 64)
    splits = max(1, min(_PAIR_SPLIT_MAX, pairs // tiles if tiles else 1, k_blocks // 8))
    if splits < 2:
        return 1
    if k_blocks < _PAIR_SPLIT_MIN_K_BLOCKS and not (k_blocks >= 48 and M > 256):
        return 1
    return splits


def select_row_tile_splits_256(M: int, N: int, K: int) -> int:
    """K splits of the one-CTA kernel with 128 x 256 tiles (1 = do not use them) for one row tile of 64..128 rows and a wide
    output: with 32 to 74 tiles of 256 columns, three or more K splits put one (tile, split) item on nearly every SM, and an
    item fetches a third of the activations and half as many of them per flop as a 128-wide tile. Measured at N = 12288, K = 3072
    (three splits, 144 CTAs): 128 rows 25.1 -> 22.8 us, 96 rows 24.9 -> 22.4, 64 rows 23.2 -> 21.9; N = 8192 (four splits) 20.4 -> 19.5."""
    if not 64 <= M <= _SKINNY_MAX_M:
        return 1
    tiles = -(-N // 256)
    if tiles < 32 or tiles > sm_count() // 2:
        return 1
    splits = min(_PAIR_SPLIT_MAX, sm_count() // tiles, -(-K // 64) // 8)
    return splits if splits >= 3 else 1


_TICKETS: dict = {}


def _ticket_counters(device: torch.device, n: int) -> torch.Tensor:
    """Zeroed ticket counters for the split-K launches of the current stream of `device`. Every launch leaves them
    at zero, so one buffer per (device, stream) serves all calls; launches of one stream cannot overlap."""
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    need = -(-n // 64)
    buf = _TICKETS.get(key)
    if buf is None or buf.numel() < need:
        buf = torch.zeros(max(need, 1024), device=device, dtype=torch.int32)
        _TICKETS[key] = buf
    return buf


def reset_split_k_state() -> None:
    """Forget the cached ticket counters. A split-K launch whose bounded device wait ran out (reported by
    `feather_scaled_mm_status`) can leave its tickets non-zero; after such a failure the next launch must start
    from fresh zeroed counters, which this guarantees. `_lib.read_status` calls it when it sees a failure."""
    _TICKETS.clear()


def _launch(a, b_prepacked, scale, bias, out, tile) -> None:
    torch.ops.feather_ops.scaled_mm.default(a, b_prepacked, scale, bias, out, *tile[:5], bool(tile[5]))


@custom_op("feather_ops::scaled_mm_auto", mutates_args=("out",))
def _scaled_mm_auto(a: torch.Tensor, b_prepacked: torch.Tensor, scale: torch.Tensor | None, bias: torch.Tensor | None, out: torch.Tensor) -> None:
    """Tile choice + launch as one opaque node, so a compiled caller does not specialize on the heuristic."""
    m, k = a.shape
    n = b_prepacked.shape[1]
    if 0 < m <= _SKINNY_MAX_M and warp_mma_takes(m, n, k):
        # the launcher runs these on the vector or the warp-MMA kernel when the tile is 64 wide: no scratch to allocate
        _launch(a, b_prepacked, scale, bias, out, _TILE_N64)
        return
    splits = select_pair_splits(m, n, k)
    if splits > 1:
        pair_tiles = -(-m // 256) * -(-n // 256)
        partials = torch.empty(splits * pair_tiles * 256 * 256, device=a.device, dtype=torch.float32)
        torch.ops.feather_ops.scaled_mm_splitk.default(a, b_prepacked, scale, bias, out, partials, _ticket_counters(a.device, 64 * 3 * pair_tiles), splits, 256)
        return
    splits = select_row_tile_splits_256(m, n, k)
    if splits > 1:
        tiles = -(-n // 256)
        partials = torch.empty(splits * tiles * 128 * 256, device=a.device, dtype=torch.float32)
        torch.ops.feather_ops.scaled_mm_splitk.default(a, b_prepacked, scale, bias, out, partials, _ticket_counters(a.device, 64 * 2 * tiles), splits, 256)
        return
    splits = select_wide_splits(m, n, k)
    if splits > 1:
        tiles = -(-m // 128) * -(-n // 128)
        partials = torch.empty(splits * tiles * 128 * 128, device=a.device, dtype=torch.float32)
        torch.ops.feather_ops.scaled_mm_splitk.default(a, b_prepacked, scale, bias, out, partials, _ticket_counters(a.device, 64 * 2 * tiles), splits, 128)
        return
    if 0 < m <= _SKINNY_MAX_M:
        splits = select_scaled_mm_splits(m, n, k)
        if m > _SKINNY_WIDE_M and -(-n // 128) >= sm_count() // 2:
            # enough 128-wide tiles to occupy half the SMs: every activation byte is fetched half as often
            _launch(a, b_prepacked, scale, bias, out, _TILE_N128)
            return
        if splits == 1:
            # a narrow tile with at most one row tile is the skinny kernel without split: no scratch, no extra launch
            _launch(a, b_prepacked, scale, bias, out, _TILE_N64)
            return
        partials = torch.empty(splits * m * n, device=a.device, dtype=torch.float32)
        torch.ops.feather_ops.scaled_mm_splitk.default(a, b_prepacked, scale, bias, out, partials, _ticket_counters(a.device, n), splits)
        return
    _launch(a, b_prepacked, scale, bias, out, select_scaled_mm_config(m, n, k))


def scaled_mm_hip(a, b_prepacked, scale, bias, out_dtype, tile=None):
    """`(a @ W) * scale + bias` against the prepacked fp8 weight. `tile` pins a row of `SCALED_MM_TILES`."""
    out = torch.empty((a.shape[0], b_prepacked.shape[1]), device=a.device, dtype=out_dtype)
    if tile is None:
        _scaled_mm_auto(a, b_prepacked, scale, bias, out)
    else:
        _launch(a, b_prepacked, scale, bias, out, tile)
    return out



def prepack_b_for_scaled_mm(b: torch.Tensor) -> torch.Tensor:
    """`[K, N]` fp8 -> `[K_pad/16, N, 16]` with K zero padded to a multiple of 128: the sixteen consecutive k
    of one column become one 16-byte cell (the reference's layout, `feather_ops/scaled_mm.py:137-150`)."""
    k, n = b.shape
    k_pad = (k + 127) // 128 * 128
    cells = b.new_zeros((k_pad // 16, 16, n)) if k_pad != k else None
    if cells is None:
        cells = b.reshape(k // 16, 16, n)
    else:
        cells.reshape(k_pad, n)[:k] = b
    return cells.transpose(1, 2).contiguous()


def tile_shape(tile) -> tuple[int, int, int]:
    """`(block_m, block_n, chunk_k)` the tuple names in the public vocabulary."""
    return gemm_block_sizes(tile)


def umma_tile(tile):
    """The sm_100a tile the tuple runs on."""
    return SCALED_MM_UMMA[tuple(tile)]
