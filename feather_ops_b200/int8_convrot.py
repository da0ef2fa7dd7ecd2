"""Int8 ConvRot linear layers: fused rotate+quantize of the activation, int8 GEMM over a prepacked weight.

The weight format is the released one (`weight` int8 `[N, K]` in the rotated basis plus a float32 scale per
output channel). `prepack_int8_weight` permutes it into 4x4 byte micro-tiles once, and both GEMMs of a
training step read that copy:

    forward   C[M, N] = A[M, K] @ W[N, K]^T
    backward  C[M, K] = A[M, N] @ W[N, K]      (`transposed_b=True`)

Function names, arguments and error behaviour follow the reference module (`feather_ops/int8_convrot.py`).

On sm_100a the released `[N, K]` matrix is itself what the tensor cores want: the copy engine's 128 x 128 byte boxes of it
are K-major (forward) or MN-major (backward) operands as they land, while the micro-tile prepack has to pass through a
re-layout stage in shared memory, which bounds that kernel. So the `weight_packed=False` calls, for which the reference
permutes the weight on every call, run `int8_scaled_mm_plain` on the weight as it is, and that is the faster of the two
paths here; `weight_packed=True` keeps accepting the reference's prepack unchanged. Both give the same bits.
"""

import os
import weakref

import torch
from torch.library import custom_op

from .scaled_mm import sm_count
from .tiles import INT8_UMMA

CONVROT_GROUP = 256  # the quantizer implements the regular Hadamard over 256 channels only

_TILE_N256 = (4, 4, 2, 4, 4)
_TILE_N128 = (2, 4, 2, 4, 2)
_TILE_N64 = (2, 2, 2, 2, 2)
# Measured time of one wave of tiles per 128-deep k block, in microseconds (N = K = 3072 sweeps over M): 256-wide
# tiles run as 256 x 256 tiles on CTA pairs (also for a single row tile), the others as 128-row tiles on single
# CTAs, whose weight re-layout is much slower.
_WAVE_COST_US = {256: 0.47, 128: 0.98, 64: 0.78}
_TILE_OF_WIDTH = {256: _TILE_N256, 128: _TILE_N128, 64: _TILE_N64}


def select_int8_config(M: int, N: int, K: int, transposed_b: bool):
    """Tile tuple for one `(M, N, K)` cell and direction (`N`/`K` are the weight's output/input axes, as
    in the reference's `select_int8_config`, `feather_ops/int8_convrot.py:28-82`). Same rule as `scaled_mm`:
    waves of tiles times the measured cost of a wave, CTA pairs (74) for the 256-wide tile, single CTAs (148)
    for the others."""
    out = K if transposed_b else N
    sms = sm_count()
    best = None
    for width in (256, 128, 64):
        if width == 256:
            cost = -(-(-(-M // 256) * -(-out // 256)) // (sms // 2)) * _WAVE_COST_US[256]
        else:
            cost = -(-(-(-M // 128) * -(-out // width)) // sms) * _WAVE_COST_US[width]
        if best is None or cost < best[0] - 1e-9:
            best = (cost, width)
    return _TILE_OF_WIDTH[best[1]]


def prepack_int8_weight(weight: torch.Tensor) -> torch.Tensor:
    """`[N, K]` int8 -> `[K // 4, N // 4, 4, 4]`: micro-tile `(k4, n4)` holds `W[4 n4 : 4 n4 + 4, 4 k4 : 4 k4 + 4]`
    with `k` fastest. A pure byte permutation."""
    n, k = weight.shape
    return weight.view(n // 4, 4, k // 4, 4).permute(2, 0, 1, 3).contiguous()


def unpack_int8_weight(prepacked: torch.Tensor) -> torch.Tensor:
    """Back to the released `[N, K]` form."""
    if prepacked.ndim != 4 or tuple(prepacked.shape[2:]) != (4, 4):
        raise ValueError(f"prepacked weight must end in (4, 4), got {tuple(prepacked.shape)}")
    k4, n4 = prepacked.shape[:2]
    return prepacked.permute(1, 2, 0, 3).reshape(n4 * 4, k4 * 4)


def quantize_convrot_activation(x: torch.Tensor, rotate: bool = True, col_scale: torch.Tensor | None = None):
    """Rotate each 256-wide group by the regular Hadamard and quantize per row to int8, in one kernel.

    `x` is `[M, K]` bf16/fp16 with `K % 256 == 0`. `rotate=False` quantizes as is (the input-gradient path,
    which rotates after the GEMM) and may fold a `[K]` float32 `col_scale` in first. Returns
    `(q int8 [M, K], scale float32 [M])` with `q * scale` the normalized rotated values.
    """
    q = torch.empty(x.shape, device=x.device, dtype=torch.int8)
    scale = torch.empty(x.shape[0], device=x.device, dtype=torch.float32)
    folded = None if col_scale is None else col_scale.reshape(-1).to(device=x.device, dtype=torch.float32).contiguous()
    torch.ops.feather_ops.convrot_quantize.default(x, folded, q, scale, rotate)
    return q, scale


def _launch(a, weight_prepacked, a_scale, weight_scale, bias, out, transposed_b, tile) -> None:
    torch.ops.feather_ops.int8_scaled_mm.default(
        a,
        weight_prepacked.reshape(-1),
        a_scale.reshape(-1).to(torch.float32),
        None if weight_scale is None else weight_scale.reshape(-1).to(torch.float32),
        bias,
        out,
        transposed_b,
        *tile,
    )


@custom_op("feather_ops::int8_scaled_mm_auto", mutates_args=("out",))
def _int8_scaled_mm_auto(
    a: torch.Tensor,
    weight_prepacked: torch.Tensor,
    a_scale: torch.Tensor,
    weight_scale: torch.Tensor | None,
    bias: torch.Tensor | None,
    out: torch.Tensor,
    transposed_b: bool,
) -> None:
    """Tile choice + launch as one opaque node."""
    other = weight_prepacked.numel() // a.shape[1]
    n, k = (a.shape[1], other) if transposed_b else (other, a.shape[1])
    _launch(a, weight_prepacked, a_scale, weight_scale, bias, out, transposed_b, select_int8_config(a.shape[0], n, k, transposed_b))


def int8_scaled_mm(a, weight_prepacked, a_scale, weight_scale=None, bias=None, out_dtype=torch.bfloat16, transposed_b=False, tile=None):
    """`A @ W^T` (or `A @ W` with `transposed_b`) with a per-row activation scale and, forward only, a
    per-output-channel weight scale and a bias. `a` is `[M, K]` int8, `weight_prepacked` the micro-tile
    prepack in any shape. Returns `[M, N_out]` in `out_dtype`."""
    m, k = a.shape
    if k == 0:
        raise ValueError("a must have a nonzero contraction axis")
    if transposed_b and weight_scale is not None:
        raise ValueError("transposed_b folds the weight scale into the activation quantization, so weight_scale must be None")
    out = torch.empty((m, weight_prepacked.numel() // k), device=a.device, dtype=out_dtype)
    if tile is None:
        _int8_scaled_mm_auto(a, weight_prepacked, a_scale, weight_scale, bias, out, transposed_b)
    else:
        _launch(a, weight_prepacked, a_scale, weight_scale, bias, out, transposed_b, tile)
    return out


# FEATHER_INT8_PLAIN_OFF=1 sends `weight_packed=False` calls through a per-call prepack again (A/B measurements). Read once.
_PLAIN_OFF = os.environ.get("FEATHER_INT8_PLAIN_OFF", "") == "1"


@custom_op("feather_ops::int8_scaled_mm_plain_auto", mutates_args=("out",))
def _int8_scaled_mm_plain(
    a: torch.Tensor,
    weight: torch.Tensor,
    a_scale: torch.Tensor,
    weight_scale: torch.Tensor | None,
    bias: torch.Tensor | None,
    out: torch.Tensor,
    transposed_b: bool,
) -> None:
    """The launch as one opaque node."""
    torch.ops.feather_ops.int8_scaled_mm_plain.default(a, weight, a_scale, weight_scale, bias, out, transposed_b)


def plain_weight_eligible(weight: torch.Tensor, transposed_b: bool) -> bool:
    """Whether `int8_scaled_mm_plain` takes this `[N, K]` weight. It does at any number of rows: with at most 64 the
    warp-MMA kernel reads the rows of the weight as fast as it reads a prepack (5-30 us), and the permute that a prepack per
    call costs (25 us for a 3072 x 3072 weight, 85-105 us for 12288 x 3072) is several times that."""
    if _PLAIN_OFF or weight.ndim != 2 or weight.dtype != torch.int8 or not weight.is_contiguous() or weight.data_ptr() % 16:
        return False
    n, k = weight.shape
    if k % 16 or n % (16 if transposed_b else 4):
        return False
    return True


def int8_scaled_mm_plain(a, weight, a_scale, weight_scale=None, bias=None, out_dtype=torch.bfloat16, transposed_b=False):
    """`int8_scaled_mm` over the released row-major `[N, K]` weight instead of its prepack: `A @ W^T` with both scales and the
    bias, or `A @ W` (`transposed_b`) with the row scale only. Same bits as the prepacked call. No counterpart in the
    reference, whose kernels read the prepack only."""
    if transposed_b and weight_scale is not None:
        raise ValueError("transposed_b folds the weight scale into the activation quantization, so weight_scale must be None")
    n, k = weight.shape
    out = torch.empty((a.shape[0], k if transposed_b else n), device=a.device, dtype=out_dtype)
    _int8_scaled_mm_plain(
        a,
        weight,
        a_scale.reshape(-1).to(torch.float32),
        None if weight_scale is None else weight_scale.reshape(-1).to(torch.float32),
        bias,
        out,
        transposed_b,
    )
    return out


class _UnpackedWeightCache:
    """Row-major copies of prepacked weights, one per weight version. An entry only hits for the tensor object that created it
    (a weak reference is kept): a freed tensor's address can come back with the same shape. An entry is dropped when that tensor
    is freed, so the cache does not outlive the weights."""

    def __init__(self, max_entries: int) -> None:
        self._max_entries = max_entries
        self._entries: dict = {}

    def get(self, packed: torch.Tensor, n_out: int, k_in: int) -> torch.Tensor:
        version = None if torch.is_inference_mode_enabled() else getattr(packed, "_version", None)
        key = (packed.data_ptr(), packed.device, n_out, k_in)
        hit = self._entries.get(key)
        if hit is not None:
            owner = hit[1]()
            if owner is not None and owner.data_ptr() == packed.data_ptr() and hit[2] == version:
                return hit[0]
        while key not in self._entries and len(self._entries) >= self._max_entries:
            self._entries.pop(next(iter(self._entries)))
        plain = unpack_int8_weight(packed.reshape(k_in // 4, n_out // 4, 4, 4)).contiguous()
        entries = self._entries
        # one copy per weight: a new version replaces the old one, and the copy goes when the prepacked tensor does
        self._entries[key] = (plain, weakref.ref(packed, lambda _ref, key=key: entries.pop(key, None)), version)
        return plain


_UNPACKED_CACHE: _UnpackedWeightCache | None = _UnpackedWeightCache(256) if os.environ.get("FEATHER_INT8_UNPACK_CACHE", "") == "1" else None
_UNPACKED_MIN_ROWS = 65  # the forward product of at most 64 rows over a prepack runs on the warp-MMA kernel, which is faster still


def cache_unpacked_weights(enabled: bool = True, max_entries: int = 256) -> None:
    """Opt in to (or out of) row-major copies of the prepacked weights that `convrot_int8_linear` / `convrot_int8_dgrad`
    receive with `weight_packed=True`: the first call with a weight version un-permutes it once, later calls run the faster
    plain-weight kernel on the copy (same bits). Costs the weight's bytes a second time, hence off by default (the
    environment variable FEATHER_INT8_UNPACK_CACHE=1 turns it on at import). No counterpart in the reference."""
    global _UNPACKED_CACHE
    _UNPACKED_CACHE = _UnpackedWeightCache(max_entries) if enabled else None


def _unpacked_or_none(packed: torch.Tensor, n_out: int, k_in: int, rows: int, transposed_b: bool):
    if _UNPACKED_CACHE is None or _PLAIN_OFF or (not transposed_b and rows < _UNPACKED_MIN_ROWS):
        return None
    if n_out % (16 if transposed_b else 4) or k_in % 16 or not packed.is_contiguous():
        return None
    return _UNPACKED_CACHE.get(packed, n_out, k_in)


_HADAMARD_CACHE: dict = {}


def build_hadamard(size: int = CONVROT_GROUP, device="cpu", dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Normalized regular Hadamard of a power-of-four `size`: the Kronecker power of the 4x4 matrix whose rows
    have a single -1 on the anti-diagonal, divided by `sqrt(size)`. Symmetric and orthogonal. Cached."""
    probe = size
    while probe > 1 and probe % 4 == 0:
        probe //= 4
    if probe != 1:
        raise ValueError(f"the regular Hadamard size must be a power of four, got {size}")
    key = (size, str(device), dtype)
    if key not in _HADAMARD_CACHE:
        base = torch.ones((4, 4), dtype=dtype, device=device)
        for i in range(4):
            base[i, 3 - i] = -1
        h = base
        while h.shape[0] < size:
            h = torch.kron(h, base)
        _HADAMARD_CACHE[key] = h / (size**0.5)
    return _HADAMARD_CACHE[key]


def rotate(x: torch.Tensor, hadamard: torch.Tensor, groupsize: int = CONVROT_GROUP) -> torch.Tensor:
    """Group-wise `x @ H^T` along the last axis (its own inverse, `H` being orthogonal and symmetric)."""
    width = x.shape[-1]
    if width % groupsize:
        raise ValueError(f"last axis {width} is not divisible by the group size {groupsize}")
    grouped = x.reshape(*x.shape[:-1], width // groupsize, groupsize)
    return torch.matmul(grouped, hadamard.T.to(dtype=x.dtype, device=x.device)).reshape(x.shape)


def quantize_rowwise_int8(x: torch.Tensor, scale=None):
    """Per-row int8 codes of an already rotated tensor, `scale = absmax / 127` unless given. Codes are clamped
    to the symmetric range [-127, 127]."""
    if scale is None:
        scale = (x.abs().amax(dim=-1).float() / 127.0).clamp(min=1e-30)
    elif isinstance(scale, torch.Tensor):
        scale = scale.reshape(-1).to(device=x.device, dtype=torch.float32)
    else:
        scale = torch.tensor(scale, device=x.device, dtype=torch.float32)
    per_row = scale.reshape(-1, *([1] * (x.ndim - 1)))
    return torch.clamp(torch.round(x.float() / per_row), -127.0, 127.0).to(torch.int8), scale


def quantize_convrot_weight(weight: torch.Tensor, groupsize: int = CONVROT_GROUP, rotate_dtype: torch.dtype | None = None):
    """Offline weight quantization: rotate per group with a matmul (in `rotate_dtype`, default the weight's
    own dtype), then `quantize_rowwise_int8`."""
    hadamard = build_hadamard(groupsize, device=weight.device, dtype=torch.float32)
    return quantize_rowwise_int8(rotate(weight.to(rotate_dtype or weight.dtype), hadamard, groupsize))


def dequantize_convrot_weight(q: torch.Tensor, scale: torch.Tensor, groupsize: int = CONVROT_GROUP) -> torch.Tensor:
    """`code * scale` rotated back to the original basis, float32."""
    hadamard = build_hadamard(groupsize, device=q.device, dtype=torch.float32)
    return rotate(q.float() * scale.reshape(-1, 1), hadamard, groupsize)


def convrot_int8_supported(shape, groupsize: int = CONVROT_GROUP, backward: bool = True) -> tuple[bool, str]:
    """Whether the kernels can run an `[N, K]` ConvRot weight, with the reason if not."""
    n, k = int(shape[0]), int(shape[1])
    if groupsize != CONVROT_GROUP:
        return False, f"only group size {CONVROT_GROUP} is implemented, got {groupsize}"
    if k % groupsize:
        return False, f"in_features {k} is not a multiple of the group size {groupsize}"
    if k % 16:
        return False, f"in_features {k} is not a multiple of the 16-wide reduction step"
    if n % 4:
        return False, f"out_features {n} is not a multiple of 4"
    if backward and n % 16:
        return False, f"out_features {n} is not a multiple of 16, which the input gradient contracts"
    return True, ""


def _weight_extent(weight: torch.Tensor, weight_scale: torch.Tensor) -> tuple[int, int]:
    """`(N, K)` from the byte count and the number of per-channel scales (works for both weight layouts)."""
    n_out = int(weight_scale.numel())
    if n_out == 0 or weight.numel() % n_out:
        raise ValueError(f"weight of {weight.numel()} bytes does not divide into {n_out} output channels")
    return n_out, int(weight.numel() // n_out)


def convrot_int8_linear(x, weight, weight_scale, bias=None, out_dtype=torch.bfloat16, groupsize=CONVROT_GROUP, rotate_activation=True, weight_packed=False):
    """Forward `x @ W^T + bias`: fused rotate+quantize of `x`, then the int8 GEMM with both scales."""
    n_out, k_in = _weight_extent(weight, weight_scale)
    if x.shape[-1] != k_in:
        raise ValueError(f"activation has {x.shape[-1]} features, the weight {k_in}")
    q, scale = quantize_convrot_activation(x.reshape(-1, k_in), rotate=rotate_activation)
    plain = _unpacked_or_none(weight, n_out, k_in, q.shape[0], False) if weight_packed else (weight if plain_weight_eligible(weight, False) else None)
    if plain is not None:
        out = int8_scaled_mm_plain(q, plain, scale, weight_scale.reshape(-1), bias, out_dtype, False)
    else:
        packed = weight if weight_packed else prepack_int8_weight(weight)
        out = int8_scaled_mm(q, packed, scale, weight_scale.reshape(-1), bias, out_dtype, False)
    return out.reshape(*x.shape[:-1], n_out)


def convrot_int8_dgrad(grad_out, weight, weight_scale, out_dtype=torch.bfloat16, groupsize=CONVROT_GROUP, rotate_activation=True, weight_packed=False):
    """Input gradient `g @ W` (then rotated back): the per-channel weight scale cannot leave a sum over
    channels, so it is folded into the row-wise quantization of `grad_out`."""
    n_out, k_in = _weight_extent(weight, weight_scale)
    q, scale = quantize_convrot_activation(grad_out.reshape(-1, grad_out.shape[-1]), False, col_scale=weight_scale.reshape(-1))
    plain = _unpacked_or_none(weight, n_out, k_in, q.shape[0], True) if weight_packed else (weight if plain_weight_eligible(weight, True) else None)
    if plain is not None:
        out = int8_scaled_mm_plain(q, plain, scale, None, None, out_dtype, True)
    else:
        packed = weight if weight_packed else prepack_int8_weight(weight)
        out = int8_scaled_mm(q, packed, scale, None, None, out_dtype, True)
    if rotate_activation:
        out = rotate(out, build_hadamard(groupsize, device=out.device, dtype=out.dtype), groupsize)
    return out.reshape(*grad_out.shape[:-1], k_in)


def umma_tile(tile):
    """The sm_100a tile the tuple runs on."""
    return INT8_UMMA[tuple(tile)]
