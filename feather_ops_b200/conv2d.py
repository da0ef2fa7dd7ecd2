"""3x3, stride 1, padding 1 NCHW conv2d (bf16 / fp16) on the sm_100a implicit-GEMM kernel.

`conv2d` mirrors `torch.nn.functional.conv2d` and hands anything the kernel does not cover to torch, so it
is a safe drop-in; `conv3x3_eligibility` gives the same decision as a reason string for logs. The weight
is prepacked once per weight version into the kernel's k order `(16-channel group, tap, channel % 16)`.
API and reason strings follow the reference module (`feather_ops/conv2d.py`).

Backend policy on B200 (`select_backend`): the reference delegates fp16 to MIOpen's Winograd and keeps
bf16, which is a property of gfx11. Here both dtypes run the kernel whenever it can tile the shape, and
only `C_in % 8 != 0` is delegated to the vendor library path (`"miopen"` keeps its name and means
cuDNN through `F.conv2d`).
"""

import contextlib
import weakref

import torch
import torch.nn.functional as F
from torch.library import custom_op

from .tiles import CONV_PREFETCH_MIN_C_IN, CONV_TILES, conv_block_sizes

_TILE_TWO_ROWS_128 = (4, 4, 2, 2, 2)  # 128 output channels x 2 rows x 128 pixels
_TILE_ONE_ROW_256 = (4, 4, 2, 4, 1)   # 128 x 256 pixels of one row
_TILE_ONE_ROW_128 = (4, 4, 2, 2, 1)
_TILE_ONE_ROW_64 = (2, 2, 2, 2, 1)


def select_conv3x3_config(c_out: int, width: int):
    """`(warps_m, warps_n, repeat_m, repeat_n, rows)` for one convolution, or None if `width < 1`.

    The sm_100a kernel tiles any `C_out` (128 channels per CTA, the tail zero filled) and any width
    (stores are predicated), so unlike the reference's selector this one only picks the pixel-segment
    shape: two rows of 128 pixels when the image is at least 128 wide and even (a 4-row halo for 2
    output rows reads the input twice instead of three times), else one row of the narrowest segment
    that covers the width. With at most 128 output channels (one CTA per tile) and rows that the copy
    engine can stage (`width % 8 == 0`), one row of 256 pixels is faster when 256-pixel segments waste at most an
    eighth of the row: its 256-wide UMMAs read a third less shared memory per flop than two 128-wide ones
    (measured at 128 channels: 512 x 512 92 against 100 us, 256 x 256 29 against 33; 64 channels at 512 x 512 49 against 52).
    """
    if width < 1:
        return None
    if c_out <= 128 and width >= 256 and width % 8 == 0 and (-width % 256) * 8 <= width:
        return _TILE_ONE_ROW_256
    if width >= 128 and width % 2 == 0:
        return _TILE_TWO_ROWS_128
    if width > 128:
        return _TILE_ONE_ROW_256
    return _TILE_ONE_ROW_128 if width > 64 else _TILE_ONE_ROW_64


def conv3x3_prefetch(tile, c_in: int) -> bool:
    """The reference's register-prefetch switch. The sm_100a pipeline always runs ahead, so the flag is
    accepted by the operator and ignored; the rule is kept for API compatibility."""
    block_m, block_n, rows = conv_block_sizes(tile)
    if c_in < CONV_PREFETCH_MIN_C_IN or block_n < 128:
        return False
    return not (rows == 2 and block_m == 64)


def select_backend(dtype: torch.dtype, c_in: int, c_out: int, height: int, width: int) -> str:
    """`"kernel"`, `"miopen"` (vendor library through `F.conv2d` with cuDNN forced on) or `"torch"`."""
    del height
    if dtype in (torch.bfloat16, torch.float16) and c_in % 8 == 0 and select_conv3x3_config(c_out, width) is not None:
        return "kernel"
    if dtype in (torch.bfloat16, torch.float16):
        return "miopen"
    return "torch"


@contextlib.contextmanager
def miopen_flags():
    """`cudnn.enabled = True`, `cudnn.benchmark = False` for one call, then restored."""
    saved = (torch.backends.cudnn.enabled, torch.backends.cudnn.benchmark)
    torch.backends.cudnn.enabled, torch.backends.cudnn.benchmark = True, False
    try:
        yield
    finally:
        torch.backends.cudnn.enabled, torch.backends.cudnn.benchmark = saved


def conv2d_miopen(input, weight, bias, stride=1, padding=0, dilation=1, groups: int = 1):
    """`F.conv2d` with the vendor convolution library forced on, for the delegated shapes."""
    with miopen_flags():
        return F.conv2d(input, weight, bias, stride, padding, dilation, groups)


def prepack_conv2d_weight_3x3(weight: torch.Tensor) -> torch.Tensor:
    """`[C_out, C_in, 3, 3]` -> `[ceil(C_in / 16) * 18, C_out, 8]`.

    Row `g * 18 + tap * 2 + half` holds, for every output channel, input channels
    `g * 16 + half * 8 .. + 7` of tap `tap = kh * 3 + kw`. `C_in` is zero padded to a multiple of 16.
    """
    if weight.ndim != 4 or tuple(weight.shape[2:]) != (3, 3):
        raise ValueError(f"expected a [C_out, C_in, 3, 3] weight, got {tuple(weight.shape)}")
    c_out, c_in = weight.shape[:2]
    groups = (c_in + 15) // 16
    w = weight.detach()
    if groups * 16 != c_in:
        w = F.pad(w, (0, 0, 0, 0, 0, groups * 16 - c_in))
    # [m, g, half, j, tap] -> [g, tap, half, m, j]
    return w.reshape(c_out, groups, 2, 8, 9).permute(1, 4, 2, 0, 3).reshape(groups * 18, c_out, 8).contiguous()


def _launch(x, w_packed, bias, out, tile, prefetch: bool) -> None:
    torch.ops.feather_ops.conv2d_3x3.default(x, w_packed, bias, out, *tile, prefetch)


@custom_op("feather_ops::conv3x3_auto", mutates_args=("out",))
def _conv3x3_auto(x: torch.Tensor, w_packed: torch.Tensor, bias: torch.Tensor | None, out: torch.Tensor) -> None:
    """Tile choice + launch as one opaque node."""
    tile = select_conv3x3_config(w_packed.shape[1], x.shape[3])
    if tile is None:
        raise RuntimeError(f"no kernel tile for C_out={w_packed.shape[1]} W={x.shape[3]}")
    _launch(x, w_packed, bias, out, tile, conv3x3_prefetch(tile, x.shape[1]))


def conv3x3_prepacked(x, w_packed, bias=None, tile=None, prefetch=None):
    """3x3 / stride 1 / padding 1 conv over a prepacked weight, no fallback. `C_in % 8 == 0`."""
    out = torch.empty((x.shape[0], w_packed.shape[1], x.shape[2], x.shape[3]), device=x.device, dtype=x.dtype)
    if tile is None:
        _conv3x3_auto(x, w_packed, bias, out)
    else:
        _launch(x, w_packed, bias, out, tile, conv3x3_prefetch(tile, x.shape[1]) if prefetch is None else prefetch)
    return out


def _pair(value) -> tuple[int, ...]:
    return (value, value) if isinstance(value, int) else tuple(int(v) for v in value)


def conv3x3_eligibility(x, weight, bias=None, stride=1, padding=1, dilation=1, groups: int = 1) -> str | None:
    """None if `conv3x3_prepacked` can run this call, else a short, stable reason string."""
    if groups != 1:
        return f"{groups} groups"
    if x.ndim != 4:
        return f"input has {x.ndim} dimensions"
    if x.dtype not in (torch.bfloat16, torch.float16) or weight.dtype != x.dtype:
        return f"dtype {x.dtype} / weight {weight.dtype}"
    if not (x.is_cuda and weight.is_cuda and x.device == weight.device):
        return "input and weight are not on the same CUDA device"
    if _pair(stride) != (1, 1) or _pair(dilation) != (1, 1):
        return f"stride {_pair(stride)}, dilation {_pair(dilation)}"
    if _pair(padding) != (1, 1):
        return f"padding {_pair(padding)}"
    if tuple(weight.shape[2:]) != (3, 3) or weight.shape[1] != x.shape[1]:
        return f"weight shape {tuple(weight.shape)}"
    if not (x.is_contiguous() and weight.is_contiguous()):
        return "input or weight is not contiguous"
    if torch.is_grad_enabled() and (x.requires_grad or weight.requires_grad):
        return "autograd is enabled"
    if bias is not None and (bias.dtype != x.dtype or bias.numel() != weight.shape[0]):
        return f"bias {bias.dtype} / {bias.numel()} elements"
    return None


def weight_cache_key(weight: torch.Tensor) -> tuple:
    """Identity of a weight version: storage address, version counter (absent under inference mode), dtype, device."""
    version = None if torch.is_inference_mode_enabled() else getattr(weight, "_version", None)
    return (weight.data_ptr(), version, weight.dtype, weight.device)


class _PackedWeightCache:
    """Prepack cache of the functional API. An entry only hits for the tensor object that created it (a weak
    reference is kept), because a freed tensor's address can come back at version 0 with the same shape."""

    def __init__(self, max_entries: int = 128) -> None:
        self._max_entries = max_entries
        self._entries: dict = {}

    def get(self, weight: torch.Tensor) -> torch.Tensor:
        key = (*weight_cache_key(weight), weight.shape)
        hit = self._entries.get(key)
        if hit is not None:
            owner = hit[1]()
            if owner is not None and owner.data_ptr() == weight.data_ptr():
                return hit[0]
        while len(self._entries) >= self._max_entries:
            self._entries.pop(next(iter(self._entries)))
        packed = prepack_conv2d_weight_3x3(weight)
        self._entries[key] = (packed, weakref.ref(weight))
        return packed


_PACKED_CACHE = _PackedWeightCache()


def conv2d(input, weight, bias=None, stride=1, padding=0, dilation=1, groups: int = 1):
    """Drop-in for `torch.nn.functional.conv2d`: the kernel for eligible 3x3 / stride 1 / padding 1 calls,
    torch for everything else."""
    if conv3x3_eligibility(input, weight, bias, stride, padding, dilation, groups) is not None:
        return F.conv2d(input, weight, bias, stride, padding, dilation, groups)
    backend = select_backend(input.dtype, input.shape[1], weight.shape[0], input.shape[2], input.shape[3])
    if backend == "kernel":
        return conv3x3_prepacked(input, _PACKED_CACHE.get(weight), None if bias is None else bias.contiguous())
    if backend == "miopen":
        return conv2d_miopen(input, weight, bias, stride, padding, dilation, groups)
    return F.conv2d(input, weight, bias, stride, padding, dilation, groups)


assert all(tile in CONV_TILES for tile in (_TILE_TWO_ROWS_128, _TILE_ONE_ROW_256, _TILE_ONE_ROW_128, _TILE_ONE_ROW_64))
