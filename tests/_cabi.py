"""Calls into libfeather_ops_b200.so through ctypes with raw device pointers, as a foreign host would."""

import torch

from feather_ops_b200 import _lib


def _ptr(t):
    return None if t is None else t.data_ptr()


# Guard bands: every output buffer handed to a launcher sits between two bands of a sentinel byte, and
# `assert_clean` (called after the launches of a test) checks that no band was written. A store one row or a few
# bytes past a ragged tile would otherwise land in a neighbouring live tensor and pass every parity check.
GUARD_BYTES = 4096
_SENTINEL = 0xA5
_guards: list = []


def guarded_empty(shape, device, dtype) -> torch.Tensor:
    """An uninitialized tensor of `shape` with sentinel bands before and after it (checked by `check_guards`)."""
    count = 1
    for extent in shape:
        count *= int(extent)
    nbytes = count * torch.empty((), dtype=dtype).element_size()
    padded = (nbytes + 15) // 16 * 16
    buffer = torch.full((2 * GUARD_BYTES + padded,), _SENTINEL, device=device, dtype=torch.uint8)
    _guards.append((buffer, nbytes))
    return buffer[GUARD_BYTES : GUARD_BYTES + nbytes].view(dtype).view(*shape)


def check_guards() -> None:
    """Every sentinel band registered since the last check is intact (synchronizes)."""
    pending, _guards[:] = list(_guards), []
    for buffer, nbytes in pending:
        before = buffer[:GUARD_BYTES]
        after = buffer[GUARD_BYTES + nbytes :]
        assert bool((before == _SENTINEL).all().item()), "a launch wrote before the start of its output buffer"
        assert bool((after == _SENTINEL).all().item()), "a launch wrote past the end of its output buffer"


def _stream():
    return torch.cuda.current_stream().cuda_stream


def scaled_mm(a, b_prepacked, scale, bias, out_dtype, tile=(1, 8, 4, 8, 2, 0)):
    m, k = a.shape
    n = b_prepacked.shape[1]
    c = guarded_empty((m, n), a.device, out_dtype)
    ok = _lib.load().launch_scaled_mm(
        _ptr(a), _ptr(b_prepacked), _ptr(scale), _ptr(bias), _ptr(c), m, n, k, int(scale is not None), int(bias is not None),
        b_prepacked.dtype == torch.float8_e5m2, a.dtype == torch.bfloat16, out_dtype == torch.bfloat16, *tile[:5], bool(tile[5]), _stream(),
    )
    assert ok, "launch_scaled_mm refused the call"
    return c


def convrot_quantize(x, rotate=True, col_scale=None):
    m, k = x.shape
    q = guarded_empty((m, k), x.device, torch.int8)
    scale = guarded_empty((m,), x.device, torch.float32)
    ok = _lib.load().launch_convrot_quantize(_ptr(x), _ptr(col_scale), _ptr(q), _ptr(scale), m, k, int(x.dtype == torch.float16), rotate, _stream())
    assert ok, "launch_convrot_quantize refused the call"
    return q, scale


def int8_scaled_mm(a, w_prepacked, a_scale, w_scale, bias, out_dtype, transposed_b, n_out, tile=(4, 4, 2, 4, 4)):
    m, kc = a.shape
    c = guarded_empty((m, n_out), a.device, out_dtype)
    weight_out = kc if transposed_b else n_out
    inner = weight_out // 4
    stride_kc, stride_out = (1, inner) if transposed_b else (inner, 1)
    ok = _lib.load().launch_int8_scaled_mm(
        _ptr(a), _ptr(w_prepacked), _ptr(a_scale), _ptr(w_scale), _ptr(bias), _ptr(c), m, n_out, kc, stride_kc, stride_out, transposed_b, *tile,
        int(out_dtype == torch.bfloat16), _stream(),
    )
    assert ok, "launch_int8_scaled_mm refused the call"
    return c


def int8_scaled_mm_plain(a, weight, a_scale, w_scale, bias, out_dtype, transposed_b):
    """The int8 GEMM over the row-major `[N, K]` weight. Returns None if the launcher refuses the call."""
    n, k = weight.shape
    c = guarded_empty((a.shape[0], k if transposed_b else n), a.device, out_dtype)
    ok = _lib.load().launch_int8_scaled_mm_plain(
        _ptr(a), _ptr(weight), _ptr(a_scale), _ptr(w_scale), _ptr(bias), _ptr(c), a.shape[0], n, k, transposed_b, int(out_dtype == torch.bfloat16), _stream()
    )
    return c if ok else None


def conv3x3(x, w_prepacked, bias, tile=(4, 4, 2, 4, 1)):
    b, c_in, h, w = x.shape
    c_out = w_prepacked.shape[1]
    y = guarded_empty((b, c_out, h, w), x.device, x.dtype)
    rc = _lib.load().feather_conv3x3_launch(
        _ptr(x), _ptr(w_prepacked), _ptr(bias), _ptr(y), b, c_in, c_out, h, w, int(bias is not None), *tile, int(x.dtype == torch.bfloat16), 0, _stream()
    )
    assert rc == 0, f"feather_conv3x3_launch returned {rc}"
    return y


def assert_clean(symbol):
    """No bounded device wait ran out and no launch wrote outside its output buffer (also synchronizes)."""
    assert _lib.read_status(symbol) == (0, 0)
    check_guards()


def scaled_mm_splitk_wide(a, b_prepacked, scale, bias, out_dtype, block_n, splits, partials=None, counters=None):
    """Split-K launcher of the one-CTA kernel (128 x block_n tiles) with caller-provided scratch. Returns (c, partials, counters)."""
    m, k = a.shape
    n = b_prepacked.shape[1]
    lib = _lib.load()
    floats = lib.feather_scaled_mm_splitk_wide_partial_floats(m, n, k, block_n, splits)
    if partials is None:
        partials = guarded_empty((max(int(floats), 1),), a.device, torch.float32)
    if counters is None:
        counters = torch.zeros(max(int(lib.feather_scaled_mm_splitk_wide_counters(m, n, block_n)), 1), device=a.device, dtype=torch.int32)
    assert partials.numel() >= floats
    c = guarded_empty((m, n), a.device, out_dtype)
    ok = lib.launch_scaled_mm_splitk_wide(
        _ptr(a), _ptr(b_prepacked), _ptr(scale), _ptr(bias), _ptr(c), m, n, k, int(scale is not None), int(bias is not None),
        b_prepacked.dtype == torch.float8_e5m2, a.dtype == torch.bfloat16, out_dtype == torch.bfloat16, block_n, splits, _ptr(partials), _ptr(counters),
        _stream(),
    )
    assert ok, "launch_scaled_mm_splitk_wide refused the call"
    return c, partials, counters


def scaled_mm_splitk(a, b_prepacked, scale, bias, out_dtype, splits, partials=None, counters=None):
    """Skinny split-K launcher with caller-provided scratch. Returns (c, partials, counters)."""
    m, k = a.shape
    n = b_prepacked.shape[1]
    lib = _lib.load()
    floats = lib.feather_scaled_mm_splitk_partial_floats(m, n, k, splits)
    if partials is None:
        partials = guarded_empty((max(int(floats), 1),), a.device, torch.float32)
    if counters is None:
        counters = torch.zeros(-(-n // 64), device=a.device, dtype=torch.int32)
    assert partials.numel() >= floats
    c = guarded_empty((m, n), a.device, out_dtype)
    ok = lib.launch_scaled_mm_splitk(
        _ptr(a), _ptr(b_prepacked), _ptr(scale), _ptr(bias), _ptr(c), m, n, k, int(scale is not None), int(bias is not None),
        b_prepacked.dtype == torch.float8_e5m2, a.dtype == torch.bfloat16, out_dtype == torch.bfloat16, splits, _ptr(partials), _ptr(counters), _stream(),
    )
    assert ok, "launch_scaled_mm_splitk refused the call"
    return c, partials, counters
