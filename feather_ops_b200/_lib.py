"""ctypes view of the C-ABI library (`libfeather_ops_b200.so`), for callers that bind the launchers directly.

The torch operators do not go through here (the `_C` extension links the library), but the parity tests
and the benchmark call the C ABI through these prototypes, exactly as a foreign-language host would.
There is no fallback: if the library is missing, loading raises with the build command.
"""

import ctypes
import pathlib

_PATH = pathlib.Path(__file__).resolve().parent / "libfeather_ops_b200.so"

_c_bool = ctypes.c_bool
_c_int = ctypes.c_int
_i64 = ctypes.c_int64
_ptr = ctypes.c_void_p

# name -> (restype, argtypes), in the order of include/feather_ops_b200.h
PROTOTYPES = {
    "launch_scaled_mm": (
        _c_bool,
        [_ptr, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _c_int, _c_int, _c_bool, _c_bool, _c_bool, _c_int, _c_int, _c_int, _c_int, _c_int, _c_bool, _ptr],
    ),
    "launch_scaled_mm_splitk": (
        _c_bool,
        [_ptr, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _c_int, _c_int, _c_bool, _c_bool, _c_bool, _c_int, _ptr, _ptr, _ptr],
    ),
    "launch_scaled_mm_splitk_wide": (
        _c_bool,
        [_ptr, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _c_int, _c_int, _c_bool, _c_bool, _c_bool, _c_int, _c_int, _ptr, _ptr, _ptr],
    ),
    "feather_scaled_mm_splitk_wide_partial_floats": (_i64, [_i64, _i64, _i64, _c_int, _c_int]),
    "feather_scaled_mm_splitk_wide_counters": (_i64, [_i64, _i64, _c_int]),
    "feather_scaled_mm_splitk_partial_floats": (_i64, [_i64, _i64, _i64, _c_int]),
    "launch_scaled_mm_splitk_static": (
        _c_int,
        [_ptr, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _c_int, _c_int, _c_bool, _c_bool, _c_bool, _c_int, _ptr, ctypes.c_char_p, ctypes.c_size_t],
    ),
    "feather_scaled_mm_set_sm_margin": (_c_int, [_c_int]),
    "launch_interleave_slabs": (_c_bool, [_ptr, _ptr, _i64, _i64, _i64, _ptr]),
    "feather_scaled_mm_pair_tile_width": (_c_int, [_i64, _i64, _c_int]),
    "feather_scaled_mm_status": (_c_int, [_ptr]),
    "launch_convrot_quantize": (_c_bool, [_ptr, _ptr, _ptr, _ptr, _i64, _i64, _c_int, _c_bool, _ptr]),
    "launch_int8_scaled_mm": (
        _c_bool,
        [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _i64, _c_bool, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _ptr],
    ),
    "launch_int8_scaled_mm_plain": (_c_bool, [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _c_bool, _c_int, _ptr]),
    "feather_int8_plain_tile_width": (_c_int, [_i64, _i64, _c_int, _c_bool]),
    "feather_int8_mm_status": (_c_int, [_ptr]),
    "feather_conv3x3_launch": (
        _c_int,
        [_ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _ptr],
    ),
    "feather_conv3x3_status": (_c_int, [_ptr]),
    "feather_selftest_wait_runs_out": (_c_int, [ctypes.c_longlong, _ptr, _ptr, _ptr]),
}

_lib = None


def load() -> ctypes.CDLL:
    """The loaded library with prototypes applied to every symbol it exports."""
    global _lib
    if _lib is None:
        if not _PATH.exists():
            raise RuntimeError(f"{_PATH.name} is not built: run `python -m feather_ops_b200._build` (needs nvcc, no GPU)")
        lib = ctypes.CDLL(str(_PATH))
        for name, (restype, argtypes) in PROTOTYPES.items():
            fn = getattr(lib, name, None)
            if fn is not None:
                fn.restype = restype
                fn.argtypes = argtypes
        _lib = lib
    return _lib


def read_status(symbol: str) -> tuple[int, int]:
    """`(site, block)` from one of the `feather_*_status` diagnostics. `(0, 0)` means every wait completed."""
    out = (ctypes.c_uint32 * 2)()
    rc = getattr(load(), symbol)(out)
    if rc != 0:
        raise RuntimeError(f"{symbol} failed (a CUDA error is pending on this device)")
    if symbol == "feather_scaled_mm_status" and out[0] != 0:
        # a split-K launch that gave up may have left its tickets non-zero: never reuse them
        from . import scaled_mm

        scaled_mm.reset_split_k_state()
    return int(out[0]), int(out[1])
