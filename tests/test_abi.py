"""The C-ABI library loads without a GPU and exports every function `include/*.h` declares."""

import ctypes
import pathlib
import re

from feather_ops_b200 import _lib

ROOT = pathlib.Path(__file__).resolve().parents[1]


def declared_functions() -> list[str]:
    names = []
    for header in sorted((ROOT / "include").glob("*.h")):
        text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
        names += re.findall(r"^\s*(?:bool|int|int64_t|void)\s+(\w+)\s*\(", text, flags=re.M)
    return names


def test_header_declares_the_reference_launchers():
    names = declared_functions()
    for required in ("launch_scaled_mm", "launch_int8_scaled_mm", "launch_convrot_quantize", "feather_conv3x3_launch"):
        assert required in names


def test_library_exports_every_declared_symbol(lib):
    for name in declared_functions():
        assert isinstance(getattr(lib, name), ctypes._CFuncPtr), name


def test_ctypes_prototypes_cover_the_header():
    assert set(declared_functions()) <= set(_lib.PROTOTYPES)


def test_int8_plain_tile_width_fills_the_last_round(lib):
    # rounds of 74 CTA pairs x (width + 24): 4096 x 3072 in 256-wide tiles are 192 tiles = three rounds, of which the last is 60 % full
    def width(m, n, pairs, transposed=False):
        return lib.feather_int8_plain_tile_width(m, n, pairs, transposed)

    assert width(4096, 3072, 74) == 240      # 208 tiles, three rounds of shorter tiles
    assert width(8192, 8192, 74) == 256      # 13.8 rounds: nothing to gain
    assert width(1024, 12288, 74) == 224     # 220 tiles = 2.97 rounds instead of 192 = 2.6
    assert width(2048, 3072, 74) == 176      # 144 tiles = two rounds instead of 96 = 1.3
    assert width(512, 3072, 74) == 128       # one round either way: the narrowest tile, on 48 pairs instead of 24
    assert width(65536, 12288, 74) == 256
    for m, n in ((1, 16), (300, 260), (4096, 12288), (100000, 4112)):
        assert 128 <= width(m, n, 74) <= 256 and width(m, n, 74) % 16 == 0
        # backward: a CTA's half of the columns is the x coordinate of its weight boxes (16-byte rule), and 80 or 112 columns per CTA are slow
        assert width(m, n, 74, True) in (128, 192, 256)
    assert width(2048, 3072, 74, True) == 192 and width(512, 3072, 74, True) == 128 and width(4096, 3072, 74, True) == 256
    assert width(4128, 3840, 74, True) == 256 and width(4096, 4096, 74, True) == 256   # five rounds of 192 columns do not beat four of 256
    assert width(16, 5376, 74, True) == 256   # a few rows: bound by streaming the weight, and a narrower tile's boxes fetch as much
    assert width(4096, 3072, 0) == 256


def test_scaled_mm_pair_tile_width_only_narrows_to_fill_a_round(lib):
    # rounds of 74 CTA pairs x (width + 304): a tile fetches its 256 activation rows whatever its width
    width = lib.feather_scaled_mm_pair_tile_width
    assert width(4096, 12288, 74) == 256     # the metric shape: 768 tiles = 10.4 rounds, nothing narrower pays
    assert width(4096, 3072, 74) == 256
    assert width(65536, 12288, 74) == 256
    assert width(1024, 12288, 74) == 224     # 220 tiles = 2.97 rounds instead of 192 = 2.6
    assert width(2048, 3072, 74) == 192      # 128 tiles = 1.7 rounds instead of 96 = 1.3
    assert width(512, 3072, 74) == 128       # one round either way
    for m, n in ((129, 16), (300, 272), (4096, 9216), (100000, 4112)):
        w = width(m, n, 74)
        assert 128 <= w <= 256 and w % 32 == 0
    assert width(4096, 3072, 0) == 256


def test_launchers_reject_bad_arguments_without_touching_a_device(lib):
    # unknown tile tuple, bad divisibility: refused before any CUDA call
    assert not lib.launch_scaled_mm(None, None, None, None, None, 16, 32, 32, 0, 0, True, True, True, 9, 9, 9, 9, 9, False, None)
    assert not lib.launch_scaled_mm(None, None, None, None, None, 16, 40, 32, 0, 0, True, True, True, 1, 8, 4, 8, 2, False, None)
    assert not lib.launch_int8_scaled_mm(None, None, None, None, None, None, 16, 32, 32, 8, 1, False, 7, 7, 7, 7, 7, 1, None)
    assert not lib.launch_int8_scaled_mm_plain(None, None, None, None, None, None, 16, 32, 40, False, 1, None)   # K % 16
    assert not lib.launch_int8_scaled_mm_plain(None, None, None, None, None, None, 16, 36, 64, True, 1, None)    # backward: N % 16
    assert lib.launch_int8_scaled_mm_plain(None, None, None, None, None, None, 0, 32, 64, False, 1, None)        # no rows: nothing to launch
    assert not lib.launch_convrot_quantize(None, None, None, None, 4, 300, 0, True, None)
    assert lib.feather_conv3x3_launch(None, None, None, None, 1, 8, 8, 8, 8, 0, 9, 9, 9, 9, 1, 1, 0, None) == 1
    assert lib.feather_conv3x3_launch(None, None, None, None, 1, 8, 8, 8, 9, 0, 4, 4, 2, 2, 2, 1, 0, None) == 1  # two rows, odd W
    # empty problems are accepted and launch nothing
    assert lib.launch_scaled_mm(None, None, None, None, None, 0, 32, 32, 0, 0, True, True, True, 1, 8, 4, 8, 2, False, None)
    assert lib.launch_convrot_quantize(None, None, None, None, 0, 256, 0, True, None)
