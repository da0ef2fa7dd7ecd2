"""Seeded random shapes through the C ABI against the oracles: ragged rows, widths that are not multiples of any tile,
contraction lengths with tails, every tile width, optional scale and bias. The fixed-shape tests cover the
reference's own cases; this sweep is there to catch index arithmetic that only breaks off the beaten path
(partial row tiles of a CTA pair, a single column tile, a contraction shorter than one pipeline slot)."""

import random

import pytest
import torch

from oracle import conv2d as oc
from oracle import int8_convrot as o8
from oracle import scaled_mm as osm
from tests import _cabi

pytestmark = pytest.mark.gpu

SCALED_MM_TILES = [(1, 8, 4, 8, 2, 0), (1, 4, 2, 4, 2, 1), (1, 2, 4, 1, 2, 1)]  # 256-, 128- and 64-wide
INT8_TILES = [(4, 4, 2, 4, 4), (2, 4, 2, 4, 2), (2, 2, 2, 2, 2)]
CONV_TILES = [(4, 4, 2, 2, 2), (4, 4, 2, 4, 1), (4, 4, 2, 2, 1), (2, 2, 2, 2, 1)]


def _scaled_mm_shapes():
    rng = random.Random(1234)
    shapes = []
    for _ in range(14):
        m = rng.choice([rng.randint(1, 40), rng.randint(100, 300), rng.randint(300, 1200)])
        n = 16 * rng.randint(1, 60)
        k = 16 * rng.randint(1, 50)
        shapes.append((m, n, k))
    return shapes


@pytest.mark.parametrize("shape", _scaled_mm_shapes())
def test_scaled_mm_random_shapes(cuda_device, shape):
    from feather_ops_b200.tiles import SCALED_MM_TILES as TABLE

    m, n, k = shape
    rng = random.Random(m * 7919 + n * 31 + k)
    a_dtype = rng.choice([torch.float16, torch.bfloat16])
    b_dtype = rng.choice([torch.float8_e5m2, torch.float8_e4m3fn])
    out_dtype = rng.choice([torch.float16, torch.bfloat16])
    a, packed, scale, bias = osm.make_inputs(m, n, k, a_dtype, b_dtype, out_dtype, seed=m + n + k)
    if rng.random() < 0.3:
        scale = None
    if rng.random() < 0.3:
        bias = None
    ref = osm.scaled_mm_f32(a, packed, scale, bias, out_dtype, b_prepacked=True).float()
    dev = [None if t is None else t.to(cuda_device) for t in (a, packed, scale, bias)]
    for tile in SCALED_MM_TILES:
        assert tile in TABLE
        out = _cabi.scaled_mm(*dev, out_dtype, tile)
        _cabi.assert_clean("feather_scaled_mm_status")
        rel = ((out.float().cpu() - ref).norm() / ref.norm().clamp(min=1e-6)).item()
        assert rel <= 1e-3, (shape, tile, rel)


def _int8_shapes():
    rng = random.Random(99)
    return [(rng.choice([rng.randint(1, 130), rng.randint(130, 700)]), 16 * rng.randint(1, 40), 16 * rng.randint(1, 40)) for _ in range(12)]


@pytest.mark.parametrize("transposed", [False, True])
@pytest.mark.parametrize("shape", _int8_shapes())
def test_int8_random_shapes(cuda_device, shape, transposed):
    from feather_ops_b200.tiles import INT8_TILES as TABLE

    m, n, k = shape
    gen = torch.Generator().manual_seed(m * 131 + n + k)
    w = torch.randint(-127, 128, (n, k), generator=gen, dtype=torch.int8)
    kc, n_out = (n, k) if transposed else (k, n)
    a = torch.randint(-127, 128, (m, kc), generator=gen, dtype=torch.int8)
    a_scale = torch.rand(m, generator=gen) * 0.01 + 0.001
    w_scale = None if transposed else torch.rand(n, generator=gen) * 0.01 + 0.001
    bias = None if transposed or m % 2 else torch.randn(n, generator=gen).to(torch.bfloat16)
    ref = o8.int8_scaled_mm(a, w, a_scale, w_scale, bias, torch.bfloat16, transposed).double()
    dev = lambda t: None if t is None else t.to(cuda_device)  # noqa: E731
    args = (dev(a), dev(o8.prepack_int8_weight(w)), dev(a_scale), dev(w_scale), dev(bias))
    for tile in INT8_TILES:
        assert tile in TABLE
        out = _cabi.int8_scaled_mm(*args, torch.bfloat16, transposed, n_out, tile)
        _cabi.assert_clean("feather_int8_mm_status")
        err = ((out.double().cpu() - ref).abs() / ref.abs().clamp(min=1e-3)).max().item()
        assert err < 0.02, (shape, transposed, tile, err)


def _conv_shapes():
    rng = random.Random(7)
    shapes = []
    for _ in range(10):
        shapes.append((rng.randint(1, 3), 8 * rng.randint(1, 20), rng.choice([8, 24, 64, 128, 136, 200, 256, 320]), rng.randint(1, 40), rng.randint(1, 300)))
    return shapes


@pytest.mark.parametrize("shape", _conv_shapes())
def test_conv_random_shapes(cuda_device, shape):
    from feather_ops_b200.tiles import CONV_TILES as TABLE

    b, c_in, c_out, h, w = shape
    dtype = torch.bfloat16 if (h + w) % 2 else torch.float16
    x, weight, bias = oc.make_inputs(b, c_in, c_out, h, w, dtype, seed=c_in + w, with_bias=bool(h % 3))
    ref = oc.conv3x3_fp64(x, weight, bias)
    packed = oc.prepack_conv2d_weight_3x3(weight).to(cuda_device)
    tol = 4e-3 if dtype == torch.bfloat16 else 6e-4
    first = None
    for tile in CONV_TILES:
        assert tile in TABLE
        if tile[4] == 2 and w % 2:
            continue
        y = _cabi.conv3x3(x.to(cuda_device), packed, None if bias is None else bias.to(cuda_device), tile)
        _cabi.assert_clean("feather_conv3x3_status")
        rel = ((y.double().cpu() - ref).norm() / ref.norm().clamp(min=1e-12)).item()
        assert rel < tol, (shape, tile, rel)
        first = y if first is None else first
        assert torch.equal(y, first), (shape, tile)  # every tile accumulates in the same order
