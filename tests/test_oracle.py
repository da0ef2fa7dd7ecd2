"""The CPU oracle against the committed golden vectors (outputs of the reference's own Python) and, when
the reference checkout is present, against the reference functions directly."""

import importlib
import os
import pathlib
import sys
import types

import pytest
import torch

from oracle import conv2d as oc
from oracle import int8_convrot as o8
from oracle import scaled_mm as osm

# a checkout of woct0rdho/feather-ops, when one is at hand: the tests that import it skip otherwise
# FEATHER_OPS_REFERENCE, or a directory named `reference` beside this repository
REFERENCE = pathlib.Path(os.environ["FEATHER_OPS_REFERENCE"]) if os.environ.get("FEATHER_OPS_REFERENCE") else pathlib.Path(__file__).resolve().parents[2] / "reference"
if not (REFERENCE / "feather_ops" / "naive.py").exists():
    REFERENCE = None


def _fp8(raw: torch.Tensor, name: str) -> torch.Tensor:
    return raw.view(torch.float8_e5m2 if name.endswith("e5m2") else torch.float8_e4m3fn)


def test_scaled_mm_naive_matches_golden(golden):
    for case in golden["scaled_mm"]:
        b = _fp8(case["b"], case["b_dtype"])
        packed = osm.prepack_b(b)
        assert torch.equal(packed.view(torch.uint8), case["b_prepacked"])
        assert torch.equal(osm.unpack_b(packed, b.shape[0]).view(torch.uint8), case["b"])
        y = osm.scaled_mm_naive(case["a"], packed, case["scale"], case["bias"], case["y"].dtype, b_prepacked=True)
        assert torch.equal(y, case["y"])  # same torch ops on the same inputs: bit identical


def test_scaled_mm_f32_is_within_the_reference_tolerance_of_naive(golden):
    # tests/test_scaled_mm_hip.py:8-12 of the reference: Frobenius rel <= 0.01, max-abs <= 2 (fp16) / 16 (bf16)
    for case in golden["scaled_mm"]:
        b = _fp8(case["b_prepacked"], case["b_dtype"]).reshape(-1, case["b"].shape[1], 16)
        y = osm.scaled_mm_f32(case["a"], b, case["scale"], case["bias"], case["y"].dtype, b_prepacked=True)
        diff = (y.float() - case["y"].float()).abs()
        assert (diff.norm() / case["y"].float().norm()).item() <= 2e-3
        assert diff.max().item() <= (2.0 if case["y"].dtype == torch.float16 else 16.0)


def test_naive_overflows_on_the_benchmark_distribution_and_f32_does_not():
    a, packed, scale, _ = osm.make_inputs(64, 128, 512, torch.float16, torch.float8_e5m2, torch.float16, weight_std=0.02, with_bias=False)
    naive = osm.scaled_mm_naive(a, packed, scale, None, torch.float16, b_prepacked=True)
    f32 = osm.scaled_mm_f32(a, packed, scale, None, torch.float16, b_prepacked=True)
    assert not torch.isfinite(naive).all()
    assert torch.isfinite(f32).all()


def test_hadamard_matches_golden_and_is_orthogonal(golden):
    h = o8.build_hadamard(256)
    assert torch.equal(h[5], golden["hadamard_row5"])
    weights = torch.arange(256 * 256, dtype=torch.float32).reshape(256, 256)
    assert (h * weights).sum().item() == golden["hadamard_checksum"]
    assert torch.equal(h, h.T)
    assert torch.allclose(h @ h, torch.eye(256), atol=1e-6)
    with pytest.raises(ValueError):
        o8.build_hadamard(128)


def test_weight_recipe_and_prepack_match_golden(golden):
    g = golden["weight"]
    q, scale = o8.quantize_convrot_weight(g["w"])
    assert torch.equal(q, g["q"]) and torch.equal(scale, g["scale"])
    packed = o8.prepack_int8_weight(q)
    assert torch.equal(packed, g["prepacked"])
    assert torch.equal(o8.unpack_int8_weight(packed), q)


def test_rowwise_quantizer_clamps_like_the_reference(golden):
    g = golden["rowwise_stored_scale"]
    q, scale = o8.quantize_rowwise_int8(g["x"], scale=1.0)
    assert torch.equal(q, g["q"]) and torch.equal(scale, g["scale"])
    assert q.min().item() == -127 and q.max().item() == 127


def test_radix4_rotation_equals_the_hadamard_matrix_on_integers():
    gen = torch.Generator().manual_seed(3)
    x = torch.randint(-8, 9, (7, 256), generator=gen).float()
    h = o8.build_hadamard(256) * 16.0
    assert torch.equal(o8.hadamard256_radix4(x), x @ h.T)


def _within_recipe_bounds(q, scale, q_recipe, scale_recipe):
    # tests/test_int8_convrot.py:280-286 of the reference: code mismatch rate < 1e-3 (differences of one code), scale
    # rel < 1e-2, dequantized rel < 1e-3. The recipe rotates with a matmul in the input dtype, the kernel in fp32.
    assert (q != q_recipe).float().mean().item() < 1e-3
    assert (q.int() - q_recipe.int()).abs().max().item() <= 1
    assert ((scale - scale_recipe).abs() / scale_recipe).max().item() < 1e-2
    deq = q.float() * scale[:, None]
    ref = q_recipe.float() * scale_recipe[:, None]
    assert ((deq - ref).norm() / ref.norm()).item() < 1e-3


def test_kernel_restatement_stays_within_the_reference_bounds_of_the_recipe(golden):
    for case in golden["activation"]:
        _within_recipe_bounds(*o8.convrot_quantize(case["x"], True), case["q_recipe"], case["scale_recipe"])


def test_kernel_restatement_on_the_reference_recipe_shapes(golden):
    # the reference test's seven shapes and distribution, both dtypes; the inputs are re-made from the seed
    from tests.golden import make_golden as mg

    assert [tuple(c["shape"]) for c in golden["activation_reference_shapes"][:7]] == mg.ACTIVATION_SHAPES
    for case in golden["activation_reference_shapes"]:
        dtype = torch.bfloat16 if "bfloat16" in case["dtype"] else torch.float16
        x = mg.reference_activation(*case["shape"], dtype)
        assert mg.checksum(x) == case["x_checksum"]
        _within_recipe_bounds(*o8.convrot_quantize(x, True), case["q_recipe"], case["scale_recipe"])
        # the oracle's own restatement of the recipe equals the reference's output bit for bit
        q_port, s_port = o8.quantize_rowwise_int8(o8.rotate(x, o8.build_hadamard(256)))
        assert torch.equal(q_port, case["q_recipe"]) and torch.equal(s_port, case["scale_recipe"])


def test_quantizer_without_rotation_folds_the_column_scale():
    x = o8.make_activation(5, 512, torch.bfloat16, seed=11)
    col = torch.rand(512) + 0.5
    q, scale = o8.convrot_quantize(x, False, col)
    folded = (x.float() * col).to(torch.bfloat16)
    q_ref, scale_ref = o8.quantize_rowwise_int8(folded)
    assert torch.equal(scale, scale_ref)
    assert (q.int() - q_ref.int()).abs().max().item() <= 1  # `v * (1 / d)` against `v / d`
    with pytest.raises(ValueError, match="multiple of the ConvRot group size"):
        o8.convrot_quantize(torch.zeros(2, 300, dtype=torch.bfloat16))


def test_conv_prepack_matches_golden(golden):
    g = golden["conv_prepack"]
    packed = oc.prepack_conv2d_weight_3x3(g["w"])
    assert torch.equal(packed, g["packed"])
    assert packed.shape == (2 * 18, 12, 8)
    # channels 24..31 of the second group are padding
    assert packed[18 + 1 :: 2][:9].abs().sum().item() == 0


def test_empty_inputs():
    q, scale = o8.convrot_quantize(torch.zeros(0, 256, dtype=torch.bfloat16))
    assert q.shape == (0, 256) and scale.shape == (0,)
    a, packed, s, b = osm.make_inputs(0, 32, 64, torch.bfloat16, torch.float8_e5m2, torch.bfloat16)
    assert osm.scaled_mm_f32(a, packed, s, b, torch.bfloat16, b_prepacked=True).shape == (0, 32)


@pytest.mark.skipif(REFERENCE is None, reason="set FEATHER_OPS_REFERENCE to a checkout of the reference to run this")
def test_oracle_equals_the_reference_python_directly():
    pkg = types.ModuleType("feather_ops")
    pkg.__path__ = [str(REFERENCE / "feather_ops")]
    saved = sys.modules.get("feather_ops")
    sys.modules["feather_ops"] = pkg
    try:
        ref_i8 = importlib.import_module("feather_ops.int8_convrot")
        ref_conv = importlib.import_module("feather_ops.conv2d")
        ref_naive = importlib.import_module("feather_ops.naive")
        gen = torch.Generator().manual_seed(5)
        w = torch.randn((32, 768), generator=gen).to(torch.float16)
        assert all(torch.equal(x, y) for x, y in zip(ref_i8.quantize_convrot_weight(w), o8.quantize_convrot_weight(w)))
        cw = torch.randn((16, 40, 3, 3), generator=gen).to(torch.float16)
        assert torch.equal(ref_conv.prepack_conv2d_weight_3x3(cw), oc.prepack_conv2d_weight_3x3(cw))
        a, packed, scale, bias = osm.make_inputs(21, 64, 400, torch.bfloat16, torch.float8_e4m3fn, torch.bfloat16, seed=9)
        assert torch.equal(
            ref_naive.scaled_mm_naive(a, packed, scale, bias, torch.bfloat16, b_prepacked=True),
            osm.scaled_mm_naive(a, packed, scale, bias, torch.bfloat16, b_prepacked=True),
        )
    finally:
        for name in [n for n in sys.modules if n == "feather_ops" or n.startswith("feather_ops.")]:
            del sys.modules[name]
        if saved is not None:
            sys.modules["feather_ops"] = saved
