"""Generates `reference_vectors.pt` by running the reference's own Python implementations on CPU.

    python tests/golden/make_golden.py /path/to/reference/checkout

The reference package cannot be imported whole without its compiled extension, so its pure-Python modules
are imported under a stub parent package. Inputs are seeded and stored beside the outputs, so the fixture
is self-contained: the tests never need the reference checkout.
"""

import importlib
import os
import pathlib
import sys
import types

import torch


def load_reference(root: str):
    pkg = types.ModuleType("feather_ops")
    pkg.__path__ = [str(pathlib.Path(root) / "feather_ops")]
    sys.modules["feather_ops"] = pkg
    names = ("naive", "scaled_mm", "int8_convrot", "conv2d", "tiles")
    return {name: importlib.import_module(f"feather_ops.{name}") for name in names}


ACTIVATION_SHAPES = [(1, 256), (4, 512), (512, 1024), (1024, 2048), (300, 4096), (16, 8192), (8, 16384)]
ACTIVATION_ROWS = 16


def reference_activation(m: int, k: int, dtype: torch.dtype) -> torch.Tensor:
    """The first ACTIVATION_ROWS rows of the reference test's activation for one shape (seed 0, N(0, 2))."""
    torch.manual_seed(0)
    return (torch.randn(m, k, dtype=torch.float32) * 2.0)[:ACTIVATION_ROWS].to(dtype).contiguous()


def checksum(x: torch.Tensor) -> int:
    """Order-dependent 63-bit checksum of a 16-bit tensor's bit patterns."""
    bits = x.contiguous().view(torch.int16).to(torch.int64) & 0xFFFF
    weights = torch.arange(1, bits.numel() + 1, dtype=torch.int64) % 1000003
    return int((bits.reshape(-1) * weights).sum().item() & 0x7FFFFFFFFFFFFFFF)


def main() -> None:
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("FEATHER_OPS_REFERENCE")
    if not root:
        raise SystemExit("usage: make_golden.py /path/to/feather-ops (or set FEATHER_OPS_REFERENCE)")
    ref = load_reference(root)
    gen = torch.Generator().manual_seed(20240607)
    out: dict = {}

    # scaled_mm: the naive path on the reference tests' distribution, every dtype combination
    cases = []
    for a_dtype in (torch.float16, torch.bfloat16):
        for b_dtype, out_dtype in ((torch.float8_e5m2, torch.float16), (torch.float8_e5m2, torch.bfloat16), (torch.float8_e4m3fn, torch.bfloat16)):
            m, n, k = 19, 32, 144
            a = torch.randn((m, k), generator=gen).to(a_dtype)
            b = torch.randn((k, n), generator=gen).to(b_dtype)
            scale = torch.tensor(2.34, dtype=torch.float32)
            bias = torch.randn((n,), generator=gen).to(out_dtype)
            packed = ref["scaled_mm"].prepack_b_for_scaled_mm(b)
            y = ref["naive"].scaled_mm_naive(a, packed, scale, bias, out_dtype, b_prepacked=True)
            cases.append({"a": a, "b": b.view(torch.uint8), "b_dtype": str(b_dtype), "b_prepacked": packed.view(torch.uint8), "scale": scale, "bias": bias, "y": y})
    out["scaled_mm"] = cases
    out["scaled_mm_heuristic"] = {shape: ref["scaled_mm"].select_scaled_mm_config(*shape) for shape in ((1, 128, 128), (4096, 12288, 3072), (4096, 3072, 12288))}

    # int8 ConvRot: Hadamard, weight recipe, prepack, and the activation recipe (matmul rotation + row-wise int8)
    i8 = ref["int8_convrot"]
    h = i8.build_hadamard(256)
    out["hadamard_row5"] = h[5].clone()
    out["hadamard_checksum"] = (h * torch.arange(256 * 256, dtype=torch.float32).reshape(256, 256)).sum().item()
    w = (torch.randn((24, 512), generator=gen) * 0.02).to(torch.bfloat16)
    wq, ws = i8.quantize_convrot_weight(w)
    out["weight"] = {"w": w, "q": wq, "scale": ws, "prepacked": i8.prepack_int8_weight(wq)}
    acts = []
    for dtype in (torch.bfloat16, torch.float16):
        x = torch.randn((9, 768), generator=gen)
        x[:, ::97] *= 20
        x = x.to(dtype)
        q, s = i8.quantize_rowwise_int8(i8.rotate(x, i8.build_hadamard(256)))
        acts.append({"x": x, "q_recipe": q, "scale_recipe": s})
    out["activation"] = acts
    # The seven shapes and the input distribution of the reference's own recipe test (tests/test_int8_convrot.py:270-286
    # there: `torch.manual_seed(0); randn(M, K) * 2`), both dtypes, through the reference's rotate + row-wise quantize.
    # Rows are independent, so only the first ACTIVATION_ROWS rows of each shape are kept; the inputs are not stored but
    # re-made from the seed by the tests, which check them against the stored checksum first.
    shaped = []
    for dtype in (torch.bfloat16, torch.float16):
        for m, k in ACTIVATION_SHAPES:
            x = reference_activation(m, k, dtype)
            q, s = i8.quantize_rowwise_int8(i8.rotate(x, i8.build_hadamard(256)))
            shaped.append({"shape": (m, k), "dtype": str(dtype), "x_checksum": checksum(x), "q_recipe": q, "scale_recipe": s})
    out["activation_reference_shapes"] = shaped
    codes = torch.tensor([[-300.0, -127.4, -0.5, 0.5, 1.5, 126.6, 500.0, 0.0]])
    q, s = i8.quantize_rowwise_int8(codes, scale=1.0)
    out["rowwise_stored_scale"] = {"x": codes, "q": q, "scale": s}
    out["int8_supported"] = {shape: i8.convrot_int8_supported(shape) for shape in ((64, 512), (62, 512), (64, 500), (68, 256))}

    # conv: the prepack permutation
    cw = torch.randn((12, 24, 3, 3), generator=gen).to(torch.bfloat16)
    out["conv_prepack"] = {"w": cw, "packed": ref["conv2d"].prepack_conv2d_weight_3x3(cw)}

    # tile vocabulary
    out["tiles"] = {"scaled_mm": list(ref["tiles"].SCALED_MM_TILES), "int8": list(ref["tiles"].INT8_TILES), "conv": list(ref["tiles"].CONV_TILES)}

    target = pathlib.Path(__file__).with_name("reference_vectors.pt")
    torch.save(out, target)
    print(f"wrote {target} ({target.stat().st_size} bytes)")


if __name__ == "__main__":
    main()
